"""One causal DiT block (and two consecutive chunks through the rolling NVFP4 cache) against the
CPU oracle composition, on a reduced configuration (dim 256, 2 heads, FFN 512, 48 tokens/frame: 144-token cache blocks).

Tolerance: every stage matches its oracle to within a bf16 ulp, but a one-ulp difference ahead of
a quantizer can flip an E2M1 code (a ~6 % change of that element), so block outputs are compared
with a relative Frobenius error <= 3e-2 and <= 1 % of elements outside 8 bf16 ulps + 2^-5 mean|ref|."""
import numpy as np
import pytest
import torch

import longlive_b200 as L
from longlive_b200 import dit, ops
from oracle import dit_oracle as DO
from oracle import nvfp4_oracle as O
from tests import util

pytestmark = pytest.mark.gpu

CFG = dict(dim=256, ffn_dim=512, heads=2, layers=1, text_len=128, text_dim=64, freq_dim=32, grid_h=6, grid_w=8,
           frames_per_chunk=3, window_frames=9, sink_frames=3, in_channels=4)


def trip(qt):
    return qt.values.cpu().numpy(), util.u8(qt.scale_factors), np.float32(qt.amax.item())


def params_of(blk, ffn_dim):
    f = lambda t: t.float().cpu().numpy()
    p = {"ffn_dim": ffn_dim}
    for name in ("q", "k", "v", "o", "cq", "ck", "cv", "co", "ffn0", "ffn2"):
        lin = getattr(blk, name)
        p[name] = trip(lin.q)
        p[name + "_b"] = f(lin.bias)
    for name in ("norm_q", "norm_k", "cnorm_q", "cnorm_k", "norm3_w", "norm3_b"):
        p[name] = f(getattr(blk, name))
    return p


def close(got, ref, rel_tol=3e-2):
    got = got.float().cpu().numpy().reshape(ref.shape)
    rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert rel <= rel_tol, rel
    tol = np.abs(ref) * 2.0 ** -4 + 2.0 ** -5 * np.abs(ref).mean()
    assert (np.abs(got - ref) > tol).mean() < 0.01


def test_block_and_cache_roll_vs_oracle():
    cfg = dit.DiTConfig(**CFG)
    model = dit.CausalDiT(cfg, seed=3)
    blk = model.blocks[0]
    p = params_of(blk, cfg.ffn_dim)
    g = torch.Generator().manual_seed(5)
    S, C, F = cfg.chunk_tokens, cfg.dim, cfg.frames_per_chunk
    ctx = torch.randn(cfg.text_len, C, generator=g).bfloat16()
    ctx_kn, ctx_v = DO.text_kv(ctx.float().numpy(), p, cfg.heads)
    past_k, past_v = [], []
    for chunk in range(4):                       # window of 3 blocks: the 4th chunk evicts the first non-sink block
        x = (torch.randn(S, C, generator=g) * 1.5).bfloat16()
        e = (blk.modulation.cpu() + torch.randn(F, 6, C, generator=g).bfloat16() * 0.3).contiguous()
        cos, sin = dit.rope_tables(cfg, chunk * F, "cuda")
        model.cache.begin_chunk()
        out = model.block_forward(0, x.cuda(), model.x_b, e.cuda(), ctx.cuda(), cos, sin)
        torch.cuda.synchronize()
        ref, nk, nv = DO.block_forward(x.float().numpy(), e.float().numpy(), p, ctx_kn, ctx_v, cos.cpu().numpy(),
                                       sin.cpu().numpy(), past_k, past_v, cfg.heads, cfg.frame_tokens, cfg.chunk_tokens)
        close(out, ref)
        # the cache block written by the kernels dequantizes to (nearly) what the oracle's block holds
        cur = model.cache.current_slot()
        got_k = ops.kv_dequant([model.cache.k[0][cur].values], [model.cache.k[0][cur].scale_factors],
                               [model.cache.k[0][cur].amax], cfg.heads, S, torch.bfloat16, 6, 256)
        ref_k = O.dequantize_kv_cache([nk], cfg.heads, S)
        close(got_k, ref_k, rel_tol=2e-2)
        # oracle-side cache bookkeeping: sink block + the newest (max_blocks - 2) blocks + current
        past_k.append(nk)
        past_v.append(nv)
        if len(past_k) > cfg.max_blocks - 1:
            del past_k[1], past_v[1]
    assert model.cache.order != list(range(cfg.max_blocks))     # the block table was permuted, no slot copies


def test_full_model_chunk_runs_and_fills_cache():
    cfg = dit.DiTConfig(**{**CFG, "layers": 2})
    model = dit.CausalDiT(cfg, seed=1)
    g = torch.Generator().manual_seed(2)
    ctx = model.encode_text(torch.randn(cfg.text_len, cfg.text_dim, generator=g).bfloat16().cuda())
    for chunk in range(2):
        lat = torch.randn(cfg.chunk_tokens, cfg.patch_dim, generator=g).bfloat16().cuda()
        x = model.run_chunk(lat, ctx, chunk)
        assert x.shape == lat.shape and torch.isfinite(x.float()).all()
    assert model.cache.filled == 2
    for layer in range(cfg.layers):
        for slot in model.cache.order[:2]:
            assert float(model.cache.k[layer][slot].amax.item()) > 0 and int(model.cache.k[layer][slot].values.max().item()) > 0


def test_graph_replay_equals_eager():
    """The captured-graph forward (one graph per state of the KV block table) reproduces the eager
    launch sequence bit for bit over the fill phase and two full periods of the rolling table."""
    cfg = dit.DiTConfig(**{**CFG, "layers": 2})
    eager = dit.CausalDiT(cfg, seed=3)
    graphed = dit.CausalDiT(cfg, seed=3, use_graphs=True)
    g = torch.Generator().manual_seed(5)
    raw = torch.randn(cfg.text_len, cfg.text_dim, generator=g).bfloat16().cuda()
    ctx_e, ctx_g = eager.encode_text(raw), graphed.encode_text(raw)
    period = cfg.max_blocks - cfg.sink_frames // cfg.frames_per_chunk
    for chunk in range(cfg.max_blocks + 2 * period):
        lat = torch.randn(cfg.chunk_tokens, cfg.patch_dim, generator=g).bfloat16().cuda()
        a = eager.run_chunk(lat, ctx_e, chunk)
        b = graphed.run_chunk(lat, ctx_g, chunk)
        assert torch.equal(a, b), chunk
    assert len(graphed._graphs) == 5 * period        # per table state: one graph per timestep of a chunk
    assert eager.cache.order == graphed.cache.order
    for layer in range(cfg.layers):
        for slot in range(cfg.max_blocks):
            for side in ("k", "v"):
                te, tg = getattr(eager.cache, side)[layer][slot], getattr(graphed.cache, side)[layer][slot]
                assert torch.equal(te.values, tg.values) and torch.equal(te.amax, tg.amax)
                assert torch.equal(te.scale_factors.view(torch.uint8), tg.scale_factors.view(torch.uint8))


def test_scene_cut_clean_recache_and_pinned_sink():
    """A scene cut with clean re-cache: the re-cache forward sees only the chunk itself, so the cache
    block it writes equals the block a fresh model writes for the same clean latents at the same
    position; afterwards the chunk is pinned and replaces the sink, in eager and graph mode alike."""
    cfg = dit.DiTConfig(**{**CFG, "layers": 2})
    eager = dit.CausalDiT(cfg, seed=3)
    graphed = dit.CausalDiT(cfg, seed=3, use_graphs=True)
    g = torch.Generator().manual_seed(9)
    raw = torch.randn(cfg.text_len, cfg.text_dim, generator=g).bfloat16().cuda()
    ctx_e, ctx_g = eager.encode_text(raw), graphed.encode_text(raw)
    cut = cfg.max_blocks + 1
    for chunk in range(cut + cfg.max_blocks + 3):
        lat = torch.randn(cfg.chunk_tokens, cfg.patch_dim, generator=g).bfloat16().cuda()
        a = eager.run_chunk(lat, ctx_e, chunk, scene_cut=chunk == cut)
        b = graphed.run_chunk(lat, ctx_g, chunk, scene_cut=chunk == cut)
        assert torch.equal(a, b), chunk
        assert eager.cache.order == graphed.cache.order and eager.cache.filled == graphed.cache.filled
        if chunk == cut:
            assert eager.cache.filled == 1 and eager.cache.pinned == eager.cache.current_slot()
            pinned, clean = eager.cache.pinned, a
            # a fresh model that caches the same clean latents at the same frame position writes the same block
            fresh = dit.CausalDiT(cfg, seed=3)
            fresh.cache.begin_chunk()
            fresh.forward(clean, torch.zeros(cfg.frames_per_chunk, device="cuda"), fresh.encode_text(raw), chunk * cfg.frames_per_chunk)
            for layer in range(cfg.layers):
                for side in ("k", "v"):
                    te, tf = getattr(eager.cache, side)[layer][pinned], getattr(fresh.cache, side)[layer][fresh.cache.current_slot()]
                    assert torch.equal(te.values, tf.values) and torch.equal(te.amax, tf.amax)
    assert eager.cache.pinned == pinned and eager.cache.order[0] == pinned          # the pinned chunk became the sink
    for layer in range(cfg.layers):
        for slot in range(cfg.max_blocks):
            te, tg = eager.cache.k[layer][slot], graphed.cache.k[layer][slot]
            assert torch.equal(te.values, tg.values) and torch.equal(te.amax, tg.amax)


def test_checkpoint_round_trip(tmp_path):
    """A model saved in the reference's NVFP4 generator format and loaded into a model with other
    weights reproduces the first model's forward bit for bit; bf16 master weights are quantized on load."""
    from longlive_b200 import checkpoint as ck
    cfg = dit.DiTConfig(**{**CFG, "layers": 2})
    a, b = dit.CausalDiT(cfg, seed=5), dit.CausalDiT(cfg, seed=6)
    path = str(tmp_path / "gen_nvfp4.pt")
    ck.save_checkpoint(a, path)
    saved = torch.load(path, map_location="cpu", weights_only=False)
    assert saved["checkpoint_format"] == "longlive_generator_nvfp4" and saved["checkpoint_version"] == 1
    assert sorted(saved["generator"]) == sorted(ck.expected_keys(cfg)) and ck.is_nvfp4_state_dict(saved["generator"])
    assert ck.load_checkpoint(b, path) == []
    g = torch.Generator().manual_seed(2)
    raw = torch.randn(cfg.text_len, cfg.text_dim, generator=g).bfloat16().cuda()
    lat = torch.randn(cfg.chunk_tokens, cfg.patch_dim, generator=g).bfloat16().cuda()
    outs = [m.run_chunk(lat, m.encode_text(raw), 0) for m in (a, b)]
    assert torch.equal(outs[0], outs[1])
    # a bf16 checkpoint of one Linear: quantized on load with the stated rule
    sd = dict(saved["generator"])
    w = (torch.randn(cfg.dim, cfg.dim, generator=g) * 0.02).bfloat16()
    for s in ("values", "scale_factors", "amax", "metadata"):
        del sd[f"model.blocks.0.self_attn.q.quantized_weight_{s}"]
    sd["model.blocks.0.self_attn.q.weight"] = w
    assert ck.load_state_dict_into(b, sd) == []
    ref = L.quantize_to_fp4(w.cuda(), L.QuantizationConfig(scale_rule="mse"))
    assert torch.equal(b.blocks[0].q.q.values, ref.values) and torch.equal(b.blocks[0].q.q.amax, ref.amax)
    with pytest.raises(KeyError):
        ck.load_state_dict_into(b, {k: v for k, v in sd.items() if not k.endswith("norm3.bias")})


def test_single_pass_ffn_requant_stays_close_to_two_pass():
    """With ``ffn_requant='single_pass'`` the FFN GEMM's epilogue quantizes the hidden with the previous forward's
    amax.  The first forward calibrates (two-pass form, bit-identical); later chunks differ from the two-pass model
    only through the scale of that one tensor: relative Frobenius difference of a chunk's result below 2 %."""
    cfg = dit.DiTConfig(**{**CFG, "layers": 2})
    a = dit.CausalDiT(cfg, seed=3)
    b = dit.CausalDiT(cfg, seed=3, ffn_requant="single_pass")
    g = torch.Generator().manual_seed(5)
    raw = torch.randn(cfg.text_len, cfg.text_dim, generator=g).bfloat16().cuda()
    ctx_a, ctx_b = a.encode_text(raw), b.encode_text(raw)
    lat = torch.randn(cfg.chunk_tokens, cfg.patch_dim, generator=g).bfloat16().cuda()
    t = torch.full((cfg.frames_per_chunk,), 700.0, device="cuda")
    a.cache.begin_chunk()
    b.cache.begin_chunk()
    assert torch.equal(a.forward(lat, t, ctx_a, 0), b.forward(lat, t, ctx_b, 0))       # calibration forward
    assert b._ffn_calibrated and float(b.ffn_amax_use.min().item()) > 0
    for chunk in range(1, 4):
        lat = torch.randn(cfg.chunk_tokens, cfg.patch_dim, generator=g).bfloat16().cuda()
        ya, yb = a.run_chunk(lat, ctx_a, chunk).float(), b.run_chunk(lat, ctx_b, chunk).float()
        assert torch.isfinite(yb).all()
        assert float((ya - yb).norm() / ya.norm()) < 2e-2
    torch.cuda.synchronize()
    ops.check_status()


def test_block_matches_the_reference_block_fixture(golden):
    """The CUDA block against the REFERENCE's own block (tests/golden/dit_block.npz: the reference's
    CausalWanAttentionBlock run on CPU with its PyTorch NVFP4 backends for four consecutive chunks, the fourth rolling
    the cache).  Same tolerance as against the oracle composition; the reference's CPU path dequantizes cache blocks
    with its PyTorch rounding, the CUDA path with its fused kernel's, which can differ in the last bf16 bit of a
    cached value."""
    g = golden("dit_block.npz")
    dim, ffn, heads, text_len, gh, gw, frames, window_frames, sink_frames = (int(v) for v in g["cfg"])
    cfg = dit.DiTConfig(dim=dim, ffn_dim=ffn, heads=heads, layers=1, text_len=text_len, text_dim=64, freq_dim=32, grid_h=gh, grid_w=gw,
                        frames_per_chunk=frames, window_frames=window_frames, sink_frames=sink_frames, in_channels=4)
    model = dit.CausalDiT(cfg, seed=0)
    blk = model.blocks[0]
    tb = lambda name: util.bf16_np_to_torch(g[name])
    for attr in ("q", "k", "v", "o", "cq", "ck", "cv", "co", "ffn0", "ffn2"):
        lin = getattr(blk, attr)
        lin.q = L.quantize_to_fp4(tb(f"w_{attr}"), L.QuantizationConfig(scale_rule="mse"))
        lin.bias = tb(f"b_{attr}")
    for attr in ("norm_q", "norm_k", "cnorm_q", "cnorm_k", "norm3_w", "norm3_b"):
        setattr(blk, attr, tb(attr))
    blk.fuse_qkv()
    ctx = tb("context")
    mod = tb("modulation")                                     # [1, 6, C]
    for chunk in range(cfg.max_blocks + 1):
        x = tb(f"x{chunk}")
        e = (mod + tb(f"e{chunk}")).contiguous()               # causal_model.py:863, a bf16 add
        cos, sin = dit.rope_tables(cfg, chunk * frames, "cuda")
        model.cache.begin_chunk()
        out = model.block_forward(0, x, model.x_b, e, ctx, cos, sin)
        torch.cuda.synchronize()
        close(out, O.bf16_from_bits(g[f"y{chunk}"]))
        # the cache block the kernels wrote against the block the reference wrote: same amax, nearly all codes equal
        cur = model.cache.current_slot()
        for side in ("k", "v"):
            qt = getattr(model.cache, side)[0][cur]
            assert abs(float(qt.amax.item()) - float(g[f"{side}_amax{chunk}"])) <= 2.0 ** -7 * float(g[f"{side}_amax{chunk}"])
            rows = cfg.chunk_tokens * heads
            assert (qt.values.cpu().numpy()[:rows] != g[f"{side}_codes{chunk}"][:rows]).mean() <= 0.03, (chunk, side)
    ops.check_status()
