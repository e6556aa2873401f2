"""Chunk attention parity against the oracle (fp32 softmax(QK^T/sqrt(d))V, bf16 result).

Tolerance: the kernel multiplies bf16-rounded probabilities with V on the tensor cores and uses a
hardware exp2, the oracle works in fp32 throughout; results are compared after the bf16 output
rounding with relative Frobenius error <= 1e-2 and |diff| <= 2^-6 |ref| + 2^-7 mean|ref|."""
import numpy as np
import pytest
import torch

import longlive_b200 as L
from longlive_b200 import _lib, ops
from oracle import nvfp4_oracle as O
from tests import util

pytestmark = pytest.mark.gpu


def check(got, ref):
    got = got.float().cpu().numpy().reshape(ref.shape)
    rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert rel <= 1e-2, rel
    tol = np.abs(ref) * 2.0 ** -6 + 2.0 ** -7 * np.abs(ref).mean()
    frac = (np.abs(got - ref) > tol).mean()
    assert frac < 2e-3, frac


@pytest.mark.parametrize("lq,lk,heads,sigma", [(128, 128, 1, 1.0), (200, 300, 2, 1.0), (256, 1320, 3, 1.0), (130, 77, 2, 3.0), (384, 640, 2, 0.2)])
def test_attention_vs_oracle(lq, lk, heads, sigma):
    g = torch.Generator().manual_seed(lq + lk)
    q = (torch.randn(lq, heads, 128, generator=g) * sigma).bfloat16()
    k = (torch.randn(lk, heads, 128, generator=g) * sigma).bfloat16()
    v = torch.randn(lk, heads, 128, generator=g).bfloat16()
    out = ops.attention_bf16(q.reshape(lq, -1).cuda(), k.reshape(lk, -1).cuda(), v.reshape(lk, -1).cuda(), heads)
    torch.cuda.synchronize()
    assert _lib.lib().llnv_check_status(None) == 0, _lib.lib().llnv_last_error()
    ref = O.attention(q.float().numpy(), k.float().numpy(), v.float().numpy())
    check(out, ref.reshape(lq, -1))


def test_attention_growing_maxima_exercise_lazy_rescale():
    """Keys whose scores keep growing tile after tile force the deferred rescale of the output."""
    lq, lk, heads = 128, 1024, 1
    g = torch.Generator().manual_seed(3)
    q = torch.randn(lq, heads, 128, generator=g).bfloat16()
    k = torch.randn(lk, heads, 128, generator=g)
    ramp = torch.linspace(0.2, 6.0, lk).view(lk, 1, 1)
    k = (k * ramp).bfloat16()
    v = torch.randn(lk, heads, 128, generator=g).bfloat16()
    out = ops.attention_bf16(q.reshape(lq, -1).cuda(), k.reshape(lk, -1).cuda(), v.reshape(lk, -1).cuda(), heads)
    check(out, O.attention(q.float().numpy(), k.float().numpy(), v.float().numpy()).reshape(lq, -1))


def test_attention_matches_reference_fixture(golden):
    g = golden("elementwise_small.npz")
    q = util.bf16_np_to_torch(g["att_q"])[0]
    k = util.bf16_np_to_torch(g["att_k"])[0]
    v = util.bf16_np_to_torch(g["att_v"])[0]
    heads = q.shape[1]
    out = ops.attention_bf16(q.reshape(q.shape[0], -1), k.reshape(k.shape[0], -1), v.reshape(v.shape[0], -1), heads)
    check(out, O.bf16_from_bits(g["att_y"])[0].reshape(q.shape[0], -1))


def test_window_attention_with_nvfp4_cache():
    """The reference's quantized-cache attention: dequantized NVFP4 blocks (un-smoothed keys) followed by
    the current chunk with k_smooth-ed keys (wan_5b/modules/causal_model.py:628-652, 781)."""
    heads, T, blocks, lq = 2, 96, 2, 96
    g = torch.Generator().manual_seed(11)
    cache_k = [torch.randn(T * heads, 128, generator=g).bfloat16() for _ in range(blocks)]
    cache_v = [torch.randn(T * heads, 128, generator=g).bfloat16() for _ in range(blocks)]
    q = torch.randn(lq, heads, 128, generator=g).bfloat16()
    k_new = torch.randn(lq, heads, 128, generator=g).bfloat16()
    v_new = torch.randn(lq, heads, 128, generator=g).bfloat16()
    kq = [L.quantize_to_fp4(t.cuda()) for t in cache_k]
    vq = [L.quantize_to_fp4(t.cuda()) for t in cache_v]
    lk = blocks * T + lq
    win_k = torch.empty(lk, heads * 128, dtype=torch.bfloat16, device="cuda")
    win_v = torch.empty_like(win_k)
    L.dequantize_kv_cache(kq, blocks, heads, T, torch.bfloat16, "cuda", out=win_k[: blocks * T].view(1, blocks * T, heads, 128))
    L.dequantize_kv_cache(vq, blocks, heads, T, torch.bfloat16, "cuda", out=win_v[: blocks * T].view(1, blocks * T, heads, 128))
    # current chunk: smoothed keys and values written straight into the window tail
    ops.rmsnorm_rope(k_new.reshape(lq, -1).cuda(), out=torch.empty(lq, heads * 128, dtype=torch.bfloat16, device="cuda"),
                     out_smooth=win_k[blocks * T:])
    win_v[blocks * T:] = v_new.reshape(lq, -1).cuda()
    out = ops.attention_bf16(q.reshape(lq, -1).cuda(), win_k, win_v, heads)

    def trip(qt):
        return qt.values.cpu().numpy(), util.u8(qt.scale_factors), np.float32(qt.amax.item())
    ref = O.window_attention(q.float().numpy(), k_new.float().numpy(), v_new.float().numpy(),
                             [trip(t) for t in kq], [trip(t) for t in vq], heads, T)
    check(out, ref.reshape(lq, -1))


@pytest.mark.parametrize("splits", [1, 2, 3, 5])
def test_attention_key_splits(splits):
    """Every split count gives the single-pass result (ragged last key tile, ragged query tile,
    keys whose scores grow along the window so the splits end with very different maxima)."""
    lq, lk, heads = 300, 5 * 128 + 37, 2
    g = torch.Generator().manual_seed(17)
    q = torch.randn(lq, heads, 128, generator=g).bfloat16()
    k = (torch.randn(lk, heads, 128, generator=g) * torch.linspace(0.2, 2.5, lk)[:, None, None]).bfloat16()
    v = torch.randn(lk, heads, 128, generator=g).bfloat16()
    out = ops.attention_bf16(q.reshape(lq, -1).cuda(), k.reshape(lk, -1).cuda(), v.reshape(lk, -1).cuda(), heads, key_splits=splits)
    torch.cuda.synchronize()
    assert _lib.lib().llnv_check_status(None) == 0, _lib.lib().llnv_last_error()
    ref = O.attention(q.float().numpy(), k.float().numpy(), v.float().numpy())
    check(out, ref.reshape(lq, -1))


def test_attention_key_split_arguments():
    lib = _lib.lib()
    q = torch.zeros(128, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="more key splits"):
        ops.attention_bf16(q, q, q, 1, key_splits=2)               # one key tile cannot be split
    assert lib.llnv_attention_workspace_bytes(2640, 3, 1) == 0
    assert lib.llnv_attention_workspace_bytes(2640, 3, 4) == 4 * 2640 * 3 * 130 * 4
    # the full-size single-GPU call fills the device by itself; an 8-way head shard of it does not
    assert lib.llnv_attention_key_splits(2640, 13200, 3) > 1
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    if sms == 148:
        # 264 tiles on 148 SMs: a last wave of 116 tiles, which tail balancing cuts; 296 tiles fill two waves exactly
        assert lib.llnv_attention_key_splits(2640, 13200, 24) == ops.SPLIT_TAIL
        assert lib.llnv_attention_key_splits(256 * 37, 13200, 8) == 1
    assert lib.llnv_attention_workspace_bytes(2640, 24, ops.SPLIT_TAIL) == 2 * 2640 * 24 * 130 * 4


def test_attention_tail_balancing():
    """More (query tile, head) items than SMs with a last partial wave: the items of that wave are cut once and merged in
    fp32.  The result agrees with the uncut call to bf16 rounding, its amax is exact, the NVFP4-window kernel cut the same
    way is bit-identical to dequantize-then-attend, and a call that needs the workspace refuses to run without it."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    heads, T, blocks = 8, 1024, 3
    lq = 256 * ((sms + sms // 2) // heads) + 40            # about 1.5 waves of items, ragged last query tile
    g = torch.Generator(device="cuda").manual_seed(77)
    kq, vq = _cache_blocks(blocks, T, heads, g), _cache_blocks(blocks, T, heads, g, scale=2.0)
    q = torch.randn(lq, heads * 128, generator=g, device="cuda").bfloat16()
    k_cur = torch.randn(T, heads * 128, generator=g, device="cuda").bfloat16()
    v_cur = torch.randn(T, heads * 128, generator=g, device="cuda").bfloat16()
    lib = _lib.lib()
    assert lib.llnv_attention_key_splits(lq, (blocks + 1) * T, heads) == ops.SPLIT_TAIL
    am = [torch.full((1,), 9.0, device="cuda") for _ in range(3)]
    whole = _dequant_then_attention(q, kq, vq, T, k_cur, v_cur, heads, key_splits=1, out_amax=am[0])
    ref = _dequant_then_attention(q, kq, vq, T, k_cur, v_cur, heads, key_splits=ops.SPLIT_TAIL, out_amax=am[1])
    out = ops.attention_nvfp4kv(q, kq, vq, T, k_cur, v_cur, heads, key_splits=ops.SPLIT_TAIL, out_amax=am[2])
    torch.cuda.synchronize()
    assert lib.llnv_check_status(None) == 0, lib.llnv_last_error()
    assert torch.equal(out, ref) and torch.equal(am[1], am[2])
    assert float(am[2].item()) == float(out.float().abs().max().item())
    assert not torch.equal(out, whole)                         # the cut items went through the merge
    d = (out.float() - whole.float()).abs()
    assert float(d.max()) <= 2.0 ** -7 * float(whole.float().abs().max()) and float((d > 0).float().mean()) < 0.2
    with pytest.raises(RuntimeError, match="workspace"):
        ops._check(lib.llnv_attention_bf16_ex(q.data_ptr(), lq, q.stride(0), k_cur.data_ptr(), v_cur.data_ptr(), 4 * T, heads * 128, heads * 128, heads,
                                              0.1, out.data_ptr(), out.stride(0), ops.SPLIT_TAIL, None, 0, None, None))


@pytest.mark.parametrize("lq,splits", [(300, 1), (300, 3), (256, 1)])
def test_attention_output_amax(lq, splits):
    """The epilogue's amax is exactly the maximum magnitude of the bf16 output (rows beyond Lq of
    the last query tile, which are computed but never stored, do not count)."""
    lk, heads = 4 * 128 + 5, 2
    g = torch.Generator().manual_seed(23)
    q = torch.randn(lq, heads * 128, generator=g).bfloat16().cuda()
    k = torch.randn(lk, heads * 128, generator=g).bfloat16().cuda()
    v = (torch.randn(lk, heads * 128, generator=g) * 3).bfloat16().cuda()
    amax = torch.full((1,), 123.0, dtype=torch.float32, device="cuda")
    out = ops.attention_bf16(q, k, v, heads, key_splits=splits, out_amax=amax)
    torch.cuda.synchronize()
    assert float(amax.item()) == float(out.float().abs().max().item())


def test_attention_full_window_properties():
    """At the benchmark window (2640 queries, 13200 keys): with V = 1 every output is 1 (the softmax
    weights of a row sum to one), and the key-split schedule agrees with the single pass."""
    lq, lk, heads = 2640, 13200, 3
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(lq, heads * 128, generator=g, device="cuda").bfloat16()
    k = torch.randn(lk, heads * 128, generator=g, device="cuda").bfloat16()
    ones = torch.ones(lk, heads * 128, device="cuda").bfloat16()
    for splits in (1, 4):
        out = ops.attention_bf16(q, k, ones, heads, key_splits=splits)
        assert float((out.float() - 1).abs().max()) <= 2.0 ** -7
    v = torch.randn(lk, heads * 128, generator=g, device="cuda").bfloat16()
    a = ops.attention_bf16(q, k, v, heads, key_splits=1).float()
    b = ops.attention_bf16(q, k, v, heads, key_splits=4).float()
    torch.cuda.synchronize()
    assert _lib.lib().llnv_check_status(None) == 0, _lib.lib().llnv_last_error()
    assert float((a - b).abs().max()) <= 2.0 ** -8 + 2.0 ** -6 * float(a.abs().max())


# ---- NVFP4 K/V decoded inside the attention kernel ----------------------------------------------------

def _cache_blocks(n, T, heads, gen, scale=1.0):
    return [L.quantize_to_fp4((torch.randn(T * heads, 128, generator=gen, device="cuda") * scale * (1 + 0.5 * i)).bfloat16())
            for i in range(n)]


def _dequant_then_attention(q, kq, vq, T, k_cur, v_cur, heads, key_splits=None, out_amax=None):
    """Today's two-step form: llnv_kv_dequant into one bf16 window, then llnv_attention_bf16_ex on it."""
    n = len(kq)
    l_cur = 0 if k_cur is None else k_cur.shape[0]
    lk = n * T + l_cur
    win_k = torch.empty(lk, heads * 128, dtype=torch.bfloat16, device="cuda")
    win_v = torch.empty_like(win_k)
    if n:
        L.dequantize_kv_cache(kq, n, heads, T, torch.bfloat16, "cuda", out=win_k[: n * T].view(1, n * T, heads, 128))
        L.dequantize_kv_cache(vq, n, heads, T, torch.bfloat16, "cuda", out=win_v[: n * T].view(1, n * T, heads, 128))
    if l_cur:
        win_k[n * T:] = k_cur
        win_v[n * T:] = v_cur
    return ops.attention_bf16(q, win_k, win_v, heads, key_splits=key_splits, out_amax=out_amax)


@pytest.mark.parametrize("heads,T,blocks,l_cur,lq,splits", [
    (2, 136, 2, 96, 96, 1),         # cached keys end inside a tile: one tile mixes cache rows and current-chunk rows
    (1, 128, 3, 128, 256, 1),       # tile-aligned segments (the smallest block the kernel accepts)
    (3, 130, 5, 80, 300, 1),        # every tile spans two cache blocks; five blocks cycle through the two table slots
    (2, 200, 2, 0, 130, 1),         # the window is the cache alone, ragged last tile
    (2, 250, 3, 7, 64, 1),          # the current chunk is a few rows inside the last decoded tile
    (2, 264, 4, 264, 264, 3),       # key splits: a split may start in the cache and end in the current chunk
    (4, 330, 4, 330, 330, 2),
    (2, 96, 0, 200, 96, 1),         # no cached block yet (first chunk)
])
def test_nvfp4kv_attention_is_bit_identical_to_dequant_then_attention(heads, T, blocks, l_cur, lq, splits):
    g = torch.Generator(device="cuda").manual_seed(heads * 1000 + T + blocks)
    kq, vq = _cache_blocks(blocks, T, heads, g), _cache_blocks(blocks, T, heads, g, scale=2.0)
    q = torch.randn(lq, heads * 128, generator=g, device="cuda").bfloat16()
    k_cur = torch.randn(l_cur, heads * 128, generator=g, device="cuda").bfloat16() if l_cur else None
    v_cur = torch.randn(l_cur, heads * 128, generator=g, device="cuda").bfloat16() if l_cur else None
    am_a = torch.full((1,), 9.0, device="cuda")
    am_b = torch.full((1,), 9.0, device="cuda")
    ref = _dequant_then_attention(q, kq, vq, T, k_cur, v_cur, heads, key_splits=splits, out_amax=am_a)
    out = ops.attention_nvfp4kv(q, kq, vq, T, k_cur, v_cur, heads, key_splits=splits, out_amax=am_b)
    torch.cuda.synchronize()
    assert _lib.lib().llnv_check_status(None) == 0, _lib.lib().llnv_last_error()
    assert torch.equal(out, ref)
    assert torch.equal(am_a, am_b)


def test_nvfp4kv_attention_strided_current_chunk_and_arguments():
    heads, T = 2, 128
    g = torch.Generator(device="cuda").manual_seed(4)
    kq, vq = _cache_blocks(2, T, heads, g), _cache_blocks(2, T, heads, g)
    q = torch.randn(100, heads * 128, generator=g, device="cuda").bfloat16()
    wide = torch.randn(70, 2 * heads * 128 + 64, generator=g, device="cuda").bfloat16()
    k_cur, v_cur = wide[:, : heads * 128], wide[:, heads * 128 + 64:]          # row stride larger than heads * 128
    out = ops.attention_nvfp4kv(q, kq, vq, T, k_cur, v_cur, heads)
    assert torch.equal(out, _dequant_then_attention(q, kq, vq, T, k_cur.contiguous(), v_cur.contiguous(), heads))
    with pytest.raises(RuntimeError, match="cache block"):
        ops.attention_nvfp4kv(q, kq, vq, 4 * T, k_cur, v_cur, heads)                 # blocks too small for that many tokens
    with pytest.raises(RuntimeError, match="same length"):
        ops.attention_nvfp4kv(q, kq, vq[:1], T, k_cur, v_cur, heads)
    with pytest.raises(RuntimeError, match="0 to 16 cache blocks"):
        ops.attention_nvfp4kv(q, kq * 9, vq * 9, T, k_cur, v_cur, heads)
    with pytest.raises(RuntimeError, match="at least 128"):
        ops.attention_nvfp4kv(q, kq, vq, 64, k_cur, v_cur, heads)


def test_config3_window_attention_full_size_vs_oracle():
    """The benchmark's attention configuration: 24 heads, a chunk of 2640 queries at frames 12-14, window = 4
    cached NVFP4 blocks of 2640 tokens (RoPE'd at their frame positions, frames 0-11) + the current chunk
    (k_smooth-ed keys) = 13200 keys.  Cache write and attention run at full size on the GPU; the oracle
    (dequantize with the fused rounding, fp32 attention) checks 2 of the 24 heads, and the cache blocks bit for bit."""
    heads, T, blocks, fh, fw = 24, 2640, 4, 22, 40
    C = heads * 128
    g = torch.Generator(device="cuda").manual_seed(33)
    ones = torch.ones(C, dtype=torch.bfloat16, device="cuda")
    kq, vq = [], []
    for b in range(blocks):
        cos, sin = (torch.from_numpy(t).cuda() for t in O.rope_tables(3 * b, 3, fh, fw))
        k_raw = torch.randn(T, C, generator=g, device="cuda").bfloat16()
        v_raw = torch.randn(T, C, generator=g, device="cuda").bfloat16()
        k_rot, _, _ = ops.rmsnorm_rope(k_raw, None, cos, sin)
        kq.append(L.quantize_to_fp4(k_rot.reshape(T * heads, 128)))
        vq.append(L.quantize_to_fp4(v_raw.reshape(T * heads, 128)))
        if b == 1:      # the written block is the oracle's quantization of the rotated keys, bit for bit
            # (the rotation itself is compared with the oracle in tests/test_gpu_rope_norm.py: equal up to one bf16 ulp)
            oc, osf, oam = O.quantize_nvfp4(k_rot.float().cpu().numpy().reshape(T * heads, 128), "mse")
            assert np.array_equal(kq[-1].values.cpu().numpy(), oc) and np.array_equal(util.u8(kq[-1].scale_factors), osf)
            assert float(kq[-1].amax.item()) == float(oam)
    cos, sin = (torch.from_numpy(t).cuda() for t in O.rope_tables(12, 3, fh, fw))
    q_raw = torch.randn(T, C, generator=g, device="cuda").bfloat16()
    k_raw = torch.randn(T, C, generator=g, device="cuda").bfloat16()
    v_new = torch.randn(T, C, generator=g, device="cuda").bfloat16()
    q_rot, _, _ = ops.rmsnorm_rope(q_raw, None, cos, sin)
    k_rot, k_sm, _ = ops.rmsnorm_rope(k_raw, None, cos, sin, want_smooth=True)
    out = ops.attention_nvfp4kv(q_rot, kq, vq, T, k_sm, v_new, heads)
    torch.cuda.synchronize()
    assert _lib.lib().llnv_check_status(None) == 0, _lib.lib().llnv_last_error()
    sel = [5, 23]
    def head_blocks(qs):
        outs = []
        for t in qs:
            d = O.dequantize(t.values.cpu().numpy(), util.u8(t.scale_factors), np.float32(t.amax.item()), "mse", (T * heads, 128),
                             O.DEQ_FUSED_CUDA, out_bf16=True)
            outs.append(d.reshape(T, heads, 128)[:, sel])
        return np.concatenate(outs, 0)
    kw = np.concatenate([head_blocks(kq), k_sm.float().cpu().numpy().reshape(T, heads, 128)[:, sel]], 0)
    vw = np.concatenate([head_blocks(vq), v_new.float().cpu().numpy().reshape(T, heads, 128)[:, sel]], 0)
    ref = O.attention(q_rot.float().cpu().numpy().reshape(T, heads, 128)[:, sel], kw, vw)
    got = out.view(T, heads, 128)[:, sel]
    check(got, ref)


def test_amax_accumulate_mode_keeps_the_larger_value():
    """llnv_set_amax_accumulate(1): the attention entry points no longer clear out_amax themselves, so the scalar ends up as
    max(what it held, max |out|); with the mode off (the default) it is overwritten.  The previous mask is returned."""
    lib = _lib.lib()
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(200, 256, generator=g, device="cuda").bfloat16()
    k = torch.randn(300, 256, generator=g, device="cuda").bfloat16()
    v = torch.randn(300, 256, generator=g, device="cuda").bfloat16()
    amax = torch.full((1,), 1.0e6, device="cuda")
    out = ops.attention_bf16(q, k, v, 2, out_amax=amax)
    true_max = float(out.float().abs().max().item())
    assert float(amax.item()) == true_max                     # default: overwritten
    assert lib.llnv_set_amax_accumulate(1) == 0
    try:
        amax.fill_(1.0e6)
        ops.attention_bf16(q, k, v, 2, out_amax=amax)
        assert float(amax.item()) == 1.0e6                    # kept: larger than anything the call produces
        amax.zero_()
        ops.attention_bf16(q, k, v, 2, out_amax=amax)
        assert float(amax.item()) == true_max                 # cleared by the caller: the call's own maximum
    finally:
        assert lib.llnv_set_amax_accumulate(0) == 1


def test_attention_caller_owned_workspace():
    """A split call uses the caller's workspace when one is given (same result as with a per-call allocation) and refuses
    one that is too small."""
    g = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randn(300, 256, generator=g, device="cuda").bfloat16()
    k = torch.randn(1024, 256, generator=g, device="cuda").bfloat16()
    v = torch.randn(1024, 256, generator=g, device="cuda").bfloat16()
    need = ops.attention_workspace_bytes(300, 1024, 2, key_splits=4)
    assert need == 4 * 300 * 2 * 130 * 4 and ops.attention_workspace_bytes(300, 1024, 2, key_splits=1) == 0
    ws = torch.empty(need + 64, dtype=torch.uint8, device="cuda")
    a = ops.attention_bf16(q, k, v, 2, key_splits=4, workspace=ws)
    b = ops.attention_bf16(q, k, v, 2, key_splits=4)
    assert torch.equal(a, b)
    with pytest.raises(RuntimeError, match="workspace"):
        ops.attention_bf16(q, k, v, 2, key_splits=4, workspace=ws[: need - 16])
