"""RMSNorm -> RoPE -> k_smooth prologue against the oracle and the reference's eager outputs.

Floating-point path: the reference pins none of these bit for bit (its Triton and eager RoPE
differ by one bf16 ulp, utils/rope_triton.py header); results must agree with the oracle within
one bf16 ulp on at most 1 % of the elements, and exactly elsewhere."""
import numpy as np
import pytest
import torch

from longlive_b200 import ops
from oracle import nvfp4_oracle as O
from tests import util

pytestmark = pytest.mark.gpu


def close(got, ref, frac=0.01, ulps=1):
    got = got.float().cpu().numpy().reshape(ref.shape)
    diff = np.abs(got - ref)
    assert (diff > 0).mean() <= frac, (diff > 0).mean()
    assert np.all(diff <= np.abs(ref) * 2.0 ** -7 * ulps + 2.0 ** -9)


def test_rope_matches_reference_fixture(golden):
    g = golden("elementwise_small.npz")
    F, H, W, start = [int(v) for v in g["rope_grid"]]
    x = util.bf16_np_to_torch(g["rope_x"])[0]                # [S, heads, 128]
    s, heads, d = x.shape
    cos, sin = O.rope_tables(start, F, H, W)
    out, _, _ = ops.rmsnorm_rope(x.reshape(s, heads * d), None, torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda())
    close(out, O.bf16_from_bits(g["rope_y"])[0].reshape(s, heads * d))


def test_rmsnorm_matches_reference_fixture(golden):
    g = golden("elementwise_small.npz")
    x = util.bf16_np_to_torch(g["norm_x"])[0]
    w = util.bf16_np_to_torch(g["rms_w"])
    out, _, _ = ops.rmsnorm_rope(x, w)
    close(out, O.bf16_from_bits(g["rms_y"])[0])


@pytest.mark.parametrize("s,heads", [(48, 2), (880, 24)])
def test_full_prologue_vs_oracle(s, heads):
    c = heads * 128
    g = torch.Generator().manual_seed(s)
    x = (torch.randn(s, c, generator=g) * 1.7).bfloat16()
    w = (1 + 0.2 * torch.randn(c, generator=g)).bfloat16()
    f, hh, ww = (1, 22, 40) if s == 880 else (2, 4, 6)
    cos, sin = O.rope_tables(7, f, hh, ww)
    out, sm, amax = ops.rmsnorm_rope(x.cuda(), w.cuda(), torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda(),
                                     want_smooth=True, want_amax=True)
    y = O.rms_norm(x.float().numpy(), w.float().numpy())
    r = O.rope_apply(y.reshape(s, heads, 128), cos, sin)
    close(out, r.reshape(s, c), frac=0.02)
    # smooth and amax are checked against the kernel's own rotated output (exact chain from there)
    got = out.float().cpu().numpy().reshape(s, heads, 128)
    assert float(amax.item()) == float(np.abs(got).max())
    close(sm, O.k_smooth(got).reshape(s, c), frac=0.005)


def test_prologue_writes_into_strided_window_buffer():
    s, c = 64, 256
    x = torch.randn(s, c, generator=torch.Generator().manual_seed(1)).bfloat16().cuda()
    window = torch.zeros(3 * s, c, dtype=torch.bfloat16, device="cuda")
    ref, _, _ = ops.rmsnorm_rope(x)
    ops.rmsnorm_rope(x, out=window[2 * s:])
    assert torch.equal(window[2 * s:], ref) and torch.equal(ref, x) and int(window[: 2 * s].abs().max().item()) == 0


@pytest.mark.parametrize("shards", [2, 4])
def test_prologue_head_sharded_outputs(shards):
    """shards > 1 writes [shards, S, C/shards] (the send layout of the token -> head exchange) with the
    same values as the plain [S, C] call."""
    s_, heads = 70, 4
    c = heads * 128
    g = torch.Generator().manual_seed(41)
    x = torch.randn(s_, c, generator=g).bfloat16().cuda()
    w = (1 + 0.1 * torch.randn(c, generator=g)).bfloat16().cuda()
    ang = torch.rand(s_, 64, generator=g) * 6.28
    cos, sin = ang.cos().float().cuda().contiguous(), ang.sin().float().cuda().contiguous()
    out, sm, am = ops.rmsnorm_rope(x, w, cos, sin, want_smooth=True, want_amax=True)
    out2, sm2, am2 = ops.rmsnorm_rope(x, w, cos, sin, want_smooth=True, want_amax=True, shards=shards)
    assert out2.shape == (shards, s_, c // shards)
    assert torch.equal(out2.permute(1, 0, 2).reshape(s_, c), out)
    assert torch.equal(sm2.permute(1, 0, 2).reshape(s_, c), sm)
    assert torch.equal(am, am2)


def test_qk_prologue_in_one_launch():
    """llnv_rmsnorm_rope_qk gives exactly what the two separate calls give."""
    s_, heads = 90, 4
    c = heads * 128
    g = torch.Generator().manual_seed(43)
    xq, xk = torch.randn(s_, c, generator=g).bfloat16().cuda(), (torch.randn(s_, c, generator=g) * 2).bfloat16().cuda()
    wq, wk = (1 + 0.1 * torch.randn(c, generator=g)).bfloat16().cuda(), (1 + 0.1 * torch.randn(c, generator=g)).bfloat16().cuda()
    ang = torch.rand(s_, 64, generator=g) * 6.28
    cos, sin = ang.cos().float().cuda().contiguous(), ang.sin().float().cuda().contiguous()
    q_ref, _, _ = ops.rmsnorm_rope(xq, wq, cos, sin)
    k_ref, ks_ref, am_ref = ops.rmsnorm_rope(xk, wk, cos, sin, want_smooth=True, want_amax=True)
    q, k, ks = torch.empty_like(q_ref), torch.empty_like(k_ref), torch.empty_like(ks_ref)
    am = torch.zeros(1, dtype=torch.float32, device="cuda")
    ops.rmsnorm_rope_qk(xq, wq, [q.data_ptr()], c, xk, wk, [k.data_ptr()], c, [ks.data_ptr()], c, am, cos, sin, 1e-6)
    assert torch.equal(q, q_ref) and torch.equal(k, k_ref) and torch.equal(ks, ks_ref) and torch.equal(am, am_ref)
