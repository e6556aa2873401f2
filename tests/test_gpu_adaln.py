"""adaLN / LayerNorm fused into the quantizer.

The normalisation involves fp32 reductions whose order the reference does not pin (its Triton
kernel and its eager path already differ by up to one bf16 ulp, utils/adaln_triton.py header),
so the modulated activation y is compared with the oracle within one bf16 ulp on a small
fraction of elements, while the quantizer stage is checked bit-exactly: codes / scales / amax
must equal the oracle's quantization of exactly the y the kernel produced."""
import numpy as np
import pytest
import torch

import longlive_b200 as L
from longlive_b200 import ops
from oracle import nvfp4_oracle as O
from tests import util

pytestmark = pytest.mark.gpu


def _inputs(m, c, frames, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(m, c, generator=g) * 2 + 0.3)
    x = torch.where(torch.rand(m, c, generator=g) < 0.001, x * 20, x).bfloat16()
    mod = (torch.randn(1, frames, 6, c, generator=g) * 0.2).bfloat16()
    return x, mod


@pytest.mark.parametrize("m,c,frames,rule", [(96, 256, 3, "mse"), (264, 3072, 3, "mse"), (130, 512, 2, "static_6"), (880, 3072, 1, "abs_max")])
def test_adaln_quantize(m, c, frames, rule):
    frame_rows = m // frames
    x, mod = _inputs(frame_rows * frames, c, frames, seed=m)
    m = x.shape[0]
    xd, modd = x.cuda(), mod.cuda()
    scale, shift = modd[0, :, 1], modd[0, :, 0]            # strided [F, C] views, stride 6*C
    rid = L.ScaleRule(rule).cuda_id()
    codes, sf, amax, y = ops.adaln_quantize_nvfp4(xd, scale, shift, frame_rows, rid, want_y=True)
    y_np = y.float().cpu().numpy()
    ref = O.adaln_modulate(x.float().numpy(), mod[0, :, 1].float().numpy(), mod[0, :, 0].float().numpy(), frame_rows)
    diff = np.abs(y_np - ref)
    assert (diff > 0).mean() < 0.01
    assert np.all(diff <= np.abs(ref) * 2.0 ** -6 + 2.0 ** -7)
    oc, osf, oamax = O.quantize_nvfp4(y_np, rule)
    assert float(amax.item()) == float(oamax)
    assert np.array_equal(util.u8(sf), osf)
    assert np.array_equal(codes.cpu().numpy(), oc)
    # without the y output the quantized result is the same
    c2, s2, a2, none = ops.adaln_quantize_nvfp4(xd, scale, shift, frame_rows, rid)
    assert none is None and torch.equal(c2, codes) and torch.equal(a2, amax)
    assert torch.equal(s2.view(torch.uint8), sf.view(torch.uint8))
    # transform only (the modulated LayerNorm in front of a bf16 Linear): the same y, nothing quantized
    c3, s3, a3, y3 = ops.adaln_quantize_nvfp4(xd, scale, shift, frame_rows, rid, y_only=True)
    assert c3 is None and s3 is None and torch.equal(y3, y) and torch.equal(a3, amax)


def test_adaln_matches_reference_fixture(golden):
    g = golden("elementwise_small.npz")
    x = util.bf16_np_to_torch(g["norm_x"])[0]
    sc = util.bf16_np_to_torch(g["ada_scale"])[0, :, 0]
    sh = util.bf16_np_to_torch(g["ada_shift"])[0, :, 0]
    frames = sc.shape[0]
    _, _, _, y = ops.adaln_quantize_nvfp4(x, sc, sh, x.shape[0] // frames, 3, want_y=True)
    ref = O.bf16_from_bits(g["ada_y"])[0]
    diff = np.abs(y.float().cpu().numpy() - ref)
    assert (diff > 0).mean() < 0.01 and np.all(diff <= np.abs(ref) * 2.0 ** -6 + 2.0 ** -7)


@pytest.mark.parametrize("m,c", [(200, 384), (512, 3072)])
def test_layernorm_affine_quantize(m, c):
    g = torch.Generator().manual_seed(c)
    x = (torch.randn(m, c, generator=g) * 1.5 - 0.2).bfloat16()
    w = (1 + 0.1 * torch.randn(c, generator=g)).bfloat16()
    b = (0.1 * torch.randn(c, generator=g)).bfloat16()
    codes, sf, amax, y = ops.layernorm_quantize_nvfp4(x.cuda(), w.cuda(), b.cuda(), 3, want_y=True)
    y_np = y.float().cpu().numpy()
    ref = O.layer_norm_affine(x.float().numpy(), w.float().numpy(), b.float().numpy())
    tref = torch.nn.functional.layer_norm(x.float(), (c,), w.float(), b.float(), 1e-6).bfloat16().float().numpy()
    for r in (ref, tref):
        diff = np.abs(y_np - r)
        assert (diff > 0).mean() < 0.01 and np.all(diff <= np.abs(r) * 2.0 ** -7 + 1e-6)
    oc, osf, oamax = O.quantize_nvfp4(y_np, "mse")
    assert float(amax.item()) == float(oamax) and np.array_equal(util.u8(sf), osf) and np.array_equal(codes.cpu().numpy(), oc)


def test_adaln_argument_checks():
    x = torch.zeros(64, 96, dtype=torch.bfloat16, device="cuda")
    sc = torch.zeros(1, 96, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 64"):
        ops.adaln_quantize_nvfp4(x, sc, sc, 64, 3)
