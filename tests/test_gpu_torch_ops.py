"""The custom-op seams (longlive_b200/torch_ops.py): results equal the direct calls, the fake implementations give
the real outputs' shapes and dtypes, and a module built on them traces under torch.compile(fullgraph=True)."""
import pytest
import torch

import longlive_b200 as L
from longlive_b200 import ops, torch_ops  # noqa: F401  (registers the ops)
from tests import util

pytestmark = pytest.mark.gpu


class TinyLinear(torch.nn.Module):
    """x -> fp4 GEMM against a pre-quantized weight, through the three registered ops only."""

    def __init__(self, wq):
        super().__init__()
        self.w_codes, self.w_sf, self.w_amax = wq.values, wq.scale_factors, wq.amax

    def forward(self, x):
        codes, sf, amax = torch.ops.llnvfp4.quantize_to_fp4(x, True, True, False, False, False, 3, 0)
        alpha = (amax * self.w_amax) / (6.0 * 256.0 * 6.0 * 256.0)
        y = torch.ops.llnvfp4.gemm_nvfp4nvfp4_accum_fp32_out_bf16_tnt(codes, self.w_codes, sf, self.w_sf, alpha)
        return y[: x.shape[0]]


def test_ops_equal_direct_calls_and_compile_fullgraph():
    x = util.config_activation(200, 512, seed=1).cuda()
    wq = L.quantize_to_fp4(util.config_weight(256, 512, seed=2).cuda())
    xq = L.quantize_to_fp4(x)
    direct = L.fp4_matmul(xq, wq)
    mod = TinyLinear(wq)
    eager = mod(x)
    assert torch.equal(eager, direct)
    compiled = torch.compile(mod, fullgraph=True, backend="aot_eager")
    assert torch.equal(compiled(x), direct)
    codes, sf, amax = torch.ops.llnvfp4.quantize_to_fp4(x, True, True, False, False, False, 3, 0)
    assert torch.equal(codes, xq.values) and torch.equal(amax, xq.amax) and torch.equal(sf.view(torch.uint8), xq.scale_factors.view(torch.uint8))
    with pytest.raises(RuntimeError, match="round-to-nearest"):
        torch.ops.llnvfp4.quantize_to_fp4(x, True, False, False, False, False, 3, 0)


def test_fake_implementations_match_real_shapes():
    from torch._subclasses.fake_tensor import FakeTensorMode
    x = util.config_activation(130, 256, seed=3).cuda()
    real = torch.ops.llnvfp4.quantize_to_fp4(x, True, True, False, False, False, 3, 0)
    T, H = 32, 4
    blocks = [L.quantize_to_fp4(torch.randn(T * H, 128, device="cuda").bfloat16()) for _ in range(2)]
    vals, sfs, ams = [b.values for b in blocks], [b.scale_factors for b in blocks], [b.amax for b in blocks]
    deq = torch.ops.llnvfp4.dequantize_kv_cache_fp4(vals, sfs, ams, H, T, 0, 6.0, 256.0)
    assert torch.equal(deq, L.dequantize_kv_cache(blocks, 2, H, T, torch.bfloat16, "cuda"))
    with FakeTensorMode() as mode:
        fx = mode.from_tensor(x)
        fake = torch.ops.llnvfp4.quantize_to_fp4(fx, True, True, False, False, False, 3, 0)
        fdeq = torch.ops.llnvfp4.dequantize_kv_cache_fp4([mode.from_tensor(v) for v in vals], [mode.from_tensor(s) for s in sfs],
                                                         [mode.from_tensor(a) for a in ams], H, T, 2, 6.0, 256.0)
    for r, f in zip(real, fake):
        assert r.shape == f.shape and r.dtype == f.dtype
    assert fdeq.shape == deq.shape and fdeq.dtype == torch.float32


def test_reference_op_names_can_be_installed():
    names = torch_ops.install_reference_aliases()
    assert set(names) <= {"fouroversix::quantize_to_fp4", "fouroversix::gemm_nvfp4nvfp4_accum_fp32_out_bf16_tnt",
                          "longlive_kernels::dequantize_kv_cache_fp4"}
    x = util.config_activation(128, 128, seed=5).cuda()
    a = torch.ops.fouroversix.quantize_to_fp4(x, True, True, False, False, False, 3, 0)
    b = torch.ops.llnvfp4.quantize_to_fp4(x, True, True, False, False, False, 3, 0)
    assert all(torch.equal(p.view(torch.uint8) if p.dtype == torch.float8_e4m3fn else p, q.view(torch.uint8) if q.dtype == torch.float8_e4m3fn else q)
               for p, q in zip(a, b))
    assert torch_ops.install_reference_aliases() == []          # second call: nothing left to install
