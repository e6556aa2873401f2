"""CUDA quantizer / dequantize parity: bit-exact against the numpy oracle and the golden
fixtures generated from the reference."""
import hashlib

import numpy as np
import pytest
import torch

import longlive_b200 as L
from longlive_b200 import ops
from oracle import nvfp4_oracle as O
from tests import util

pytestmark = pytest.mark.gpu
RULES = ["static_6", "static_4", "mae", "mse", "abs_max"]


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.mark.parametrize("case", ["edge", "randn", "zeros"])
@pytest.mark.parametrize("rule", RULES)
def test_quantize_matches_reference_fixtures(golden, case, rule):
    g = golden("quantize_small.npz")
    x = util.bf16_np_to_torch(g[f"{case}_x"])
    q = L.quantize_to_fp4(x, L.QuantizationConfig(scale_rule=rule))
    assert q.padded_shape == tuple(g[f"{case}_{rule}_padded"])
    assert float(q.amax.item()) == float(g[f"{case}_{rule}_amax"])
    assert np.array_equal(util.u8(q.scale_factors), g[f"{case}_{rule}_sf"])
    assert np.array_equal(q.values.cpu().numpy(), g[f"{case}_{rule}_codes"])
    for dtype, key in ((torch.float32, "deq_f32"), (torch.bfloat16, "deq_bf16")):
        d = q.dequantize(dtype)
        if dtype == torch.float32:
            assert np.array_equal(d.cpu().numpy().view(np.uint32), g[f"{case}_{rule}_{key}"].view(np.uint32))
        else:
            assert np.array_equal(util.torch_bf16_bits(d), g[f"{case}_{rule}_{key}"])


@pytest.mark.parametrize("rule", RULES)
def test_quantize_ragged_columns(golden, rule):
    g = golden("quantize_small.npz")          # [130, 320]: rows padded to 256, 320 is already a multiple of 64
    x = util.bf16_np_to_torch(g["ragged_x"])
    q = L.quantize_to_fp4(x, L.QuantizationConfig(scale_rule=rule))
    assert q.original_shape == (130, 320) and q.padded_shape == (256, 320)
    assert np.array_equal(util.u8(q.scale_factors), g[f"ragged_{rule}_sf"])
    assert np.array_equal(q.values.cpu().numpy(), g[f"ragged_{rule}_codes"])
    assert np.array_equal(util.torch_bf16_bits(q.dequantize(torch.bfloat16)), g[f"ragged_{rule}_deq_bf16"])


def test_quantize_config1_activation_and_weight(golden):
    g = golden("config1_linear.npz")
    torch.manual_seed(0)
    M, K, N = 2640, 3072, 3072
    x = torch.randn(M, K)
    x = torch.where(torch.rand(M, K) < 0.001, x * 20, x).bfloat16()
    w = (torch.randn(N, K) * 0.02).bfloat16()
    assert sha(util.torch_bf16_bits(x)) == str(g["x_sha"])
    xq = L.quantize_to_fp4(x.cuda())
    wq = L.quantize_to_fp4(w.cuda())
    assert float(xq.amax.item()) == float(g["x_amax"]) and float(wq.amax.item()) == float(g["w_amax"])
    assert sha(xq.values.cpu().numpy()) == str(g["x_codes_sha"])
    assert sha(util.u8(xq.scale_factors)) == str(g["x_sf_sha"])
    assert sha(wq.values.cpu().numpy()) == str(g["w_codes_sha"])
    assert sha(util.u8(wq.scale_factors)) == str(g["w_sf_sha"])


@pytest.mark.parametrize("shape", [(1, 64), (127, 128), (129, 192), (512, 14336), (880, 3072)])
def test_quantize_vs_oracle_shapes(shape):
    x = util.config_activation(*shape, seed=shape[0])
    q = L.quantize_to_fp4(x.cuda())
    codes, sf, amax = O.quantize_nvfp4(x.float().numpy(), "mse")
    assert float(q.amax.item()) == float(amax)
    assert np.array_equal(util.u8(q.scale_factors), sf)
    assert np.array_equal(q.values.cpu().numpy(), codes)


def test_quantize_given_amax_and_strided_input():
    x = util.config_activation(256, 512, seed=5)
    big = torch.zeros(256, 1024, dtype=torch.bfloat16)
    big[:, 256:768] = x
    view = big.cuda()[:, 256:768]
    amax = torch.tensor([37.5], dtype=torch.float32, device="cuda")
    q = L.quantize_to_fp4(view, L.QuantizationConfig(scale_rule="mse"), amax=amax)
    codes, sf, _ = O.quantize_nvfp4(x.float().numpy(), "mse", amax=np.float32(37.5))
    assert np.array_equal(q.values.cpu().numpy(), codes) and np.array_equal(util.u8(q.scale_factors), sf)


def test_quantize_properties_full_size():
    """Size-independent checks on the largest benchmark activation (10560 x 14336)."""
    m, k = 10560, 14336
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(m, k, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    q = L.quantize_to_fp4(x)
    assert float(q.amax.item()) == float(x.abs().max().item())
    d = q.dequantize(torch.float32)
    rel = ((d - x.float()).norm() / x.float().norm()).item()
    assert rel < 0.12                                    # NVFP4 4-over-6 on gaussian data: ~9 %
    # idempotence: quantizing the dequantized tensor with the same amax reproduces codes and scales
    q2 = L.quantize_to_fp4(d.bfloat16(), amax=q.amax)
    d2 = q2.dequantize(torch.float32)
    assert ((d2 - d.bfloat16().float()).abs().max() <= d.abs().max() * 0.07).item()
    # padding rows are zero codes / zero scales
    assert q.values.shape[0] == 10624 and int(q.values[m:].max().item()) == 0


def test_kv_dequant_matches_oracle_and_fixture(golden):
    g = golden("kv_small.npz")
    codes = torch.from_numpy(g["codes"]).cuda()
    sf = torch.from_numpy(g["sf"]).cuda().view(torch.float8_e4m3fn)
    amax = torch.tensor([float(g["amax"])], dtype=torch.float32, device="cuda")
    T, H = 48, 4
    qt = L.QuantizedTensor(codes, sf, amax, "nvfp4", (T * H, 128), "mse")
    out = ops.kv_dequant([codes], [sf], [amax], H, T, torch.bfloat16, 6, 256, ops.DEQ_PYTORCH)
    assert np.array_equal(util.torch_bf16_bits(out[0]), g["deq_bf16"])
    blocks = []
    for i in range(3):
        k = torch.randn(T * H, 128, generator=torch.Generator().manual_seed(40 + i)).bfloat16() * (i + 1)
        blocks.append(L.quantize_to_fp4(k.cuda()))
    fused = L.dequantize_kv_cache(blocks + [qt], 4, H, T, torch.bfloat16, "cuda")
    assert fused.shape == (1, 4 * T, H, 128)
    ref = O.dequantize_kv_cache([(b.values.cpu().numpy(), util.u8(b.scale_factors), np.float32(b.amax.item()))
                                 for b in blocks + [qt]], H, T, "mse", O.DEQ_FUSED_CUDA)
    assert np.array_equal(util.torch_bf16_bits(fused), O.bf16_bits(ref))
    for dt, name in ((torch.float16, "fp16"), (torch.float32, "fp32")):
        o = L.dequantize_kv_cache(blocks, 3, H, T, dt, "cuda")
        ref = O.dequantize_kv_cache([(b.values.cpu().numpy(), util.u8(b.scale_factors), np.float32(b.amax.item()))
                                     for b in blocks], H, T, "mse", O.DEQ_FUSED_CUDA, dtype=name)
        assert o.dtype == dt and o.shape == (1, 3 * T, H, 128)
        assert np.array_equal(o.float().cpu().numpy().view(np.uint32), ref.view(np.uint32))      # bit for bit


def test_kv_slot_helpers():
    T, H = 16, 8
    k = torch.randn(T * H, 128, generator=torch.Generator().manual_seed(2)).bfloat16().cuda()
    slot = L.quantize_to_fp4(torch.zeros_like(k))
    ptrs = (slot.values.data_ptr(), slot.scale_factors.data_ptr(), slot.amax.data_ptr())
    src = L.quantize_to_fp4(k)
    L.copy_quantized_into(slot, src)
    assert torch.equal(slot.values, src.values) and torch.equal(slot.amax, src.amax)
    assert ptrs == (slot.values.data_ptr(), slot.scale_factors.data_ptr(), slot.amax.data_ptr())
    clone = L.clone_quantized_tensor(slot)
    assert clone.values.data_ptr() != slot.values.data_ptr() and torch.equal(clone.values, slot.values)
    # in-place quantize into the slot (no staging copy)
    k2 = (k * 3).contiguous()
    L.quantize_to_fp4(k2, out=slot)
    ref = L.quantize_to_fp4(k2)
    assert torch.equal(slot.values, ref.values) and torch.equal(slot.amax, ref.amax)
    assert torch.equal(slot.scale_factors.view(torch.uint8), ref.scale_factors.view(torch.uint8))
    ks = L.k_smooth(k.view(1, T, H, 128))
    assert np.array_equal(util.torch_bf16_bits(ks), O.bf16_bits(O.k_smooth(k.view(1, T, H, 128).float().cpu().numpy())))


def test_c_abi_error_reporting():
    x = torch.zeros(128, 96, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 64"):
        ops.quantize_nvfp4(x, 3)
    with pytest.raises(RuntimeError, match="at least one cache block"):
        ops.kv_dequant([], [], [], 4, 4, torch.bfloat16, 6, 256)


def test_exact_division():
    """The quantizer's multiply-and-correct division by 6 and by 1536 must agree with IEEE division
    for every finite fp32 value whose magnitude is at least 2^-100 (the fast path never sees
    smaller operands); checked exhaustively over those bit patterns, both signs."""
    import ctypes
    from longlive_b200 import _lib
    lib = _lib.lib()
    counter = torch.zeros(1, dtype=torch.int64, device="cuda")
    lo_bits = (127 - 100) << 23                      # 2^-100
    hi_bits = 0x7F800000                             # +inf (excluded by the kernel)
    for divisor in (6, 1536):
        for sign in (0, 0x80000000):
            counter.zero_()
            rc = lib.llnv_selftest_div_const(divisor, ctypes.c_uint32(sign | lo_bits), ctypes.c_uint64(hi_bits - lo_bits),
                                             counter.data_ptr(), None)
            assert rc == 0
            torch.cuda.synchronize()
            assert int(counter.item()) == 0, (divisor, sign, int(counter.item()))


@pytest.mark.parametrize("shards", [2, 4])
def test_quantize_column_sharded_input(shards):
    """A [shards, M, K/shards] activation (the layout the head -> token exchange delivers) gives the
    codes, scales and amax of the [M, K] matrix it represents."""
    m, k = 200, 512
    g = torch.Generator().manual_seed(31)
    x = (torch.randn(m, k, generator=g) * 2).bfloat16().cuda()
    xs = x.view(m, shards, k // shards).permute(1, 0, 2).contiguous()
    ref = ops.quantize_nvfp4(x, 3)
    got = ops.quantize_nvfp4(xs, 3)
    for a, b in zip(ref, got):
        assert torch.equal(a.view(torch.uint8) if a.dtype != torch.float32 else a, b.view(torch.uint8) if b.dtype != torch.float32 else b)


def test_quantize_two_tensors_in_one_launch():
    g = torch.Generator().manual_seed(37)
    a = torch.randn(300, 128, generator=g).bfloat16().cuda()
    b = (torch.randn(300, 128, generator=g) * 5).bfloat16().cuda()
    ra, rb = L.quantize_to_fp4(a), L.quantize_to_fp4(b)
    qa, qb = L.quantize_to_fp4(torch.zeros_like(a)), L.quantize_to_fp4(torch.zeros_like(b))
    for given in (False, True):
        if given:
            qa.amax.copy_(ra.amax); qb.amax.copy_(rb.amax)
            qa.values.zero_(); qb.values.zero_()
        ops.quantize_nvfp4_pair(a, b, 3, qa, qb, amax_given=given)
        for r, q in ((ra, qa), (rb, qb)):
            assert torch.equal(r.values, q.values) and torch.equal(r.amax, q.amax)
            assert torch.equal(r.scale_factors.view(torch.uint8), q.scale_factors.view(torch.uint8))


@pytest.mark.parametrize("rule", RULES)
def test_quantize_fp16_input(golden, rule):
    """fp16 activations (accepted by the reference's CUDA backend beside bf16): codes, scales and amax equal the
    reference's PyTorch quantizer on the fixture tensor and the oracle on a larger seeded one, with and without a given
    amax; the custom op takes fp16 as well."""
    g = golden("quantize_fp16.npz")
    x = torch.from_numpy(g["x"].view(np.int16).copy()).view(torch.float16)
    q = L.quantize_to_fp4(x.cuda(), L.QuantizationConfig(scale_rule=rule))
    assert q.original_shape == tuple(x.shape) and float(q.amax.item()) == float(g[f"{rule}_amax"])
    assert np.array_equal(util.u8(q.scale_factors), g[f"{rule}_sf"]) and np.array_equal(q.values.cpu().numpy(), g[f"{rule}_codes"])
    gen = torch.Generator().manual_seed(77)
    big = (torch.randn(520, 1024, generator=gen) * 3)
    big = torch.where(torch.rand(520, 1024, generator=gen) < 0.002, big * 50, big).half()
    oc, osf, oamax = O.quantize_nvfp4(big.float().numpy(), rule)
    qb = L.quantize_to_fp4(big.cuda(), L.QuantizationConfig(scale_rule=rule))
    assert float(qb.amax.item()) == float(oamax) and np.array_equal(util.u8(qb.scale_factors), osf)
    assert np.array_equal(qb.values.cpu().numpy(), oc)
    q2 = L.quantize_to_fp4(big.cuda(), L.QuantizationConfig(scale_rule=rule), amax=qb.amax.clone())
    assert torch.equal(q2.values, qb.values) and torch.equal(q2.scale_factors.view(torch.uint8), qb.scale_factors.view(torch.uint8))
    if rule == "mse":
        import longlive_b200.torch_ops  # noqa: F401  (registers torch.ops.llnvfp4)
        v, s, a = torch.ops.llnvfp4.quantize_to_fp4(big.cuda(), True, True, False, False, False, 3, 0)
        assert torch.equal(v, qb.values) and torch.equal(s.view(torch.uint8), qb.scale_factors.view(torch.uint8)) and torch.equal(a, qb.amax)
