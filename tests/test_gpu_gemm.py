"""W4A4 GEMM parity against the oracle's dequantize-then-fp32-matmul path.

Tolerance (stated by the task for fp32-accumulate GEMMs): the kernel and the oracle both
accumulate in fp32 but in different orders and the kernel applies the tensor scales once
(alpha) instead of per element, so results are compared after the bf16 output rounding with
  |d - ref| <= 2 bf16 ulps of |ref| + K * 2^-24 * scale   and   rel. Frobenius error <= 4e-3.
"""
import ctypes

import numpy as np
import pytest
import torch

import longlive_b200 as L
from longlive_b200 import _lib, ops
from oracle import nvfp4_oracle as O
from tests import util

pytestmark = pytest.mark.gpu


def check_close(d: torch.Tensor, ref: np.ndarray, k: int, mag: np.ndarray | None = None):
    """`mag` is the magnitude the ulp tolerance refers to (the GEMM result before a bias or
    residual is added - cancellation otherwise shrinks |ref| but not the rounding error)."""
    d = d.float().cpu().numpy()
    mag = np.abs(ref) if mag is None else mag
    scale = mag.mean() + 1e-12
    tol = mag * 2.0 ** -6 + k * 2.0 ** -24 * scale + 1e-30
    bad = np.abs(d - ref) > tol
    assert not bad.any(), f"{bad.sum()} / {bad.size} outside tolerance; max abs diff {np.abs(d - ref).max()}"
    rel = np.linalg.norm(d - ref) / (np.linalg.norm(ref) + 1e-30)
    assert rel <= 4e-3, rel


def oracle_matmul(xq, wq, m, n, k):
    a = O.dequantize(xq.values.cpu().numpy(), util.u8(xq.scale_factors), np.float32(xq.amax.item()), xq.scale_rule.value, (m, k))
    b = O.dequantize(wq.values.cpu().numpy(), util.u8(wq.scale_factors), np.float32(wq.amax.item()), wq.scale_rule.value, (n, k))
    return a @ b.T


@pytest.mark.parametrize("tile_n", [128, 256, 2])     # 2 = CTA-pair kernel (256 x 256 tile per pair)
@pytest.mark.parametrize("m,n,k", [(128, 256, 256), (200, 256, 512), (880, 512, 3072), (130, 1024, 1024), (512, 3072, 3072)])
def test_gemm_matches_oracle(m, n, k, tile_n):
    x = util.config_activation(m, k, seed=m + k)
    w = util.config_weight(n, k, seed=n)
    xq = L.quantize_to_fp4(x.cuda())
    wq = L.quantize_to_fp4(w.cuda())
    y = ops.gemm_nvfp4(xq.values, xq.scale_factors, xq.amax, 3, wq.values, wq.scale_factors, wq.amax, 3, m, n, k, tile=tile_n)
    torch.cuda.synchronize()
    assert _lib.lib().llnv_check_status(None) == 0
    assert y.shape == (m, n) and y.dtype == torch.bfloat16
    check_close(y, O.bf16_round(oracle_matmul(xq, wq, m, n, k)), k)
    assert torch.equal(y, L.fp4_matmul(xq, wq))          # the public entry (automatic tiling) gives the same bits


def test_gemm_small_fixture(golden):
    g = golden("matmul_small.npz")
    a = util.bf16_np_to_torch(g["a"])
    b = util.bf16_np_to_torch(g["b"])
    for ra, rb in [("mse", "mse"), ("static_6", "static_6"), ("mse", "static_6"), ("abs_max", "mae")]:
        y = L.fp4_matmul(a, b, input_config=L.QuantizationConfig(scale_rule=ra), other_config=L.QuantizationConfig(scale_rule=rb))
        assert y.shape == (200, 136)
        check_close(y, O.bf16_from_bits(g[f"y_{ra}_{rb}"]), 256)


def test_gemm_exactness_on_integer_data():
    """Codes/scales chosen so every product and partial sum is exactly representable: the GEMM
    must be exact, which pins operand order, the scale-factor layout in tensor memory and the
    K advance inside the swizzled tile."""
    m, n, k = 256, 512, 1024
    gen = torch.Generator().manual_seed(9)
    a = torch.randint(-3, 4, (m, k), generator=gen).float()
    b = torch.randint(-3, 4, (n, k), generator=gen).float()
    # per-16-block power-of-two scaling keeps everything exact in e2m1 x e4m3
    sa = 2.0 ** torch.randint(-2, 3, (m, k // 16), generator=gen).float()
    sb = 2.0 ** torch.randint(-2, 3, (n, k // 16), generator=gen).float()
    a = (a * sa.repeat_interleave(16, 1))
    b = (b * sb.repeat_interleave(16, 1))
    a[0, 0] = 12.0 * 4   # make the tensor amax a value that keeps the scales powers of two
    b[0, 0] = 12.0 * 4
    xq = L.quantize_to_fp4(a.bfloat16().cuda(), L.QuantizationConfig(scale_rule="static_6"))
    wq = L.quantize_to_fp4(b.bfloat16().cuda(), L.QuantizationConfig(scale_rule="static_6"))
    ref = oracle_matmul(xq, wq, m, n, k)
    y = L.fp4_matmul(xq, wq)
    check_close(y, O.bf16_round(ref), k)


def test_linear_module_with_bias_matches_oracle():
    torch.manual_seed(0)
    lin = torch.nn.Linear(512, 768, bias=True).to(torch.bfloat16)
    lin.bias.data = torch.randn(768).bfloat16()
    x = util.config_activation(300, 512, seed=3).view(1, 300, 512)
    w_np = lin.weight.data.float().numpy()
    ql = L.FourOverSixLinear(lin.cuda(), L.ModuleQuantizationConfig())
    ql.materialize()
    assert ql.weight is None and ql.quantized_weight_values.shape == (768, 256)
    y = ql(x.cuda())
    assert y.shape == (1, 300, 768)
    wq = O.quantize_nvfp4(w_np, "mse")
    bias_np = lin.bias.data.float().cpu().numpy()
    ref = O.linear_forward(x[0].float().numpy(), wq, (768, 512), bias_np)
    nobias = O.linear_forward(x[0].float().numpy(), wq, (768, 512))
    check_close(y[0], ref, 512, mag=np.abs(nobias) + np.abs(bias_np)[None, :])


def test_gemm_fused_epilogue_matches_unfused_chain():
    m, n, k, frames = 264, 512, 768, 3
    x = util.config_activation(m, k, seed=1).cuda()
    w = util.config_weight(n, k, seed=2).cuda()
    xq, wq = L.quantize_to_fp4(x), L.quantize_to_fp4(w)
    g = torch.Generator().manual_seed(5)
    bias = torch.randn(n, generator=g).bfloat16().cuda()
    resid = torch.randn(m, n, generator=g).bfloat16().cuda()
    gate = torch.randn(frames, n, generator=g).bfloat16().cuda()
    base = L.fp4_matmul(xq, wq)
    args = (xq.values, xq.scale_factors, xq.amax, 3, wq.values, wq.scale_factors, wq.amax, 3, m, n, k)
    # bias
    y = ops.gemm_nvfp4(*args, bias=bias)
    assert torch.equal(y, base + bias)
    # bias + GELU(tanh)
    y = ops.gemm_nvfp4(*args, bias=bias, act=1)
    ref = torch.nn.functional.gelu((base + bias).float(), approximate="tanh").bfloat16()
    assert ((y.float() - ref.float()).abs() <= ref.float().abs() * 2.0 ** -7 + 1e-6).all()
    # bias + gate * y + residual, and the amax of the result
    amax = torch.zeros(1, dtype=torch.float32, device="cuda")
    y = ops.gemm_nvfp4(*args, bias=bias, residual=resid, gate=gate, frame_rows=m // frames, out_amax=amax)
    gl = gate.repeat_interleave(m // frames, 0)
    ref = resid + (base + bias) * gl
    assert torch.equal(y, ref)
    assert float(amax.item()) == float(y.float().abs().max().item())
    # residual without gate
    y = ops.gemm_nvfp4(*args, residual=resid)
    assert torch.equal(y, resid + base)


def test_pair_kernel_fused_epilogues_match_single_cta_kernel():
    m, n, k, frames = 700, 512, 1024, 2
    x = util.config_activation(m, k, seed=11).cuda()
    w = util.config_weight(n, k, seed=12).cuda()
    xq, wq = L.quantize_to_fp4(x), L.quantize_to_fp4(w)
    g = torch.Generator().manual_seed(6)
    bias = torch.randn(n, generator=g).bfloat16().cuda()
    resid = torch.randn(m, n, generator=g).bfloat16().cuda()
    gate = torch.randn(frames, n, generator=g).bfloat16().cuda()
    args = (xq.values, xq.scale_factors, xq.amax, 3, wq.values, wq.scale_factors, wq.amax, 3, m, n, k)
    lib = _lib.lib()
    outs = {}
    for tile in (256, 2):
        a1 = torch.zeros(1, dtype=torch.float32, device="cuda")
        a2 = torch.zeros(1, dtype=torch.float32, device="cuda")
        outs[tile] = (ops.gemm_nvfp4(*args, tile=tile), ops.gemm_nvfp4(*args, bias=bias, act=1, out_amax=a1, tile=tile),
                      ops.gemm_nvfp4(*args, bias=bias, residual=resid, gate=gate, frame_rows=m // frames, out_amax=a2, tile=tile), a1, a2)
    torch.cuda.synchronize()
    assert lib.llnv_check_status(None) == 0, lib.llnv_last_error()
    for a, b in zip(outs[256], outs[2]):
        assert torch.equal(a, b)


def test_gemm_rejects_bad_shapes():
    x = L.quantize_to_fp4(torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda"))
    w = L.quantize_to_fp4(torch.zeros(128, 128, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        L.fp4_matmul(x, w)
    with pytest.raises(ValueError):
        L.fp4_matmul(x, x, backend="pytorch")


@pytest.mark.parametrize("m,n,k", [(200, 384, 512), (300, 768, 1024), (512, 3072, 3072), (2640, 3072, 3072)])
def test_gemm_192_wide_tiles(m, n, k):
    """192-wide B tiles start 0 or 64 rows into a 128-row scale atom; results equal the oracle and,
    bit for bit, the 128-wide tiling (same products, same accumulation order along K)."""
    lib = _lib.lib()
    x = util.config_activation(m, k, seed=m + k)
    w = util.config_weight(n, k, seed=n)
    xq, wq = L.quantize_to_fp4(x.cuda()), L.quantize_to_fp4(w.cuda())
    g = torch.Generator().manual_seed(8)
    bias = torch.randn(n, generator=g).bfloat16().cuda()
    resid = torch.randn(m, n, generator=g).bfloat16().cuda()
    args = (xq.values, xq.scale_factors, xq.amax, 3, wq.values, wq.scale_factors, wq.amax, 3, m, n, k)
    outs = {}
    for tile in (192, 128):
        outs[tile] = (ops.gemm_nvfp4(*args, tile=tile), ops.gemm_nvfp4(*args, bias=bias, act=1, tile=tile),
                      ops.gemm_nvfp4(*args, bias=bias, residual=resid, tile=tile))
    torch.cuda.synchronize()
    assert lib.llnv_check_status(None) == 0, lib.llnv_last_error()
    check_close(outs[192][0], O.bf16_round(oracle_matmul(xq, wq, m, n, k)), k)
    for a, b in zip(outs[192], outs[128]):
        assert torch.equal(a, b)


@pytest.mark.parametrize("m,n_each,k", [(200, 256, 512), (700, 768, 1024), (2640, 3072, 3072), (330, 3072, 3072)])
def test_grouped_gemm_equals_separate_launches(m, n_each, k):
    """Three Linears sharing their input in one launch: every output, and the output amax, equals the separate calls."""
    x = util.config_activation(m, k, seed=m + k).cuda()
    xq = L.quantize_to_fp4(x)
    ws = [L.quantize_to_fp4(util.config_weight(n_each, k, seed=50 + i).cuda() * (1 + i)) for i in range(3)]
    g = torch.Generator().manual_seed(9)
    biases = [torch.randn(n_each, generator=g).bfloat16().cuda() for _ in range(3)]
    ref, ref_am = [], []
    for w, b in zip(ws, biases):
        am = torch.zeros(1, dtype=torch.float32, device="cuda")
        ref.append(ops.gemm_nvfp4(xq.values, xq.scale_factors, xq.amax, 3, w.values, w.scale_factors, w.amax, 3, m, n_each, k, bias=b, out_amax=am))
        ref_am.append(am)
    codes = torch.cat([w.values for w in ws], 0)
    sf = torch.cat([w.scale_factors.view(torch.uint8).reshape(-1) for w in ws], 0).view(torch.float8_e4m3fn)
    amax = torch.cat([w.amax.reshape(1) for w in ws], 0)
    big = torch.zeros(m, 2 * n_each + 64, dtype=torch.bfloat16, device="cuda")        # outputs with different row strides
    outs = [torch.empty(m, n_each, dtype=torch.bfloat16, device="cuda"), big[:, :n_each], big[:, n_each + 64:]]
    ams = [torch.full((1,), 7.0, device="cuda"), None, torch.full((1,), 7.0, device="cuda")]
    ops.gemm_nvfp4_grouped(xq.values, xq.scale_factors, xq.amax, 3, codes, sf, amax, 3, m, n_each, k, outs, bias=torch.cat(biases), out_amax=ams)
    torch.cuda.synchronize()
    assert _lib.lib().llnv_check_status(None) == 0, _lib.lib().llnv_last_error()
    for o, r in zip(outs, ref):
        assert torch.equal(o, r)
    assert torch.equal(ams[0], ref_am[0]) and torch.equal(ams[2], ref_am[2])
    assert float(big[:, n_each:n_each + 64].abs().max()) == 0.0


def test_gemm_full_size_tilings_agree():
    """At the benchmark's FFN shape the 256-, 192-... tilings and the CTA-pair kernel give bit-identical
    results (same products, same order along K), and a row of ones through identical weights repeats."""
    m, n, k = 2640, 3072, 14336
    x = util.config_activation(m, k, seed=3).cuda()
    w = util.config_weight(n, k, seed=4).cuda()
    xq, wq = L.quantize_to_fp4(x), L.quantize_to_fp4(w)
    args = (xq.values, xq.scale_factors, xq.amax, 3, wq.values, wq.scale_factors, wq.amax, 3, m, n, k)
    lib = _lib.lib()
    outs = []
    for tile in (256, 192, 128, 2):
        outs.append(ops.gemm_nvfp4(*args, tile=tile))
    torch.cuda.synchronize()
    assert lib.llnv_check_status(None) == 0, lib.llnv_last_error()
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    assert torch.isfinite(outs[0].float()).all()


def _sampled_oracle(xq, wq, m, n, k, rows):
    """Oracle result for a sample of output rows (every row of A meets all of B, so sampled rows still cover every
    N tile, every K block and every scale atom of B; the sample spreads over all M tiles and lanes)."""
    a = O.dequantize(xq.values.cpu().numpy(), util.u8(xq.scale_factors), np.float32(xq.amax.item()), xq.scale_rule.value, (m, k))
    b = O.dequantize(wq.values.cpu().numpy(), util.u8(wq.scale_factors), np.float32(wq.amax.item()), wq.scale_rule.value, (n, k))
    return a[rows] @ b.T


@pytest.mark.parametrize("m,n,k,tiles", [
    (2640, 14336, 3072, (0, 256, 2)),      # ffn.0 of the DiT block
    (2640, 3072, 14336, (0, 256, 2)),      # ffn.2 (the automatic choice is the CTA-pair kernel)
    (10560, 3072, 3072, (0, 2)),           # q/k/v/o at the largest token count of the sweep
    (10560, 14336, 3072, (0,)),
    (880, 3072, 14336, (0, 128)),
])
def test_gemm_benchmark_shapes_match_oracle(m, n, k, tiles):
    """The FFN shapes and the M = 10560 shapes of the benchmark sweep against the oracle's dequantize-then-fp32-matmul
    (not merely against another tiling): 264 output rows, 8 from every 33rd part of M with the last M tile included."""
    x = util.config_activation(m, k, seed=m + k).cuda()
    w = util.config_weight(n, k, seed=n + k).cuda()
    xq, wq = L.quantize_to_fp4(x), L.quantize_to_fp4(w)
    del x, w
    step = m // 33
    rows = np.unique(np.concatenate([np.arange(i * step + (i * 37) % 97, i * step + (i * 37) % 97 + 8) for i in range(33)] + [np.arange(m - 8, m)]))
    rows = rows[rows < m]
    ref = O.bf16_round(_sampled_oracle(xq, wq, m, n, k, rows))
    args = (xq.values, xq.scale_factors, xq.amax, 3, wq.values, wq.scale_factors, wq.amax, 3, m, n, k)
    first = None
    for tile in tiles:
        y = ops.gemm_nvfp4(*args, tile=tile)
        torch.cuda.synchronize()
        assert _lib.lib().llnv_check_status(None) == 0, _lib.lib().llnv_last_error()
        check_close(y[torch.from_numpy(rows).cuda()], ref, k)
        if first is None:
            first = y
        else:
            assert torch.equal(y, first)


@pytest.mark.parametrize("m,n,k,tile,act", [(300, 512, 768, 0, 1), (300, 512, 768, 256, 0), (264, 768, 512, 192, 1), (2640, 14336, 3072, 0, 1)])
def test_gemm_epilogue_requantizes_its_output(m, n, k, tile, act):
    """The epilogue variant that also writes the NVFP4 form of its result, with the tensor amax given up front:
    codes and scales equal the standalone quantizer's (and the oracle's) on the bf16 result, bit for bit; rows M..Mp-1
    are zero; the bf16 result is unchanged, or not written at all when the caller does not want it."""
    x = util.config_activation(m, k, seed=m + 1).cuda()
    w = util.config_weight(n, k, seed=n + 1).cuda()
    xq, wq = L.quantize_to_fp4(x), L.quantize_to_fp4(w)
    g = torch.Generator().manual_seed(3)
    bias = torch.randn(n, generator=g).bfloat16().cuda()
    args = (xq.values, xq.scale_factors, xq.amax, 3, wq.values, wq.scale_factors, wq.amax, 3, m, n, k)
    y = ops.gemm_nvfp4(*args, bias=bias, act=act, tile=tile)
    # the amax a caller would supply: here the true one and, second, a stale one that is too small (values then
    # saturate exactly as the quantizer saturates them)
    for scale in (1.0, 0.5):
        amax = (y.float().abs().max() * scale).reshape(1).bfloat16().float().contiguous()
        mp = ops.padded_rows(m)
        ref_codes, ref_sf, _ = ops.quantize_nvfp4(y, 3, amax.clone(), amax_given=True)
        codes = torch.full((mp, n // 2), 0xAB, dtype=torch.uint8, device="cuda")
        sf = torch.full((mp * n // 16,), 0x55, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
        y2 = ops.gemm_nvfp4(*args, bias=bias, act=act, tile=tile, requant=(codes, sf), requant_amax=amax)
        torch.cuda.synchronize()
        assert _lib.lib().llnv_check_status(None) == 0, _lib.lib().llnv_last_error()
        assert torch.equal(y2, y)
        assert torch.equal(codes, ref_codes) and torch.equal(sf.view(torch.uint8), ref_sf.view(torch.uint8))
        assert int(codes[m:].max().item()) == 0 if mp > m else True
        codes.fill_(0xAB)
        none = ops.gemm_nvfp4(*args, bias=bias, act=act, tile=tile, requant=(codes, sf), requant_amax=amax, store_out=False)
        assert none is None and torch.equal(codes, ref_codes)
        if m <= 512 and scale == 1.0:        # and the oracle, for the small cases (an amax below the true maximum is outside
            # what the reference's quantizer defines: its E4M3 cast does not saturate)
            oc, osf, _ = O.quantize_nvfp4(y.float().cpu().numpy(), "mse", amax=np.float32(amax.item()))
            assert np.array_equal(codes.cpu().numpy(), oc) and np.array_equal(util.u8(sf), osf)
    # the consumer GEMM reads the epilogue's codes like any quantized activation
    w2 = L.quantize_to_fp4(util.config_weight(256, n, seed=9).cuda())
    a = ops.gemm_nvfp4(codes, sf, amax, 3, w2.values, w2.scale_factors, w2.amax, 3, m, 256, n)
    b = ops.gemm_nvfp4(ref_codes, ref_sf, amax, 3, w2.values, w2.scale_factors, w2.amax, 3, m, 256, n)
    assert torch.equal(a, b)


def test_gemm_requant_argument_checks():
    x = L.quantize_to_fp4(torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda"))
    w = L.quantize_to_fp4(torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda"))
    args = (x.values, x.scale_factors, x.amax, 3, w.values, w.scale_factors, w.amax, 3, 128, 256, 256)
    codes = torch.zeros(128, 128, dtype=torch.uint8, device="cuda")
    sf = torch.zeros(128 * 16, dtype=torch.uint8, device="cuda")
    amax = torch.ones(1, device="cuda")
    with pytest.raises(ValueError, match="requant_amax"):
        ops.gemm_nvfp4(*args, requant=(codes, sf))
    with pytest.raises(RuntimeError, match="residual"):
        ops.gemm_nvfp4(*args, requant=(codes, sf), requant_amax=amax, residual=torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError, match="store_out"):
        ops.gemm_nvfp4(*args, store_out=False)


def test_fp4_mma_rate_probe_runs_and_reports_its_flop():
    """The MMA issue-rate probe launches (bounded wait inside), leaves the status word clean and reports
    2 * 128 * 256 * 256 flop per K block and SM."""
    import ctypes
    lib = _lib.lib()
    flop = ctypes.c_double()
    _lib.check(lib.llnv_fp4_mma_rate(64, ctypes.byref(flop), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert lib.llnv_check_status(None) == 0, lib.llnv_last_error()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert flop.value == 2.0 * 128 * 256 * 256 * 64 * sms
    with pytest.raises(Exception):
        _lib.check(lib.llnv_fp4_mma_rate(0, None, None))
