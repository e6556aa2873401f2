"""CPU restatement (numpy) of the reference's NVFP4 path.  TEST INFRASTRUCTURE ONLY.

This module is the parity checker for the CUDA kernels and the timed CPU baseline.
Only the test-suite, the smoke check and the benchmark's cpu-baseline leg may import
it; nothing in the product package does.

Parity status: PINNED for the quantizer, the scale-factor swizzle, dequantize and the
dequantize-then-matmul path - the committed fixtures under ``tests/golden`` were
produced by importing the reference's own PyTorch backend
(``tests/golden/make_golden.py``) and ``tests/test_oracle_golden.py`` checks this file
against them bit for bit.  RoPE / adaLN / RMSNorm / k_smooth / window attention are
pinned the same way against the reference's eager PyTorch code.

Every function cites the reference file:line (paths relative to the reference
repository root) whose arithmetic it follows.  All arithmetic is IEEE fp32 with each
operation rounded separately (numpy float32 does exactly that).
"""
from __future__ import annotations

import numpy as np

f32 = np.float32

E2M1_MAX = 6.0
E2M1_MAX_FOUR = 4.0
E4M3_MAX = 448.0
E4M3_MAX_FOUROVERSIX = 256.0

# ScaleRule.cuda_id(): fouroversix/src/fouroversix/utils.py:113-122
RULE_IDS = {"static_6": 0, "static_4": 1, "mae": 2, "mse": 3, "abs_max": 4}
RULE_NAMES = {v: k for k, v in RULE_IDS.items()}


def rule_limits(rule: str) -> tuple[float, float]:
    """(max E2M1 value, max E4M3 value) of a scale rule.

    fouroversix/src/fouroversix/utils.py:124-134.
    """
    e2 = 4.0 if rule == "static_4" else 6.0
    e4 = 448.0 if rule in ("static_6", "static_4") else 256.0
    return e2, e4


# --------------------------------------------------------------------------------------
# bf16 / e4m3 / e2m1 scalar formats
# --------------------------------------------------------------------------------------

def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round fp32 to the nearest bf16 (ties to even); returns fp32 holding bf16 values."""
    x = np.ascontiguousarray(x, dtype=f32)
    u = x.view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    out = rounded.astype(np.uint32).view(f32)
    return np.where(np.isnan(x), x, out).astype(f32)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """uint16 bit pattern of fp32 values that are exactly representable in bf16."""
    return (np.ascontiguousarray(x, dtype=f32).view(np.uint32) >> 16).astype(np.uint16)


def bf16_from_bits(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(f32)


def e4m3_decode(code: np.ndarray) -> np.ndarray:
    """float8_e4m3fn bit pattern -> fp32."""
    code = np.asarray(code, dtype=np.uint8)
    s = (code >> 7).astype(np.int32)
    e = ((code >> 3) & 0xF).astype(np.int32)
    m = (code & 0x7).astype(np.int32)
    mag = np.where(e == 0, m.astype(f32) * f32(2.0 ** -9),
                   np.ldexp((8 + m).astype(f32), e - 10)).astype(f32)
    mag = np.where((e == 15) & (m == 7), f32(np.nan), mag)
    return np.where(s == 1, -mag, mag).astype(f32)


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """fp32 -> float8_e4m3fn bit pattern, round-to-nearest-even.

    Follows torch's ``.to(torch.float8_e4m3fn)`` (the cast the reference uses at
    fouroversix/src/fouroversix/quantize/pytorch/reference.py:157): magnitudes that
    round beyond 448 become NaN (0x7F), no saturation.
    """
    x = np.ascontiguousarray(x, dtype=f32)
    sign = (x.view(np.uint32) >> 31).astype(np.uint8) << 7
    a = np.abs(x).astype(np.float64)
    out = np.zeros(x.shape, dtype=np.uint8)
    # spacing of the e4m3 grid at |x|: 2^(max(e,-6) - 3)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.maximum(e, -6.0)
    step = np.exp2(e - 3.0)
    q = np.rint(a / step)            # np.rint is ties-to-even; a/step is exact (power of 2)
    v = q * step                     # rounded magnitude (may have carried to next binade)
    nz = v > 0
    ev = np.where(nz, np.floor(np.log2(np.where(nz, v, 1.0))), -7.0)
    is_sub = ev < -6
    mant = np.where(is_sub, v / 2.0 ** -9, (v / np.exp2(ev) - 1.0) * 8.0)
    expo = np.where(is_sub, 0.0, ev + 7.0)
    bad = np.isnan(x) | (v > 448.0)
    expo = np.where(bad, 0.0, expo)
    mant = np.where(bad, 0.0, mant)
    code = (expo.astype(np.int64) << 3) | mant.astype(np.int64)
    code = np.where(v > 448.0, 0x7F, code)
    code = np.where(np.isnan(x), 0x7F, code)
    out = code.astype(np.uint8) | sign
    return out


E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=f32)


def e2m1_decode(code: np.ndarray) -> np.ndarray:
    code = np.asarray(code, dtype=np.uint8)
    mag = E2M1_VALUES[code & 7]
    return np.where(code & 8, -mag, mag).astype(f32)


def fake_quantize_to_e2m1(x: np.ndarray) -> np.ndarray:
    """Round onto +-{0,.5,1,1.5,2,3,4,6} (ties to even), value 8 possible for |x|>=7.

    fouroversix/src/fouroversix/quantize/pytorch/reference.py:13-34 (nearest style).
    Returns sign(x) * magnitude, so an input of -0.0 or one that rounds to zero gives
    +-0.0 with numpy's sign semantics matching torch's (sign(+-0) = +-0 ... times 0).
    """
    a = np.abs(x).astype(f32)
    step1 = (np.rint(f32(2) * a) / f32(2)).astype(f32)
    step2 = np.rint(a).astype(f32)
    step3 = (f32(2) * np.rint(a / f32(2))).astype(f32)
    mag = np.where(a < 2, step1, np.where(a < 4, step2, step3)).astype(f32)
    return (np.sign(x).astype(f32) * mag).astype(f32)


def e2m1_code_from_value(v: np.ndarray) -> np.ndarray:
    """4-bit code of an already-rounded value, through the bf16 bit tricks of the reference.

    fouroversix/src/fouroversix/quantize/pytorch/reference.py:37-63: sign<<3 | (exp-126)<<1 | mant,
    with zero -> exponent field 0 and 0.5 -> mantissa 1.  The value 8 (exp-126 = 4) overflows
    into bit 3 and yields code 0b1000 for either sign, exactly as the reference does.
    """
    bits = bf16_bits(v).astype(np.int32)
    s = (bits >> 15) & 1
    e = (bits >> 7) & 0xFF
    m = bits & 0x7F
    is_zero = (e == 0) & (m == 0)
    m = (m >> 6) & 1
    is_half = (e == 126) & (m == 0)
    m = np.where(is_half, 1, m)
    e = e - 126
    e = np.where(is_zero, 0, e)
    m = np.where(is_zero, 0, m)
    code = (s << 3) | (e << 1) | m
    return (code & 0xFF).astype(np.uint8)


# --------------------------------------------------------------------------------------
# scale-factor swizzle (128 x 4 atoms of 512 bytes)
# --------------------------------------------------------------------------------------

def swizzled_sf_offset(rows: int, cols: int) -> np.ndarray:
    """offset[r, c] into the flat swizzled scale array for a [rows, cols] scale matrix.

    fouroversix/src/fouroversix/quantize/utils.py:88-96 (``to_blocked``); identical to
    utils/kernel/kv_dequant_cuda.cu:41-57.
    """
    assert rows % 128 == 0 and cols % 4 == 0
    r = np.arange(rows, dtype=np.int64)[:, None]
    c = np.arange(cols, dtype=np.int64)[None, :]
    tile = (r // 128) * (cols // 4) + (c // 4)
    return tile * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + (c % 4)


def to_blocked(sf: np.ndarray) -> np.ndarray:
    off = swizzled_sf_offset(*sf.shape)
    out = np.empty(sf.size, dtype=sf.dtype)
    out[off.reshape(-1)] = sf.reshape(-1)
    return out


def from_blocked(flat: np.ndarray, shape: tuple[int, int]) -> np.ndarray:
    """fouroversix/src/fouroversix/quantize/quantized_tensor.py:10-18."""
    off = swizzled_sf_offset(*shape)
    return np.asarray(flat).reshape(-1)[off]


# --------------------------------------------------------------------------------------
# quantizer
# --------------------------------------------------------------------------------------

def padded_shape(shape: tuple[int, int]) -> tuple[int, int]:
    """Rows to a multiple of 128, columns to a multiple of 64.

    fouroversix/src/fouroversix/quantize/pytorch/backend.py:55-75,
    fouroversix/src/fouroversix/quantize/quantized_tensor.py:99-112.
    """
    m, k = shape
    return (m + (-m) % 128, k + (-k) % 64)


def _block_error_sum16(d: np.ndarray) -> np.ndarray:
    """Sum of 16 fp32 values per row in the order torch's CPU reduction uses.

    Verified against the reference's PyTorch backend in this build's container:
    ``t.sum(-1)`` over a contiguous [n, 16] fp32 tensor equals
    acc[i] = v[i] + v[i+8] (8 lanes), then ((((((acc0+acc1)+acc2)+acc3)+acc4)+acc5)+acc6)+acc7.
    """
    acc = (d[:, :8] + d[:, 8:]).astype(f32)
    e = acc[:, 0]
    for i in range(1, 8):
        e = (e + acc[:, i]).astype(f32)
    return e


def quantize_nvfp4(x: np.ndarray, rule: str = "mse", amax=None):
    """bf16-valued fp32 matrix [M, K] -> (codes u8 [Mp, Kp/2], swizzled scales u8 [Mp*Kp/16], amax f32).

    fouroversix/src/fouroversix/quantize/pytorch/reference.py:242-368 (nvfp4, 1-D blocks,
    round-to-nearest), including the padding its backend applies first
    (fouroversix/src/fouroversix/quantize/pytorch/backend.py:55-75).
    """
    x = np.asarray(x, dtype=f32)
    m, k = x.shape
    mp, kp = padded_shape((m, k))
    xp = np.zeros((mp, kp), dtype=f32)
    xp[:m, :k] = x
    xb = xp.reshape(-1, 16)
    if amax is None:
        amax = f32(np.abs(xb).max()) if xb.size else f32(0)     # reference.py:262-267
    amax = f32(amax)
    e2max, e4max = rule_limits(rule)
    nblk = xb.shape[0]

    bmax = np.abs(xb).max(axis=1).astype(f32)
    if amax == 0:                                                # reference.py:135-141
        hp = np.zeros(nblk, dtype=f32)
        enc = f32(np.inf)
    else:
        enc = f32(f32(e2max * e4max) / amax)                     # reference.py:142-151
        hp = ((bmax / f32(e2max)).astype(f32) * enc).astype(f32)

    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        dec = f32(f32(1) / f32(f32(e2max * e4max) / amax)) if amax != 0 else f32(0)   # reference.py:159-166

        def branch(expansion):
            h = hp if expansion is None else (hp * f32(expansion)).astype(f32)        # reference.py:154-155
            s_code = e4m3_encode(h)                                                   # reference.py:157
            s = e4m3_decode(s_code)
            inv = (f32(1) / (dec * s).astype(f32)).astype(f32)                        # reference.py:169
            xs = np.where(s[:, None] != 0, (xb * inv[:, None]).astype(f32), f32(0))   # reference.py:167-171
            return xs.astype(f32), s, s_code

        if rule in ("static_6", "static_4"):
            xs, s, s_code = branch(None)
            fq = fake_quantize_to_e2m1(xs)
        else:
            xs6, s6, c6 = branch(None)
            xs4, s4, c4 = branch(1.5)
            fq6 = fake_quantize_to_e2m1(xs6)
            fq4 = fake_quantize_to_e2m1(xs4)
            den = f32(E2M1_MAX * E4M3_MAX_FOUROVERSIX)                                # reference.py:196-215
            dq6 = (((fq6 * s6[:, None]).astype(f32) * amax).astype(f32) / den).astype(f32)
            dq4 = (((fq4 * s4[:, None]).astype(f32) * amax).astype(f32) / den).astype(f32)
            d6 = (dq6 - xb).astype(f32)
            d4 = (dq4 - xb).astype(f32)
            if rule == "abs_max":                                                     # reference.py:217-225
                e6 = np.abs(d6).max(axis=1)
                e4 = np.abs(d4).max(axis=1)
            elif rule == "mae":
                e6 = _block_error_sum16(np.abs(d6).astype(f32))
                e4 = _block_error_sum16(np.abs(d4).astype(f32))
            elif rule == "mse":
                e6 = _block_error_sum16((d6 * d6).astype(f32))
                e4 = _block_error_sum16((d4 * d4).astype(f32))
            else:
                raise ValueError(rule)
            sel4 = e4 < e6                                                            # reference.py:227
            fq = np.where(sel4[:, None], fq4, fq6)
            s_code = np.where(sel4, c4, c6)

    code = e2m1_code_from_value(bf16_round(fq)).reshape(mp, kp)                       # reference.py:351-353
    packed = ((code[:, 1::2] << 4) | code[:, 0::2]).astype(np.uint8)                  # reference.py:66-87
    sf = to_blocked(s_code.reshape(mp, kp // 16))                                     # reference.py:355-366
    return packed, sf, amax


def unpack_codes(packed: np.ndarray) -> np.ndarray:
    """[R, C/2] bytes -> [R, C] decoded fp32 values (low nibble = even column)."""
    lo = e2m1_decode(packed & 0xF)
    hi = e2m1_decode(packed >> 4)
    return np.stack([lo, hi], axis=-1).reshape(packed.shape[0], packed.shape[1] * 2)


# dequantize roundings that exist in the reference
DEQ_PYTORCH = 1      # ((v*s)*amax)/(e2*e4)             quantized_tensor.py:187-209
DEQ_FUSED_CUDA = 0   # (v*s)*(amax*fp32(1/(e2*e4)))     utils/kernel/kv_dequant_cuda.cu:95-101,216
DEQ_TRITON = 2       # (v*s)*(amax/(e2*e4))             utils/quant.py:756-766, utils/nvfp4_kernel.py:125-126


def dequantize(packed, sf_swizzled, amax, rule: str, original_shape, mode: int = DEQ_PYTORCH,
               out_bf16: bool = False) -> np.ndarray:
    """NVFP4 -> fp32 (or bf16-rounded fp32) matrix of ``original_shape``.

    mode selects which of the reference's three dequantize roundings is followed (see the
    DEQ_* constants); they can differ in the last bf16 bit.
    """
    mp, kh = packed.shape
    kp = kh * 2
    v = unpack_codes(packed)
    s = e4m3_decode(from_blocked(sf_swizzled, (mp, kp // 16)))
    vs = (v * np.repeat(s, 16, axis=1)).astype(f32)
    e2, e4 = rule_limits(rule)
    amax = f32(amax)
    if mode == DEQ_PYTORCH:
        r = ((vs * amax).astype(f32) / f32(e2 * e4)).astype(f32)
    elif mode == DEQ_FUSED_CUDA:
        g = f32(amax * f32(1.0 / (e2 * e4)))
        r = (vs * g).astype(f32)
    elif mode == DEQ_TRITON:
        g = f32(amax / f32(e2 * e4))
        r = (vs * g).astype(f32)
    else:
        raise ValueError(mode)
    if out_bf16:
        r = bf16_round(r)
    return r[: original_shape[0], : original_shape[1]]


def fp4_matmul(a_q, b_q, a_shape, b_shape, a_rule="mse", b_rule="mse", out_bf16=True) -> np.ndarray:
    """``a @ b.T`` of two NVFP4 tensors: dequantize both to fp32, fp32 matmul, round to bf16.

    fouroversix/src/fouroversix/matmul/pytorch.py:22-41.  ``a_q``/``b_q`` are the
    (codes, scales, amax) triples of :func:`quantize_nvfp4`.
    """
    a = dequantize(*a_q, a_rule, a_shape, DEQ_PYTORCH)
    b = dequantize(*b_q, b_rule, b_shape, DEQ_PYTORCH)
    out = a @ b.T
    return bf16_round(out) if out_bf16 else out.astype(f32)


def gemm_alpha(amax_a, amax_b, a_rule="mse", b_rule="mse") -> np.float32:
    """Per-GEMM fp32 scale of the block-scaled kernel.

    fouroversix/src/fouroversix/matmul/cutlass/backend.py:81-90.
    """
    e2a, e4a = rule_limits(a_rule)
    e2b, e4b = rule_limits(b_rule)
    return f32(f32(f32(amax_a) * f32(amax_b)) / f32(e2a * e4a * e2b * e4b))


def linear_forward(x, w_q, w_shape, bias=None, act_rule="mse", w_rule="mse") -> np.ndarray:
    """NVFP4 linear: quantize x, fp4 matmul, bf16 result, then ``out + bias`` in bf16.

    fouroversix/src/fouroversix/model/modules/linear.py:45-46, 67-74.
    """
    xq = quantize_nvfp4(x, act_rule)
    out = fp4_matmul(xq, w_q, x.shape, w_shape, act_rule, w_rule)
    if bias is not None:
        out = bf16_round((out + np.asarray(bias, dtype=f32)[None, :]).astype(f32))
    return out


# --------------------------------------------------------------------------------------
# KV-cache helpers
# --------------------------------------------------------------------------------------

def k_smooth(k: np.ndarray) -> np.ndarray:
    """``k - k.mean(-1, keepdim=True)`` in bf16 arithmetic.  utils/quant.py:797-798.

    torch's bf16 mean on CPU accumulates in fp32 and rounds the mean to bf16; the
    subtraction rounds to bf16 again.
    """
    k = np.asarray(k, dtype=f32)
    mean = bf16_round((k.sum(axis=-1, dtype=np.float64) / k.shape[-1]).astype(f32))
    return bf16_round((k - mean[..., None]).astype(f32))


def dequantize_kv_cache(blocks, num_heads: int, block_token_size: int, rule="mse",
                        mode: int = DEQ_FUSED_CUDA, dtype: str = "bf16") -> np.ndarray:
    """List of per-block (codes, scales, amax) -> [1, blocks*T, H, 128] fp32 array holding the values of
    the output dtype ("bf16", "fp16" or "fp32": the fp32 product rounded once to that type).

    utils/quant.py:731-768; the default rounding is that of the fused CUDA kernel the
    reference calls first (utils/kernel/kv_dequant_cuda.cu:59-107; output cast :216-240).
    """
    rows = num_heads * block_token_size
    outs = []
    for codes, sf, amax in blocks:
        d = dequantize(codes, sf, amax, rule, (rows, 128), mode, out_bf16=dtype == "bf16")
        if dtype == "fp16":
            d = d.astype(np.float16).astype(f32)
        elif dtype not in ("bf16", "fp32"):
            raise ValueError(dtype)
        outs.append(d.reshape(block_token_size, num_heads, 128))
    return np.concatenate(outs, axis=0)[None]


# --------------------------------------------------------------------------------------
# RoPE, norms, adaLN, attention
# --------------------------------------------------------------------------------------

def rope_tables(start_frame: int, frames: int, h: int, w: int, d: int = 128, theta: float = 10000.0,
                t_scale: float = 1.0, temporal_offset: float = 0.0):
    """cos/sin fp32 tables [frames*h*w, d/2] for tokens in (f, h, w) row-major order.

    wan_5b/modules/model.py:29-36 (``rope_params``), wan_5b/modules/causal_model.py:1075-1081
    (three tables of 1024 positions: d-4*(d//6), 2*(d//6), 2*(d//6) channels),
    wan_5b/modules/causal_model.py:156-165 (concatenation in (f,h,w) order) and
    utils/rope_triton.py:84-91 (fp64 angles -> fp32 cos/sin).  t_scale = 1, no offset.
    """
    c = d // 2
    dims = [d - 4 * (d // 6), 2 * (d // 6), 2 * (d // 6)]

    def angles(pos, dim):
        inv = 1.0 / np.power(theta, np.arange(0, dim, 2, dtype=np.float64) / dim)
        return np.outer(pos.astype(np.float64), inv)

    at = angles((np.arange(start_frame, start_frame + frames, dtype=np.float64) + float(temporal_offset)) * float(t_scale), dims[0])
    ah = angles(np.arange(h), dims[1])
    aw = angles(np.arange(w), dims[2])
    full = np.concatenate([
        np.broadcast_to(at[:, None, None, :], (frames, h, w, at.shape[1])),
        np.broadcast_to(ah[None, :, None, :], (frames, h, w, ah.shape[1])),
        np.broadcast_to(aw[None, None, :, :], (frames, h, w, aw.shape[1])),
    ], axis=-1).reshape(frames * h * w, c)
    return np.cos(full).astype(f32), np.sin(full).astype(f32)


def rope_apply(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """Interleaved-pair rotation in fp32, result rounded to bf16.  x: [S, H, D].

    utils/rope_triton.py:36-81: out_a = a*cos - b*sin, out_b = a*sin + b*cos.
    Each product and the sum are separate fp32 roundings (no FMA).
    """
    a = x[..., 0::2].astype(f32)
    b = x[..., 1::2].astype(f32)
    cs = cos[:, None, :]
    sn = sin[:, None, :]
    oa = ((a * cs).astype(f32) - (b * sn).astype(f32)).astype(f32)
    ob = ((a * sn).astype(f32) + (b * cs).astype(f32)).astype(f32)
    out = np.empty_like(x, dtype=f32)
    out[..., 0::2] = oa
    out[..., 1::2] = ob
    return bf16_round(out)


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float = 1e-6) -> np.ndarray:
    """WanRMSNorm over the last axis: fp32 normalise, round to bf16, times bf16 weight, round.

    wan_5b/modules/model.py:82-98.
    """
    xf = x.astype(f32)
    ms = (xf * xf).astype(f32).mean(axis=-1, keepdims=True, dtype=f32)
    y = bf16_round((xf * (f32(1) / np.sqrt((ms + f32(eps)).astype(f32))).astype(f32)).astype(f32))
    return bf16_round((y * weight.astype(f32)).astype(f32))


def adaln_modulate(x: np.ndarray, scale: np.ndarray, shift: np.ndarray, frame_seqlen: int,
                   eps: float = 1e-6) -> np.ndarray:
    """LayerNorm(no affine) -> bf16 -> *(bf16(1+scale)) -> bf16 -> +shift -> bf16.

    utils/adaln_triton.py:36-86.  x: [L, C]; scale/shift: [F, C] with F = L // frame_seqlen.
    """
    xf = x.astype(f32)
    c = xf.shape[-1]
    mean = (xf.sum(axis=-1, keepdims=True, dtype=np.float64) / c).astype(f32)
    xc = (xf - mean).astype(f32)
    var = ((xc * xc).astype(f32).sum(axis=-1, keepdims=True, dtype=np.float64) / c).astype(f32)
    rstd = (f32(1) / np.sqrt((var + f32(eps)).astype(f32))).astype(f32)
    xn = bf16_round((xc * rstd).astype(f32))
    frame = np.arange(xf.shape[0]) // frame_seqlen
    sc = bf16_round((scale.astype(f32)[frame] + f32(1)).astype(f32))
    prod = bf16_round((xn * sc).astype(f32))
    return bf16_round((prod + shift.astype(f32)[frame]).astype(f32))


def layer_norm_affine(x: np.ndarray, weight: np.ndarray, bias: np.ndarray, eps: float = 1e-6) -> np.ndarray:
    """nn.LayerNorm with elementwise affine on a bf16 tensor: fp32 statistics and affine, one
    rounding to bf16 at the end.  wan_5b/modules/model.py:101-111 (``WanLayerNorm`` with
    ``elementwise_affine=True``, the cross-attention ``norm3``)."""
    xf = x.astype(f32)
    c = xf.shape[-1]
    mean = (xf.sum(axis=-1, keepdims=True, dtype=np.float64) / c).astype(f32)
    xc = (xf - mean).astype(f32)
    var = ((xc * xc).astype(f32).sum(axis=-1, keepdims=True, dtype=np.float64) / c).astype(f32)
    rstd = (f32(1) / np.sqrt((var + f32(eps)).astype(f32))).astype(f32)
    return bf16_round(((xc * rstd).astype(f32) * weight.astype(f32) + bias.astype(f32)).astype(f32))


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray) -> np.ndarray:
    """softmax(q k^T / sqrt(D)) v per head, non-causal, fp32 math, bf16 result.

    q: [Lq, H, D]; k, v: [Lk, H, D].  wan_5b/modules/attention.py:291-306 (the SDPA form of
    the call at wan_5b/modules/causal_model.py:781).
    """
    lq, h, d = q.shape
    out = np.empty((lq, h, d), dtype=f32)
    scale = f32(1.0 / np.sqrt(d))
    for i in range(h):
        s = (q[:, i].astype(f32) @ k[:, i].astype(f32).T) * scale
        s = s - s.max(axis=1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(axis=1, keepdims=True)
        out[:, i] = p @ v[:, i].astype(f32)
    return bf16_round(out)


def window_attention(q_roped, k_new_roped, v_new, cache_k_blocks, cache_v_blocks, num_heads,
                     block_token_size, rule="mse", mode=DEQ_FUSED_CUDA):
    """Chunk attention over [dequantized cached blocks | current chunk].

    wan_5b/modules/causal_model.py:628-652, 673-724, 781: cached blocks are dequantized NVFP4
    (un-smoothed keys), the current chunk's keys are ``k_smooth``-ed bf16, values are used as
    they are; attention is non-causal over the concatenation.
    """
    parts_k, parts_v = [], []
    if cache_k_blocks:
        parts_k.append(dequantize_kv_cache(cache_k_blocks, num_heads, block_token_size, rule, mode)[0])
        parts_v.append(dequantize_kv_cache(cache_v_blocks, num_heads, block_token_size, rule, mode)[0])
    parts_k.append(k_smooth(k_new_roped))
    parts_v.append(np.asarray(v_new, dtype=f32))
    return attention(q_roped, np.concatenate(parts_k, 0), np.concatenate(parts_v, 0))
