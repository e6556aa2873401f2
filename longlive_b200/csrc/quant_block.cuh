// The NVFP4 block quantizer (one 16-element block -> 8 code bytes + one E4M3 scale, "four over six" scale
// selection), bit-exact against the reference's PyTorch quantizer
// (fouroversix/src/fouroversix/quantize/pytorch/reference.py:242-368).  Shared by the standalone quantizer
// (quantize.cu) and the GEMM epilogue that requantizes its output (gemm_nvfp4.cu).  The arithmetic notes at the
// top of quantize.cu apply to everything here.
#pragma once

#include <cuda_fp4.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace llnv {
namespace quant {

// ---- exact division by a constant -------------------------------------------------------------
template <int D>
__device__ __forceinline__ float div_const(float x) {
  constexpr float d = (float)D;
  constexpr float r = 1.0f / d;                    // correctly rounded at compile time
  const float q = __fmul_rn(x, r);
  const float rem = __fmaf_rn(-d, q, x);
  return __fmaf_rn(rem, r, q);
}

template <int D>
__device__ __forceinline__ F2 div_const2(F2 x) {
  constexpr float d = (float)D;
  constexpr float r = 1.0f / d;
  const F2 q = f2_mul(x, f2_splat(r));
  const F2 rem = f2_fma(f2_splat(-d), q, x);
  return f2_fma(rem, f2_splat(r), q);
}

// ---- hardware conversions ---------------------------------------------------------------------
// two fp32 -> two E2M1 codes (lo in bits 0-3, hi in bits 4-7), round to nearest even, saturating
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
  return (uint32_t)__nv_cvt_float2_to_fp4x2(make_float2(lo, hi), __NV_E2M1, cudaRoundNearest);
}
// two E2M1 codes -> two fp32 (x = low nibble)
__device__ __forceinline__ float2 e2m1x2_to_float2(uint32_t byte) {
  const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)byte, __NV_E2M1);
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}
// two fp32 -> two E4M3 bytes (lo in bits 0-7), round to nearest even, saturating
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
  return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float2 e4m3x2_to_float2(uint32_t two) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)two, __NV_E4M3);
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

// ---- reference-faithful scalar pieces (slow path) ---------------------------------------------
// Round |xs| onto {0,.5,1,1.5,2,3,4,6,(8)} with ties to even (reference.py:13-34).
__device__ __forceinline__ float e2m1_round_mag(float a) {
  const float k = a < 2.f ? 2.f : (a < 4.f ? 1.f : 0.5f);
  const float kinv = a < 2.f ? 0.5f : (a < 4.f ? 1.f : 2.f);
  return __fmul_rn(rintf(__fmul_rn(a, k)), kinv);
}
// 4-bit code of a rounded magnitude with the sign of xs (reference.py:37-63); magnitude 8 -> 0b1000
__device__ __forceinline__ uint32_t e2m1_code(float mag, bool neg) {
  const int t = (int)(mag * 2.f);               // 0,1,2,3,4,6,8,12,16
  const uint32_t idx = t < 4 ? (uint32_t)t : (t == 4 ? 4u : (t == 6 ? 5u : (t == 8 ? 6u : (t == 12 ? 7u : 8u))));
  return idx == 8u ? 8u : (idx | (neg ? 8u : 0u));
}

template <int RULE>
__device__ __forceinline__ float err_term(float d) {
  if (RULE == LLNV_RULE_MSE) return __fmul_rn(d, d);
  return fabsf(d);
}

struct QuantConsts {
  float amax, enc, dec;
  bool fast;       // amax has <= 8 significant bits and is large enough that no error term is denormal
};

// Slow path for one candidate scale: the reference's arithmetic operation by operation.
template <int RULE>
__device__ __noinline__ void candidate_slow(const float (&x)[16], float s, float inv, float amax, uint32_t& lo, uint32_t& hi,
                                            float& err) {
  lo = hi = 0u;
  err = 0.f;
#pragma unroll 1
  for (int i = 0; i < 8; ++i) {
    float t[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float xv = x[i + 8 * h];
      const float xs = s != 0.f ? __fmul_rn(xv, inv) : 0.f;
      const float m = e2m1_round_mag(fabsf(xs));
      const uint32_t c = e2m1_code(m, xs < 0.f) << (4 * i);
      if (h == 0) lo |= c; else hi |= c;
      const float q = xs < 0.f ? -m : m;
      const float d = __fsub_rn(__fdiv_rn(__fmul_rn(__fmul_rn(q, s), amax), 1536.f), xv);
      t[h] = err_term<RULE>(d);
    }
    if (RULE == LLNV_RULE_ABS_MAX) err = fmaxf(err, fmaxf(t[0], t[1]));
    else {
      const float a = __fadd_rn(t[0], t[1]);
      err = i == 0 ? a : __fadd_rn(err, a);
    }
  }
}

// The reference's arithmetic on 16 fp32 values (whatever type they were loaded from), operation by operation.
template <int RULE>
__device__ __forceinline__ void quant_block_slow_f(const float (&x)[16], const QuantConsts& qc, float hp, uint32_t& c_lo,
                                                   uint32_t& c_hi, uint32_t& sf_out) {
  const uint32_t sc6 = float_to_e4m3(hp);
  const float s6 = e4m3_to_float(sc6);
  const float inv6 = s6 != 0.f ? __fdiv_rn(1.f, __fmul_rn(qc.dec, s6)) : 0.f;
  uint32_t l6, h6;
  float e6;
  candidate_slow<RULE>(x, s6, inv6, qc.amax, l6, h6, e6);
  if (RULE == LLNV_RULE_STATIC_6 || RULE == LLNV_RULE_STATIC_4) {
    c_lo = l6; c_hi = h6; sf_out = sc6;
    return;
  }
  const uint32_t sc4 = float_to_e4m3(__fmul_rn(hp, 1.5f));
  const float s4 = e4m3_to_float(sc4);
  const float inv4 = s4 != 0.f ? __fdiv_rn(1.f, __fmul_rn(qc.dec, s4)) : 0.f;
  uint32_t l4, h4;
  float e4;
  candidate_slow<RULE>(x, s4, inv4, qc.amax, l4, h4, e4);
  const bool sel4 = e4 < e6;
  c_lo = sel4 ? l4 : l6;
  c_hi = sel4 ? h4 : h6;
  sf_out = sel4 ? sc4 : sc6;
}

// x[16] is indexed with run-time i in candidate_slow: keep it out of the fast path's registers
template <int RULE>
__device__ __noinline__ void quant_block_slow(const uint32_t (&w)[8], const QuantConsts& qc, float hp, uint32_t& c_lo,
                                              uint32_t& c_hi, uint32_t& sf_out) {
  float x[16];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    x[2 * j] = bf16_lo(w[j]);
    x[2 * j + 1] = bf16_hi(w[j]);
  }
  quant_block_slow_f<RULE>(x, qc, hp, c_lo, c_hi, sf_out);
}

// One 16-element block of fp16 input (w: 8 words of packed halves): the values go through the reference's arithmetic as
// fp32, one operation at a time (the packed fast path below relies on bf16 inputs: a tensor amax of at most 8 significant
// bits makes several of its products exact, which an fp16 tensor does not give).  The reference's CUDA backend takes
// fp16 activations as well as bf16 (fouroversix/src/fouroversix/quantize/cuda/backend.py:45-51).
template <int RULE>
__device__ __noinline__ void quant_block_f16(const uint32_t (&w)[8], const QuantConsts& qc, uint32_t& c_lo, uint32_t& c_hi,
                                             uint32_t& sf_out) {
  float x[16];
  float bmax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
    x[2 * j] = f.x;
    x[2 * j + 1] = f.y;
    bmax = fmaxf(bmax, fmaxf(fabsf(f.x), fabsf(f.y)));
  }
  if (bmax == 0.f || qc.amax == 0.f) { c_lo = c_hi = 0u; sf_out = 0u; return; }
  const float hp = RULE == LLNV_RULE_STATIC_4 ? __fmul_rn(__fmul_rn(bmax, 0.25f), qc.enc) : __fmul_rn(__fdiv_rn(bmax, 6.f), qc.enc);
  quant_block_slow_f<RULE>(x, qc, hp, c_lo, c_hi, sf_out);
}

// One 16-element block.  w: 8 words of packed bf16 (element 2j in the low half of w[j]).
// Output: c_lo = codes of elements 0..7 (nibble j), c_hi = codes of elements 8..15, sf byte.
template <int RULE>
__device__ __forceinline__ void quant_block(const uint32_t (&w)[8], const QuantConsts& qc, uint32_t& c_lo, uint32_t& c_hi,
                                            uint32_t& sf_out) {
  constexpr bool kStatic = (RULE == LLNV_RULE_STATIC_6 || RULE == LLNV_RULE_STATIC_4);
  // block maximum on the packed 15-bit magnitudes
  uint32_t m = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) m = __vmaxu2(m, w[j] & 0x7FFF7FFFu);
  const float bmax = __uint_as_float(max(m & 0xFFFFu, m >> 16) << 16);
  float hp;
  if (qc.amax == 0.f) hp = 0.f;
  else if (RULE == LLNV_RULE_STATIC_4) hp = __fmul_rn(__fmul_rn(bmax, 0.25f), qc.enc);
  else hp = __fmul_rn(qc.fast ? div_const<6>(bmax) : __fdiv_rn(bmax, 6.f), qc.enc);

  // Slow path: the corner cases listed in the file header.  2^-100 keeps every quotient, product
  // and error term of the fast path far from the denormal range.
  const float xs_max = __fmul_rn(bmax, __frcp_rn(__fmul_rn(qc.dec, e4m3_to_float(float_to_e4m3(hp)))));
  if (!qc.fast || !(xs_max < 6.75f) || bmax < 1.0e-28f) {
    if (bmax == 0.f) { c_lo = c_hi = 0u; sf_out = 0u; return; }
    quant_block_slow<RULE>(w, qc, hp, c_lo, c_hi, sf_out);
    return;
  }

  const uint32_t sc = cvt_e4m3x2(hp, kStatic ? 0.f : __fmul_rn(hp, 1.5f));       // byte 0: 6-scale, byte 1: 4-scale
  const float2 sv = e4m3x2_to_float2(sc);
  const float s6 = sv.x, s4 = sv.y;
  const float inv6 = __frcp_rn(__fmul_rn(qc.dec, s6));                             // s6 != 0 here (xs_max finite)
  if (kStatic) {
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      lo |= cvt_e2m1x2(__fmaf_rn(bf16_lo(w[j]), inv6, 0.f), __fmaf_rn(bf16_hi(w[j]), inv6, 0.f)) << (8 * j);
      hi |= cvt_e2m1x2(__fmaf_rn(bf16_lo(w[j + 4]), inv6, 0.f), __fmaf_rn(bf16_hi(w[j + 4]), inv6, 0.f)) << (8 * j);
    }
    c_lo = lo; c_hi = hi; sf_out = sc & 0xFFu;
    return;
  }
  const float inv4 = __frcp_rn(__fmul_rn(qc.dec, s4));
  const float sa6 = __fmul_rn(s6, qc.amax), sa4 = __fmul_rn(s4, qc.amax);        // exact (4 + 8 significant bits)
  uint32_t pa[4], pb[4];
  float e6 = 0.f, e4 = 0.f;
  // pair j holds elements (2j, 2j+1) in w[j] and (2j+8, 2j+9) in w[j+4]; the error sum adds
  // element i to element i+8 first, then the eight lane sums left to right
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const F2 xa = {bf16_lo(w[j]), bf16_hi(w[j])};                    // elements 2j, 2j+1
    const F2 xb = {bf16_lo(w[j + 4]), bf16_hi(w[j + 4])};            // elements 2j+8, 2j+9
    // the +0 addend turns a -0 product (input -0.0) into +0, as the reference's sign(x)*|.| does
    const F2 zero = f2_splat(0.f);
    const F2 sa6v = f2_fma(xa, f2_splat(inv6), zero), sb6v = f2_fma(xb, f2_splat(inv6), zero);
    const F2 sa4v = f2_fma(xa, f2_splat(inv4), zero), sb4v = f2_fma(xb, f2_splat(inv4), zero);
    const uint32_t ca6 = cvt_e2m1x2(sa6v.x, sa6v.y);
    const uint32_t cb6 = cvt_e2m1x2(sb6v.x, sb6v.y);
    const uint32_t ca4 = cvt_e2m1x2(sa4v.x, sa4v.y);
    const uint32_t cb4 = cvt_e2m1x2(sb4v.x, sb4v.y);
    // candidate-6 and candidate-4 code bytes of this pair side by side; the selected ones are gathered at the end
    pa[j] = __byte_perm(ca6, ca4, 0x0040);
    pb[j] = __byte_perm(cb6, cb4, 0x0040);
    const float2 qa6 = e2m1x2_to_float2(ca6), qb6 = e2m1x2_to_float2(cb6);
    const float2 qa4 = e2m1x2_to_float2(ca4), qb4 = e2m1x2_to_float2(cb4);
    // dequantized candidates minus x, two elements per packed instruction (every lane rounds as the scalar op does)
    const F2 da6 = f2_sub(div_const2<1536>(f2_mul(F2{qa6.x, qa6.y}, f2_splat(sa6))), xa);
    const F2 db6 = f2_sub(div_const2<1536>(f2_mul(F2{qb6.x, qb6.y}, f2_splat(sa6))), xb);
    const F2 da4 = f2_sub(div_const2<1536>(f2_mul(F2{qa4.x, qa4.y}, f2_splat(sa4))), xa);
    const F2 db4 = f2_sub(div_const2<1536>(f2_mul(F2{qb4.x, qb4.y}, f2_splat(sa4))), xb);
    if (RULE == LLNV_RULE_MSE) {
      // lanes 2j and 2j+1 of the 8-lane partial sums: element i plus element i+8
      const F2 l6 = f2_add(f2_mul(da6, da6), f2_mul(db6, db6));
      const F2 l4 = f2_add(f2_mul(da4, da4), f2_mul(db4, db4));
      // running sums of both candidates side by side: (e6, e4) + lane 2j, then + lane 2j+1
      if (j == 0) {
        const F2 e = f2_add(F2{l6.x, l4.x}, F2{l6.y, l4.y});
        e6 = e.x; e4 = e.y;
      } else {
        const F2 e = f2_add(f2_add(F2{e6, e4}, F2{l6.x, l4.x}), F2{l6.y, l4.y});
        e6 = e.x; e4 = e.y;
      }
    } else {
      const float t6a0 = fabsf(da6.x), t6a1 = fabsf(da6.y), t6b0 = fabsf(db6.x), t6b1 = fabsf(db6.y);
      const float t4a0 = fabsf(da4.x), t4a1 = fabsf(da4.y), t4b0 = fabsf(db4.x), t4b1 = fabsf(db4.y);
      if (RULE == LLNV_RULE_ABS_MAX) {
        e6 = fmaxf(fmaxf(e6, fmaxf(t6a0, t6b0)), fmaxf(t6a1, t6b1));
        e4 = fmaxf(fmaxf(e4, fmaxf(t4a0, t4b0)), fmaxf(t4a1, t4b1));
      } else {
        const float l6a = __fadd_rn(t6a0, t6b0), l6b = __fadd_rn(t6a1, t6b1);   // lanes 2j and 2j+1
        const float l4a = __fadd_rn(t4a0, t4b0), l4b = __fadd_rn(t4a1, t4b1);
        e6 = j == 0 ? __fadd_rn(l6a, l6b) : __fadd_rn(__fadd_rn(e6, l6a), l6b);
        e4 = j == 0 ? __fadd_rn(l4a, l4b) : __fadd_rn(__fadd_rn(e4, l4a), l4b);
      }
    }
  }
  const bool sel4 = e4 < e6;
  // bytes (c6_0, c4_0, c6_1, c4_1) | (c6_2, c4_2, c6_3, c4_3): one permute picks the even (6) or the odd (4) bytes
  const uint32_t pick = sel4 ? 0x7531u : 0x6420u;
  c_lo = __byte_perm(__byte_perm(pa[0], pa[1], 0x5410), __byte_perm(pa[2], pa[3], 0x5410), pick);
  c_hi = __byte_perm(__byte_perm(pb[0], pb[1], 0x5410), __byte_perm(pb[2], pb[3], 0x5410), pick);
  sf_out = sel4 ? (sc >> 8) : (sc & 0xFFu);
}

// Constants of a tensor with the given amax (reference.py:142-166).
template <int RULE>
__device__ __forceinline__ QuantConsts make_consts(float amax) {
  constexpr float kE2 = RULE == LLNV_RULE_STATIC_4 ? 4.f : 6.f;
  constexpr float kE4 = (RULE == LLNV_RULE_STATIC_6 || RULE == LLNV_RULE_STATIC_4) ? 448.f : 256.f;
  QuantConsts qc;
  qc.amax = amax;
  qc.enc = __fdiv_rn(kE2 * kE4, qc.amax);     // reference.py:142-151
  qc.dec = __fdiv_rn(1.f, qc.enc);            // reference.py:159-166
  qc.fast = (__float_as_uint(qc.amax) & 0xFFFFu) == 0u && qc.amax > 1.0e-20f && qc.amax < 1.0e30f;
  return qc;
}

}  // namespace quant
}  // namespace llnv
