// bf16 -> NVFP4 quantizer (E2M1 codes, E4M3 scale per 16 elements, fp32 tensor scale, the
// "four over six" scale selection), bit-exact against the reference's PyTorch quantizer
// (fouroversix/src/fouroversix/quantize/pytorch/reference.py:242-368), optionally with the
// adaLN modulation (LayerNorm -> (1 + scale) * x + shift) or an affine LayerNorm applied on load
// so that the normalised activation never round-trips through memory.
//
// Layout of one CTA: 128 rows x 128 columns of the input, 256 threads.  Thread t owns the
// 16-element block (row = t/8 + 32*i, column block = t%8) for i = 0..3, so
//   * a warp reads 4 rows x 256 contiguous bytes per i with 128-bit loads,
//   * the 4 scale bytes of a thread land in one 16-byte unit of the 128x4 swizzled scale atom;
//     four neighbouring lanes transpose their bytes with warp shuffles and store whole words,
//     so every 512-byte scale atom is written densely by one CTA.
// The four blocks are processed in a rolled loop (next block prefetched) to keep the code small
// enough for the instruction cache.
//
// Arithmetic notes (all needed for bit-exactness of the 4-vs-6 decision, which compares two
// rounded 16-term sums):
//   * every fp32 operation uses an explicit round-to-nearest intrinsic, so nothing is contracted
//     into an FMA unless written as one;
//   * x / 6 and x / 1536 use q = x*r; q += fma(-d, q, x) * r with r = RN(1/d): for these divisors
//     the result equals the IEEE quotient for every finite fp32 x outside the denormal range
//     (checked exhaustively on the device by tests/test_gpu_quantize.py::test_exact_division);
//     blocks whose values could reach the denormal range take the IEEE-division path;
//   * codes come from the hardware conversion cvt.rn.satfinite.e2m1x2.f32.  The reference differs
//     from it in two corner cases that are reproduced: a scaled value of magnitude >= 7 (possible
//     only when the block scale is a tiny subnormal) yields code 0b1000 through the reference's
//     exponent arithmetic (reference.py:37-63), and an input of -0.0 yields code 0 (sign(x) * |.|);
//   * when the tensor amax has at most 8 significant bits (always true when it is the maximum of
//     bf16 values) (q*s)*amax is exact, so it is formed as q*(s*amax).
#include <cuda_fp4.h>

#include "common.cuh"

namespace llnv {

namespace {

// ---- tensor amax ----------------------------------------------------------------------------
__global__ void __launch_bounds__(256) amax_bf16_kernel(const uint16_t* __restrict__ x, int64_t M, int64_t K,
                                                        int64_t ldx, float* __restrict__ amax) {
  pdl_wait();
  const int64_t vec_per_row = K >> 3;
  const int64_t total = M * vec_per_row;
  uint32_t m = 0;   // two 15-bit magnitudes, compared as unsigned 16-bit lanes
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / vec_per_row, c = i - r * vec_per_row;
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + r * ldx + c * 8));
    m = __vmaxu2(m, v.x & 0x7FFF7FFFu);
    m = __vmaxu2(m, v.y & 0x7FFF7FFFu);
    m = __vmaxu2(m, v.z & 0x7FFF7FFFu);
    m = __vmaxu2(m, v.w & 0x7FFF7FFFu);
  }
  uint32_t mm = max(m & 0xFFFFu, m >> 16);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mm = max(mm, __shfl_xor_sync(0xFFFFFFFFu, mm, o));
  __shared__ uint32_t s[8];
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = mm;
  __syncthreads();
  if (threadIdx.x < 32) {
    mm = threadIdx.x < (blockDim.x >> 5) ? s[threadIdx.x] : 0u;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) mm = max(mm, __shfl_xor_sync(0xFFFFFFFFu, mm, o));
    if (threadIdx.x == 0 && mm != 0) atomicMax(reinterpret_cast<int*>(amax), (int)(mm << 16));
  }
}

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
  // regroup so that x[i] / x[i+8] pair up as in the error sum: element order is preserved
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
  uint32_t lo6 = 0, hi6 = 0, lo4 = 0, hi4 = 0;
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
    lo6 |= ca6 << (8 * j); hi6 |= cb6 << (8 * j);
    lo4 |= ca4 << (8 * j); hi4 |= cb4 << (8 * j);
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
  c_lo = sel4 ? lo4 : lo6;
  c_hi = sel4 ? hi4 : hi6;
  sf_out = sel4 ? (sc >> 8) : (sc & 0xFFu);
}

// ---- load-side transforms -----------------------------------------------------------------------
enum { kPlain = 0, kAdaLN = 1, kAffineLN = 2 };

struct Prologue {
  // kAdaLN:    y = bf16(bf16(bf16((x-mean)*rstd) * bf16(1 + scale[f])) + shift[f])   (utils/adaln_triton.py:62-86)
  // kAffineLN: y = bf16(((x-mean)*rstd) * weight + bias)                              (nn.LayerNorm with affine)
  const float* row_stats;      // [M][2] = mean, rstd
  const uint16_t* p0;          // scale [frames, stride] or weight [C]
  const uint16_t* p1;          // shift [frames, stride] or bias [C]
  int64_t stride;
  int frame_rows;
  int add_one;
  int64_t row_offset;          // added to the row index before the frame lookup (token shards)
  // column-sharded input (kPlain): x is [K / shard_cols][M][shard_cols] with row stride ldx inside a
  // shard and shard_stride elements between shards (the receive layout of the head -> token
  // exchange of sequence parallelism); 0 = one plain [M][K] matrix
  int64_t shard_cols, shard_stride;
  // second tensor of the same shape handled by the same launch (blockIdx.z == 1), e.g. the K and
  // the V block of a KV-cache write; nullptr = none
  const uint16_t* x2;
  const float* amax2;
  uint8_t* codes2;
  uint8_t* sf2;
};

template <int MODE>
__device__ __forceinline__ void transform_block(uint32_t (&w)[8], const Prologue& pr, int64_t row, int64_t col) {
  if (MODE == kPlain) return;
  const float mean = __ldg(pr.row_stats + 2 * row), rstd = __ldg(pr.row_stats + 2 * row + 1);
  const int64_t prow = MODE == kAdaLN ? ((row + pr.row_offset) / pr.frame_rows) * pr.stride : 0;
  const uint4* a4 = reinterpret_cast<const uint4*>(pr.p0 + prow + col);
  const uint4* b4 = reinterpret_cast<const uint4*>(pr.p1 + prow + col);
  const uint4 a0 = __ldg(a4), a1 = __ldg(a4 + 1), b0 = __ldg(b4), b1 = __ldg(b4 + 1);
  const uint32_t aw[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
  const uint32_t bw[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float y[2];
    const float a0f = bf16_lo(aw[j]), a1f = bf16_hi(aw[j]);
    const float b0f = bf16_lo(bw[j]), b1f = bf16_hi(bw[j]);
    float xn0 = __fmul_rn(__fsub_rn(bf16_lo(w[j]), mean), rstd);
    float xn1 = __fmul_rn(__fsub_rn(bf16_hi(w[j]), mean), rstd);
    if (MODE == kAdaLN) {
      float s0 = a0f, s1 = a1f;
      if (pr.add_one) {
        s0 = __fadd_rn(a0f, 1.f);
        s1 = __fadd_rn(a1f, 1.f);
        round_bf16x2(s0, s1);
      }
      round_bf16x2(xn0, xn1);
      float m0 = __fmul_rn(xn0, s0), m1 = __fmul_rn(xn1, s1);
      round_bf16x2(m0, m1);
      y[0] = __fadd_rn(m0, b0f);
      y[1] = __fadd_rn(m1, b1f);
    } else {
      y[0] = __fmaf_rn(xn0, a0f, b0f);
      y[1] = __fmaf_rn(xn1, a1f, b1f);
    }
    w[j] = pack_bf16x2(y[0], y[1]);
  }
}

template <int RULE, int MODE>
__global__ void __launch_bounds__(256) quantize_nvfp4_kernel(const uint16_t* x, int64_t M, int64_t K,
                                                             int64_t ldx, const float* amax_ptr,
                                                             uint8_t* codes, uint8_t* sf,
                                                             const Prologue pr, uint16_t* __restrict__ y_out, int64_t ldy) {
  pdl_wait();
  if (blockIdx.z == 1) {          // second tensor of a two-tensor launch
    x = pr.x2;
    amax_ptr = pr.amax2;
    codes = pr.codes2;
    sf = pr.sf2;
  }
  constexpr float kE2 = RULE == LLNV_RULE_STATIC_4 ? 4.f : 6.f;
  constexpr float kE4 = (RULE == LLNV_RULE_STATIC_6 || RULE == LLNV_RULE_STATIC_4) ? 448.f : 256.f;
  QuantConsts qc;
  qc.amax = *amax_ptr;
  qc.enc = __fdiv_rn(kE2 * kE4, qc.amax);     // reference.py:142-151
  qc.dec = __fdiv_rn(1.f, qc.enc);            // reference.py:159-166
  qc.fast = (__float_as_uint(qc.amax) & 0xFFFFu) == 0u && qc.amax > 1.0e-20f && qc.amax < 1.0e30f;

  // 256 threads cover 128 x 128 elements, 128 threads 128 x 64 (one scale atom): the narrower CTA
  // is launched for small tensors, whose few wide CTAs would spread unevenly over the SMs
  const int t = threadIdx.x;
  const int cshift = blockDim.x == 256 ? 3 : 2;
  const int cb = t & ((1 << cshift) - 1);
  const int r0 = t >> cshift;
  const int64_t col = (int64_t)blockIdx.x * (16 << cshift) + cb * 16;
  const int64_t row_base = (int64_t)blockIdx.y * 128;
  const bool col_ok = col < K;
  const int64_t xoff = pr.shard_cols ? (col / pr.shard_cols) * pr.shard_stride + col % pr.shard_cols : col;

  auto load_block = [&](int i, uint32_t (&w)[8]) {
    const int64_t r = row_base + r0 + 32 * i;
    if (col_ok && r < M) {
      const uint4* p = reinterpret_cast<const uint4*>(x + r * ldx + xoff);
      const uint4 a = __ldg(p), b = __ldg(p + 1);
      w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
      w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) w[j] = 0u;
    }
  };

  uint32_t nxt[8];
  load_block(0, nxt);
  uint32_t my_sf = 0;
#pragma unroll 1
  for (int i = 0; i < 4; ++i) {
    uint32_t cur[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) cur[j] = nxt[j];
    if (i < 3) load_block(i + 1, nxt);
    const int64_t r = row_base + r0 + 32 * i;
    if (MODE != kPlain && col_ok && r < M) {
      transform_block<MODE>(cur, pr, r, col);
      if (y_out) {
        uint4* yo = reinterpret_cast<uint4*>(y_out + r * ldy + col);
        yo[0] = make_uint4(cur[0], cur[1], cur[2], cur[3]);
        yo[1] = make_uint4(cur[4], cur[5], cur[6], cur[7]);
      }
    }
    uint32_t c_lo, c_hi, s;
    quant_block<RULE>(cur, qc, c_lo, c_hi, s);
    if (col_ok) *reinterpret_cast<uint2*>(codes + r * (K >> 1) + (col >> 1)) = make_uint2(c_lo, c_hi);
    my_sf |= s << (8 * i);
  }

  // Transpose the 4x4 scale bytes of each group of four lanes: lane q ends up with the word of
  // 16-byte unit r0 that holds row (r0 + 32*q), scale columns 4*(cb/4) .. +3.
  const int lane = t & 31;
  const int q = lane & 3;
  const int gbase = lane & ~3;
  uint32_t word = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t other = __shfl_sync(0xFFFFFFFFu, my_sf, gbase + j);
    word |= ((other >> (8 * q)) & 0xFFu) << (8 * j);
  }
  if (col_ok) {
    const int64_t sc = col >> 4;                                   // global scale column
    const int64_t atom = (int64_t)blockIdx.y * (K >> 6) + (sc >> 2);
    *reinterpret_cast<uint32_t*>(sf + atom * 512 + r0 * 16 + q * 4) = word;
  }
}

// ---- row statistics + amax of the transformed activation ----------------------------------------
// One warp per row: mean and rstd in fp32 (two-pass over registers), then the row's transformed
// values are formed once to find max|y|; nothing but the 8-byte statistics is stored.
// WPR warps share one row (each takes C / WPR channels): with one warp per row a chunk of 2640
// tokens is only 2640 warps and the kernel is bound by the latency of each warp's dependent steps.
template <int MODE, int WPR>
__global__ void __launch_bounds__(256) ln_stats_amax_kernel(const uint16_t* __restrict__ x, int64_t M, int64_t C, int64_t ldx,
                                                            float eps, Prologue pr, float* __restrict__ row_stats,
                                                            float* __restrict__ amax) {
  pdl_wait();
  constexpr int kVec = 16 / WPR;              // 16-byte vectors per lane: C <= 4096
  constexpr int kRows = 8 / WPR;              // rows per CTA
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int part = warp % WPR;
  const int64_t row = (int64_t)blockIdx.x * kRows + warp / WPR;
  // The modulation / affine vectors are shared by the rows of a CTA (consecutive rows touch at
  // most two frames): stage them in shared memory once instead of loading them, dependently, in
  // every step of the per-row loop.
  __shared__ uint4 pa_sh[2][4096 / 8];
  __shared__ uint4 pb_sh[2][4096 / 8];
  __shared__ float red_sh[2][8];
  const int nvec_all = (int)(C >> 3);
  const int pvec = nvec_all / WPR;            // vectors of this warp's part
  const int vbase = part * pvec;
  const int64_t first_row = (int64_t)blockIdx.x * kRows;
  const int64_t last_row = min(first_row + kRows - 1, M - 1);
  const int64_t f0 = MODE == kAdaLN ? (first_row + pr.row_offset) / pr.frame_rows : 0;
  const int64_t f1 = MODE == kAdaLN ? (last_row + pr.row_offset) / pr.frame_rows : 0;
  // (with several warps per row a CTA has too few rows to amortise the staging: each lane then
  // fetches its few vectors of the two parameter rows itself, together with x)
  if (WPR == 1) {
    for (int i = threadIdx.x; i < nvec_all; i += blockDim.x) {
      pa_sh[0][i] = __ldg(reinterpret_cast<const uint4*>(pr.p0 + f0 * pr.stride) + i);
      pb_sh[0][i] = __ldg(reinterpret_cast<const uint4*>(pr.p1 + f0 * pr.stride) + i);
      if (f1 != f0) {
        pa_sh[1][i] = __ldg(reinterpret_cast<const uint4*>(pr.p0 + f1 * pr.stride) + i);
        pb_sh[1][i] = __ldg(reinterpret_cast<const uint4*>(pr.p1 + f1 * pr.stride) + i);
      }
    }
  }
  const bool live = row < M;
  uint4 v[kVec], pa[kVec], pb[kVec];
  float sum = 0.f;
  if (live) {
    const int64_t prow = MODE == kAdaLN ? ((row + pr.row_offset) / pr.frame_rows) * pr.stride : 0;
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const int li = lane + 32 * i;
      if (li < pvec) {
        v[i] = __ldg(reinterpret_cast<const uint4*>(x + row * ldx) + vbase + li);
        if (WPR > 1) {
          pa[i] = __ldg(reinterpret_cast<const uint4*>(pr.p0 + prow) + vbase + li);
          pb[i] = __ldg(reinterpret_cast<const uint4*>(pr.p1 + prow) + vbase + li);
        }
        sum += bf16_lo(v[i].x) + bf16_hi(v[i].x) + bf16_lo(v[i].y) + bf16_hi(v[i].y) + bf16_lo(v[i].z) + bf16_hi(v[i].z) +
               bf16_lo(v[i].w) + bf16_hi(v[i].w);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
  if (lane == 0) red_sh[0][warp] = sum;
  __syncthreads();                            // vectors staged, partial sums published
  float tot = red_sh[0][warp - part];
#pragma unroll
  for (int k = 1; k < WPR; ++k) tot += red_sh[0][warp - part + k];
  const float mean = tot / (float)C;
  float sq = 0.f;
  if (live) {
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      if (lane + 32 * i < pvec) {
        const uint32_t ws[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a = bf16_lo(ws[j]) - mean, b = bf16_hi(ws[j]) - mean;
          sq += a * a + b * b;
        }
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xFFFFFFFFu, sq, o);
  if (lane == 0) red_sh[1][warp] = sq;
  __syncthreads();
  float sqt = red_sh[1][warp - part];
#pragma unroll
  for (int k = 1; k < WPR; ++k) sqt += red_sh[1][warp - part + k];
  const float rstd = 1.0f / sqrtf(sqt / (float)C + eps);
  float wmax = 0.f;
  if (live) {
    if (lane == 0 && part == 0) {
      row_stats[2 * row] = mean;
      row_stats[2 * row + 1] = rstd;
    }
    const int fsel = (MODE == kAdaLN && (row + pr.row_offset) / pr.frame_rows != f0) ? 1 : 0;
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const int li = lane + 32 * i;
      if (li < pvec) {
        const int idx = vbase + li;
        const uint4 a4 = WPR > 1 ? pa[i] : pa_sh[fsel][idx];
        const uint4 b4 = WPR > 1 ? pb[i] : pb_sh[fsel][idx];
        const uint32_t ws[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
        const uint32_t aw[4] = {a4.x, a4.y, a4.z, a4.w};
        const uint32_t bw[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a0f = bf16_lo(aw[j]), a1f = bf16_hi(aw[j]);
          const float b0f = bf16_lo(bw[j]), b1f = bf16_hi(bw[j]);
          float xn0 = __fmul_rn(__fsub_rn(bf16_lo(ws[j]), mean), rstd);
          float xn1 = __fmul_rn(__fsub_rn(bf16_hi(ws[j]), mean), rstd);
          float y0, y1;
          if (MODE == kAdaLN) {
            float s0 = a0f, s1 = a1f;
            if (pr.add_one) {
              s0 = __fadd_rn(a0f, 1.f);
              s1 = __fadd_rn(a1f, 1.f);
              round_bf16x2(s0, s1);
            }
            round_bf16x2(xn0, xn1);
            float m0 = __fmul_rn(xn0, s0), m1 = __fmul_rn(xn1, s1);
            round_bf16x2(m0, m1);
            y0 = __fadd_rn(m0, b0f);
            y1 = __fadd_rn(m1, b1f);
          } else {
            y0 = __fmaf_rn(xn0, a0f, b0f);
            y1 = __fmaf_rn(xn1, a1f, b1f);
          }
          round_bf16x2(y0, y1);
          wmax = fmaxf(wmax, fmaxf(fabsf(y0), fabsf(y1)));
        }
      }
    }
  }
  wmax = warp_max(wmax);
  __shared__ float smax[8];
  if (lane == 0) smax[warp] = wmax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = smax[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) m = fmaxf(m, smax[i]);
    if (m > 0.f) atomic_max_nonneg(amax, m);
  }
}

// Self-test of div_const: counts bit patterns in [first, first + count) whose quotient differs from
// IEEE division (used by the test-suite to pin the range on which the fast path may rely on it).
template <int D>
__global__ void div_const_selftest_kernel(uint32_t first, uint64_t count, unsigned long long* mismatches) {
  pdl_wait();
  unsigned long long bad = 0;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x) {
    const float x = __uint_as_float(first + (uint32_t)i);
    if (x != x || fabsf(x) == __uint_as_float(0x7F800000u)) continue;
    const float a = div_const<D>(x), b = __fdiv_rn(x, (float)D);
    if (__float_as_uint(a) != __float_as_uint(b)) ++bad;
  }
  if (bad) atomicAdd(mismatches, bad);
}

template <int MODE>
int launch_quantize(int rule, dim3 grid, cudaStream_t stream, const uint16_t* x, int64_t M, int64_t K, int64_t ldx,
                    const float* amax, uint8_t* codes, uint8_t* sf, const Prologue& pr, uint16_t* y_out, int64_t ldy) {
  // few 128 x 128 CTAs: halve their width (grid.x doubles)
  int threads = 256;
  if ((int64_t)grid.x * grid.y * grid.z < 6 * (int64_t)sm_count()) {
    threads = 128;
    grid.x = (unsigned)((K + 63) / 64);
  }
  switch (rule) {
    case LLNV_RULE_STATIC_6: launch_k(quantize_nvfp4_kernel<LLNV_RULE_STATIC_6, MODE>, grid, threads, 0, stream, x, M, K, ldx, amax, codes, sf, pr, y_out, ldy); break;
    case LLNV_RULE_STATIC_4: launch_k(quantize_nvfp4_kernel<LLNV_RULE_STATIC_4, MODE>, grid, threads, 0, stream, x, M, K, ldx, amax, codes, sf, pr, y_out, ldy); break;
    case LLNV_RULE_MAE: launch_k(quantize_nvfp4_kernel<LLNV_RULE_MAE, MODE>, grid, threads, 0, stream, x, M, K, ldx, amax, codes, sf, pr, y_out, ldy); break;
    case LLNV_RULE_MSE: launch_k(quantize_nvfp4_kernel<LLNV_RULE_MSE, MODE>, grid, threads, 0, stream, x, M, K, ldx, amax, codes, sf, pr, y_out, ldy); break;
    default: launch_k(quantize_nvfp4_kernel<LLNV_RULE_ABS_MAX, MODE>, grid, threads, 0, stream, x, M, K, ldx, amax, codes, sf, pr, y_out, ldy); break;
  }
  return launch_status("quantize_nvfp4_kernel");
}

}  // namespace

// Shared by the allocation-free entry point in static_scratch.cu.
int ln_quantize_impl(int mode, const void* x, int64_t M, int64_t C, int64_t ldx, const void* p0, const void* p1,
                     int64_t mod_stride, int frame_rows, float eps, int add_one, int rule, void* codes, void* sf,
                     float* amax, void* y_out, int64_t ldy, float* row_stats, cudaStream_t stream, const char* who,
                     int64_t row_offset, int phase) {
  LLNV_REQUIRE(x && p0 && p1 && codes && sf && amax && row_stats, "%s: null pointer", who);
  LLNV_REQUIRE(mode == kAdaLN || mode == kAffineLN, "%s: unknown mode %d", who, mode);
  LLNV_REQUIRE(M >= 0 && C > 0 && C % 64 == 0 && C <= 4096, "%s: C must be a multiple of 64 and at most 4096 (got %lld)", who, (long long)C);
  LLNV_REQUIRE(ldx >= C && ldx % 8 == 0, "%s: ldx must be >= C and a multiple of 8", who);
  LLNV_REQUIRE(rule >= 0 && rule <= 4, "%s: unknown scale rule %d", who, rule);
  LLNV_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)p0 & 15) == 0 && ((uintptr_t)p1 & 15) == 0 && ((uintptr_t)codes & 7) == 0 &&
                   ((uintptr_t)sf & 3) == 0 && ((uintptr_t)row_stats & 7) == 0,
               "%s: x, scale/weight and shift/bias must be 16-byte aligned, codes 8-byte, sf 4-byte, row_stats 8-byte", who);
  if (mode == kAdaLN) LLNV_REQUIRE(frame_rows > 0 && mod_stride >= C && mod_stride % 8 == 0, "%s: frame_rows must be positive and the modulation stride a multiple of 8 that is >= C", who);
  if (y_out) LLNV_REQUIRE(ldy >= C && ldy % 8 == 0 && ((uintptr_t)y_out & 15) == 0, "%s: y_out must be 16-byte aligned with ldy a multiple of 8", who);
  LLNV_REQUIRE(phase >= 0 && phase <= 2 && row_offset >= 0, "%s: phase must be 0, 1 or 2 and row_offset non-negative", who);
  if (phase != 2) LLNV_CUDA(cudaMemsetAsync(amax, 0, sizeof(float), stream));
  if (M == 0) return LLNV_OK;
  Prologue pr = {};                 // every field the mode does not use stays zero (shard_cols = 0: plain input)
  pr.row_stats = row_stats;
  pr.p0 = (const uint16_t*)p0;
  pr.p1 = (const uint16_t*)p1;
  pr.stride = mod_stride;
  pr.frame_rows = frame_rows > 0 ? frame_rows : 1;
  pr.add_one = add_one;
  pr.row_offset = row_offset;
  if (phase != 2) {
    // warps per row: four when that leaves every lane at least one 16-byte vector (C a multiple of 1024), else one
    const bool split = C % 1024 == 0;
    const unsigned sblocks = split ? (unsigned)((M + 1) / 2) : (unsigned)((M + 7) / 8);
    if (mode == kAdaLN && split) launch_k(ln_stats_amax_kernel<kAdaLN, 4>, sblocks, 256, 0, stream, (const uint16_t*)x, M, C, ldx, eps, pr, row_stats, amax);
    else if (mode == kAdaLN) launch_k(ln_stats_amax_kernel<kAdaLN, 1>, sblocks, 256, 0, stream, (const uint16_t*)x, M, C, ldx, eps, pr, row_stats, amax);
    else if (split) launch_k(ln_stats_amax_kernel<kAffineLN, 4>, sblocks, 256, 0, stream, (const uint16_t*)x, M, C, ldx, eps, pr, row_stats, amax);
    else launch_k(ln_stats_amax_kernel<kAffineLN, 1>, sblocks, 256, 0, stream, (const uint16_t*)x, M, C, ldx, eps, pr, row_stats, amax);
    int rc = launch_status("ln_stats_amax_kernel");
    if (rc != LLNV_OK) return rc;
  }
  if (phase == 1) return LLNV_OK;
  const int64_t mp = (M + 127) / 128 * 128;
  LLNV_REQUIRE(mp / 128 <= 65535, "%s: too many rows (%lld)", who, (long long)M);
  dim3 grid((unsigned)((C + 127) / 128), (unsigned)(mp / 128));
  if (mode == kAdaLN)
    return launch_quantize<kAdaLN>(rule, grid, stream, (const uint16_t*)x, M, C, ldx, amax, (uint8_t*)codes, (uint8_t*)sf, pr, (uint16_t*)y_out, ldy);
  return launch_quantize<kAffineLN>(rule, grid, stream, (const uint16_t*)x, M, C, ldx, amax, (uint8_t*)codes, (uint8_t*)sf, pr, (uint16_t*)y_out, ldy);
}

}  // namespace llnv

using namespace llnv;

extern "C" int llnv_amax_bf16(const void* x, int64_t M, int64_t K, int64_t ldx, float* amax, llnv_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  LLNV_REQUIRE(x && amax, "llnv_amax_bf16: null pointer");
  LLNV_REQUIRE(M >= 0 && K >= 0 && K % 8 == 0 && ldx >= K && ldx % 8 == 0, "llnv_amax_bf16: K and ldx must be multiples of 8 (M=%lld K=%lld ldx=%lld)",
               (long long)M, (long long)K, (long long)ldx);
  LLNV_REQUIRE(((uintptr_t)x & 15) == 0, "llnv_amax_bf16: x must be 16-byte aligned");
  LLNV_CUDA(cudaMemsetAsync(amax, 0, sizeof(float), stream));
  const int64_t total = M * (K / 8);
  if (total == 0) return LLNV_OK;
  int64_t blocks = (total + 256 * 4 - 1) / (256 * 4);
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  launch_k(amax_bf16_kernel, (unsigned)blocks, 256, 0, stream, (const uint16_t*)x, M, K, ldx, amax);
  return launch_status("amax_bf16_kernel");
}

extern "C" int llnv_quantize_nvfp4(const void* x, int64_t M, int64_t K, int64_t ldx, int rule, void* codes, void* sf,
                                   float* amax, int amax_given, llnv_stream_t stream) {
  return llnv_quantize_nvfp4_ex(x, M, K, ldx, rule, codes, sf, amax, amax_given, 1, stream);
}

extern "C" int llnv_quantize_nvfp4_ex(const void* x, int64_t M, int64_t K, int64_t ldx, int rule, void* codes, void* sf,
                                      float* amax, int amax_given, int shards, llnv_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  LLNV_REQUIRE(x && codes && sf && amax, "llnv_quantize_nvfp4: null pointer");
  LLNV_REQUIRE(M >= 0 && K > 0 && K % 64 == 0, "llnv_quantize_nvfp4: K must be a positive multiple of 64 (got %lld)", (long long)K);
  LLNV_REQUIRE(shards >= 1 && K % shards == 0 && (K / shards) % 16 == 0,
               "llnv_quantize_nvfp4: shards must divide K into multiples of 16 columns (K=%lld shards=%d)", (long long)K, shards);
  const int64_t Ks = K / shards;
  LLNV_REQUIRE(ldx >= Ks && ldx % 8 == 0, "llnv_quantize_nvfp4: ldx must be >= K / shards and a multiple of 8 (got %lld)", (long long)ldx);
  LLNV_REQUIRE(rule >= 0 && rule <= 4, "llnv_quantize_nvfp4: unknown scale rule %d", rule);
  LLNV_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)codes & 7) == 0 && ((uintptr_t)sf & 3) == 0,
               "llnv_quantize_nvfp4: x must be 16-byte, codes 8-byte, sf 4-byte aligned");
  if (M == 0) {
    if (!amax_given) LLNV_CUDA(cudaMemsetAsync(amax, 0, sizeof(float), stream));
    return LLNV_OK;
  }
  if (!amax_given) {
    int rc = llnv_amax_bf16(x, M * shards, Ks, ldx, amax, stream_);
    if (rc != LLNV_OK) return rc;
  }
  const int64_t mp = (M + 127) / 128 * 128;
  dim3 grid((unsigned)((K + 127) / 128), (unsigned)(mp / 128));
  LLNV_REQUIRE(mp / 128 <= 65535, "llnv_quantize_nvfp4: too many rows (%lld)", (long long)M);
  Prologue pr = {};
  if (shards > 1) {
    pr.shard_cols = Ks;
    pr.shard_stride = M * ldx;
  }
  return launch_quantize<kPlain>(rule, grid, stream, (const uint16_t*)x, M, K, ldx, amax, (uint8_t*)codes, (uint8_t*)sf, pr, nullptr, 0);
}

extern "C" int llnv_quantize_nvfp4_pair(const void* x0, const void* x1, int64_t M, int64_t K, int64_t ldx, int rule, void* codes0,
                                        void* sf0, float* amax0, void* codes1, void* sf1, float* amax1, int amax_given,
                                        llnv_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  LLNV_REQUIRE(x0 && x1 && codes0 && codes1 && sf0 && sf1 && amax0 && amax1, "llnv_quantize_nvfp4_pair: null pointer");
  LLNV_REQUIRE(M >= 0 && K > 0 && K % 64 == 0, "llnv_quantize_nvfp4_pair: K must be a positive multiple of 64 (got %lld)", (long long)K);
  LLNV_REQUIRE(ldx >= K && ldx % 8 == 0, "llnv_quantize_nvfp4_pair: ldx must be >= K and a multiple of 8 (got %lld)", (long long)ldx);
  LLNV_REQUIRE(rule >= 0 && rule <= 4, "llnv_quantize_nvfp4_pair: unknown scale rule %d", rule);
  LLNV_REQUIRE(((uintptr_t)x0 & 15) == 0 && ((uintptr_t)x1 & 15) == 0 && ((uintptr_t)codes0 & 7) == 0 && ((uintptr_t)codes1 & 7) == 0 &&
                   ((uintptr_t)sf0 & 3) == 0 && ((uintptr_t)sf1 & 3) == 0,
               "llnv_quantize_nvfp4_pair: x must be 16-byte, codes 8-byte, sf 4-byte aligned");
  if (!amax_given) {
    int rc = llnv_amax_bf16(x0, M, K, ldx, amax0, stream_);
    if (rc == LLNV_OK) rc = llnv_amax_bf16(x1, M, K, ldx, amax1, stream_);
    if (rc != LLNV_OK) return rc;
  }
  if (M == 0) return LLNV_OK;
  const int64_t mp = (M + 127) / 128 * 128;
  LLNV_REQUIRE(mp / 128 <= 65535, "llnv_quantize_nvfp4_pair: too many rows (%lld)", (long long)M);
  dim3 grid((unsigned)((K + 127) / 128), (unsigned)(mp / 128), 2);
  Prologue pr = {};
  pr.x2 = (const uint16_t*)x1;
  pr.amax2 = amax1;
  pr.codes2 = (uint8_t*)codes1;
  pr.sf2 = (uint8_t*)sf1;
  return launch_quantize<kPlain>(rule, grid, stream, (const uint16_t*)x0, M, K, ldx, amax0, (uint8_t*)codes0, (uint8_t*)sf0, pr, nullptr, 0);
}

extern "C" int llnv_adaln_quantize_nvfp4(const void* x, int64_t M, int64_t C, int64_t ldx, const void* scale, const void* shift,
                                         int64_t mod_stride, int frame_rows, float eps, int add_one, int rule, void* codes,
                                         void* sf, float* amax, void* y_out, int64_t ldy, float* row_stats,
                                         llnv_stream_t stream) {
  return ln_quantize_impl(kAdaLN, x, M, C, ldx, scale, shift, mod_stride, frame_rows, eps, add_one, rule, codes, sf, amax,
                          y_out, ldy, row_stats, (cudaStream_t)stream, "llnv_adaln_quantize_nvfp4", 0, 0);
}

extern "C" int llnv_adaln_quantize_nvfp4_ex(const void* x, int64_t M, int64_t C, int64_t ldx, const void* scale, const void* shift,
                                            int64_t mod_stride, int frame_rows, float eps, int add_one, int rule, void* codes,
                                            void* sf, float* amax, void* y_out, int64_t ldy, float* row_stats,
                                            int64_t row_offset, int phase, llnv_stream_t stream) {
  return ln_quantize_impl(kAdaLN, x, M, C, ldx, scale, shift, mod_stride, frame_rows, eps, add_one, rule, codes, sf, amax,
                          y_out, ldy, row_stats, (cudaStream_t)stream, "llnv_adaln_quantize_nvfp4_ex", row_offset, phase);
}

extern "C" int llnv_layernorm_quantize_nvfp4_ex(const void* x, int64_t M, int64_t C, int64_t ldx, const void* weight,
                                                const void* bias, float eps, int rule, void* codes, void* sf, float* amax,
                                                void* y_out, int64_t ldy, float* row_stats, int phase, llnv_stream_t stream) {
  return ln_quantize_impl(kAffineLN, x, M, C, ldx, weight, bias, 0, 1, eps, 0, rule, codes, sf, amax, y_out, ldy, row_stats,
                          (cudaStream_t)stream, "llnv_layernorm_quantize_nvfp4_ex", 0, phase);
}

extern "C" int llnv_layernorm_quantize_nvfp4(const void* x, int64_t M, int64_t C, int64_t ldx, const void* weight,
                                             const void* bias, float eps, int rule, void* codes, void* sf, float* amax,
                                             void* y_out, int64_t ldy, float* row_stats, llnv_stream_t stream) {
  return ln_quantize_impl(kAffineLN, x, M, C, ldx, weight, bias, 0, 1, eps, 0, rule, codes, sf, amax, y_out, ldy, row_stats,
                          (cudaStream_t)stream, "llnv_layernorm_quantize_nvfp4", 0, 0);
}

// Test hook: number of fp32 bit patterns in [first_bits, first_bits + count) for which the
// multiply-and-correct quotient x / divisor (divisor 6 or 1536) differs from IEEE division.
// `mismatches` is a device pointer to one zero-initialised 64-bit counter.
extern "C" int llnv_selftest_div_const(int divisor, uint32_t first_bits, uint64_t count, unsigned long long* mismatches,
                                       llnv_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  LLNV_REQUIRE(mismatches && (divisor == 6 || divisor == 1536), "llnv_selftest_div_const: divisor must be 6 or 1536");
  if (count == 0) return LLNV_OK;
  const unsigned blocks = (unsigned)sm_count() * 8;
  if (divisor == 6) launch_k(div_const_selftest_kernel<6>, blocks, 256, 0, stream, first_bits, count, mismatches);
  else launch_k(div_const_selftest_kernel<1536>, blocks, 256, 0, stream, first_bits, count, mismatches);
  return launch_status("div_const_selftest_kernel");
}
