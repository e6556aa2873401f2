// bf16 -> NVFP4 quantizer (E2M1 codes, E4M3 scale per 16 elements, fp32 tensor scale, the
// "four over six" scale selection), bit-exact against the reference's PyTorch quantizer
// (fouroversix/src/fouroversix/quantize/pytorch/reference.py:242-368).
//
// Layout of one CTA: 128 rows x 128 columns of the input, 256 threads.  Thread t owns the
// 16-element block (row = t/8 + 32*i, column block = t%8) for i = 0..3, so
//   * a warp reads 4 rows x 256 contiguous bytes per i with 128-bit loads,
//   * the 4 scale bytes of a thread land in one 16-byte unit of the 128x4 swizzled scale atom;
//     four neighbouring lanes transpose their bytes with warp shuffles and store whole words,
//     so every 512-byte scale atom is written densely by one CTA.
// All fp32 operations are issued with explicit round-to-nearest intrinsics so that the compiler
// cannot contract them into FMAs: the 4-vs-6 decision compares two rounded 16-term sums.
#include "common.cuh"

namespace llnv {

namespace {

// ---- tensor amax ----------------------------------------------------------------------------
__global__ void __launch_bounds__(256) amax_bf16_kernel(const uint16_t* __restrict__ x, int64_t M, int64_t K,
                                                        int64_t ldx, float* __restrict__ amax) {
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

// ---- per-element pieces ---------------------------------------------------------------------

// Round |xs| onto {0,.5,1,1.5,2,3,4,6,(8)} with ties to even (reference.py:13-34).
__device__ __forceinline__ float e2m1_round_mag(float a) {
  const float k = a < 2.f ? 2.f : (a < 4.f ? 1.f : 0.5f);
  const float kinv = a < 2.f ? 0.5f : (a < 4.f ? 1.f : 2.f);
  return __fmul_rn(rintf(__fmul_rn(a, k)), kinv);
}

// 4-bit code of a rounded magnitude with the sign of xs (reference.py:37-63).  A magnitude of 8
// (reachable only when the block scale is a tiny subnormal) maps to 0b1000 for either sign,
// as the reference's exponent arithmetic does.
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

// One candidate scale applied to a pair of elements (i, i+8) of a block.
struct Cand {
  float inv;     // 1 / (dec * s), or 0 when s == 0
  float s;       // decoded block scale
  bool zero;     // s == 0
};

template <int RULE>
__device__ __forceinline__ void quant_block(const uint32_t (&w)[8], float amax, float enc, float dec, uint64_t& codes_out,
                                            uint32_t& sf_out) {
  constexpr bool kStatic = (RULE == LLNV_RULE_STATIC_6 || RULE == LLNV_RULE_STATIC_4);
  constexpr float kE2 = RULE == LLNV_RULE_STATIC_4 ? 4.f : 6.f;
  float x[16];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    x[2 * j] = bf16_lo(w[j]);
    x[2 * j + 1] = bf16_hi(w[j]);
  }
  float bmax = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) bmax = fmaxf(bmax, fabsf(x[j]));
  const float hp = amax == 0.f ? 0.f : __fmul_rn(__fdiv_rn(bmax, kE2), enc);

  if (kStatic) {
    const uint32_t sc = float_to_e4m3(hp);
    const float s = e4m3_to_float(sc);
    const float inv = s != 0.f ? __fdiv_rn(1.f, __fmul_rn(dec, s)) : 0.f;
    uint64_t c = 0;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float xs = s != 0.f ? __fmul_rn(x[j], inv) : 0.f;
      c |= (uint64_t)e2m1_code(e2m1_round_mag(fabsf(xs)), xs < 0.f) << (4 * j);
    }
    codes_out = c;
    sf_out = sc;
    return;
  }

  const uint32_t sc6 = float_to_e4m3(hp);
  const uint32_t sc4 = float_to_e4m3(__fmul_rn(hp, 1.5f));
  const float s6 = e4m3_to_float(sc6), s4 = e4m3_to_float(sc4);
  const float inv6 = s6 != 0.f ? __fdiv_rn(1.f, __fmul_rn(dec, s6)) : 0.f;
  const float inv4 = s4 != 0.f ? __fdiv_rn(1.f, __fmul_rn(dec, s4)) : 0.f;
  uint64_t c6 = 0, c4 = 0;
  float e6 = 0.f, e4 = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float t6[2], t4[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int j = i + 8 * h;
      // candidate 6
      const float xs6 = s6 != 0.f ? __fmul_rn(x[j], inv6) : 0.f;
      const float m6 = e2m1_round_mag(fabsf(xs6));
      c6 |= (uint64_t)e2m1_code(m6, xs6 < 0.f) << (4 * j);
      const float q6 = xs6 < 0.f ? -m6 : m6;
      const float d6 = __fsub_rn(__fdiv_rn(__fmul_rn(__fmul_rn(q6, s6), amax), 1536.f), x[j]);
      t6[h] = err_term<RULE>(d6);
      // candidate 4
      const float xs4 = s4 != 0.f ? __fmul_rn(x[j], inv4) : 0.f;
      const float m4 = e2m1_round_mag(fabsf(xs4));
      c4 |= (uint64_t)e2m1_code(m4, xs4 < 0.f) << (4 * j);
      const float q4 = xs4 < 0.f ? -m4 : m4;
      const float d4 = __fsub_rn(__fdiv_rn(__fmul_rn(__fmul_rn(q4, s4), amax), 1536.f), x[j]);
      t4[h] = err_term<RULE>(d4);
    }
    if (RULE == LLNV_RULE_ABS_MAX) {
      e6 = fmaxf(e6, fmaxf(t6[0], t6[1]));
      e4 = fmaxf(e4, fmaxf(t4[0], t4[1]));
    } else {
      // torch's CPU reduction order over 16 contiguous fp32 values: lane sums v[i]+v[i+8], then
      // the eight lanes are added left to right.
      const float a6 = __fadd_rn(t6[0], t6[1]);
      const float a4 = __fadd_rn(t4[0], t4[1]);
      e6 = i == 0 ? a6 : __fadd_rn(e6, a6);
      e4 = i == 0 ? a4 : __fadd_rn(e4, a4);
    }
  }
  const bool sel4 = e4 < e6;
  codes_out = sel4 ? c4 : c6;
  sf_out = sel4 ? sc4 : sc6;
}

template <int RULE>
__global__ void __launch_bounds__(256) quantize_nvfp4_kernel(const uint16_t* __restrict__ x, int64_t M, int64_t K,
                                                             int64_t ldx, const float* __restrict__ amax_ptr,
                                                             uint8_t* __restrict__ codes, uint8_t* __restrict__ sf) {
  constexpr float kE2 = RULE == LLNV_RULE_STATIC_4 ? 4.f : 6.f;
  constexpr float kE4 = (RULE == LLNV_RULE_STATIC_6 || RULE == LLNV_RULE_STATIC_4) ? 448.f : 256.f;
  const float amax = *amax_ptr;
  const float enc = __fdiv_rn(kE2 * kE4, amax);     // reference.py:142-151
  const float dec = __fdiv_rn(1.f, enc);            // reference.py:159-166

  const int t = threadIdx.x;
  const int cb = t & 7;
  const int r0 = t >> 3;
  const int64_t col = (int64_t)blockIdx.x * 128 + cb * 16;
  const int64_t row_base = (int64_t)blockIdx.y * 128;
  const bool col_ok = col < K;

  uint32_t w[4][8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t r = row_base + r0 + 32 * i;
    if (col_ok && r < M) {
      const uint4* p = reinterpret_cast<const uint4*>(x + r * ldx + col);
      const uint4 a = __ldg(p), b = __ldg(p + 1);
      w[i][0] = a.x; w[i][1] = a.y; w[i][2] = a.z; w[i][3] = a.w;
      w[i][4] = b.x; w[i][5] = b.y; w[i][6] = b.z; w[i][7] = b.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) w[i][j] = 0u;
    }
  }

  uint32_t my_sf = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint64_t c;
    uint32_t s;
    quant_block<RULE>(w[i], amax, enc, dec, c, s);
    if (col_ok) {
      const int64_t r = row_base + r0 + 32 * i;
      *reinterpret_cast<uint2*>(codes + r * (K >> 1) + (col >> 1)) = make_uint2((uint32_t)c, (uint32_t)(c >> 32));
    }
    my_sf |= s << (8 * i);
  }

  // Transpose the 4x4 scale bytes of each group of four lanes: lane q ends up with the word that
  // holds row (r0 + 32*q) ... i.e. bytes [scale column 0..3] of 16-byte unit r0, word q.
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

}  // namespace

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
  amax_bf16_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const uint16_t*)x, M, K, ldx, amax);
  return launch_status("amax_bf16_kernel");
}

extern "C" int llnv_quantize_nvfp4(const void* x, int64_t M, int64_t K, int64_t ldx, int rule, void* codes, void* sf,
                                   float* amax, int amax_given, llnv_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  LLNV_REQUIRE(x && codes && sf && amax, "llnv_quantize_nvfp4: null pointer");
  LLNV_REQUIRE(M >= 0 && K > 0 && K % 64 == 0, "llnv_quantize_nvfp4: K must be a positive multiple of 64 (got %lld)", (long long)K);
  LLNV_REQUIRE(ldx >= K && ldx % 8 == 0, "llnv_quantize_nvfp4: ldx must be >= K and a multiple of 8 (got %lld)", (long long)ldx);
  LLNV_REQUIRE(rule >= 0 && rule <= 4, "llnv_quantize_nvfp4: unknown scale rule %d", rule);
  LLNV_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)codes & 7) == 0 && ((uintptr_t)sf & 3) == 0,
               "llnv_quantize_nvfp4: x must be 16-byte, codes 8-byte, sf 4-byte aligned");
  if (M == 0) {
    if (!amax_given) LLNV_CUDA(cudaMemsetAsync(amax, 0, sizeof(float), stream));
    return LLNV_OK;
  }
  if (!amax_given) {
    int rc = llnv_amax_bf16(x, M, K, ldx, amax, stream_);
    if (rc != LLNV_OK) return rc;
  }
  const int64_t mp = (M + 127) / 128 * 128;
  dim3 grid((unsigned)((K + 127) / 128), (unsigned)(mp / 128));
  LLNV_REQUIRE(mp / 128 <= 65535, "llnv_quantize_nvfp4: too many rows (%lld)", (long long)M);
  const uint16_t* xp = (const uint16_t*)x;
  uint8_t* cp = (uint8_t*)codes;
  uint8_t* sp = (uint8_t*)sf;
  switch (rule) {
    case LLNV_RULE_STATIC_6: quantize_nvfp4_kernel<LLNV_RULE_STATIC_6><<<grid, 256, 0, stream>>>(xp, M, K, ldx, amax, cp, sp); break;
    case LLNV_RULE_STATIC_4: quantize_nvfp4_kernel<LLNV_RULE_STATIC_4><<<grid, 256, 0, stream>>>(xp, M, K, ldx, amax, cp, sp); break;
    case LLNV_RULE_MAE: quantize_nvfp4_kernel<LLNV_RULE_MAE><<<grid, 256, 0, stream>>>(xp, M, K, ldx, amax, cp, sp); break;
    case LLNV_RULE_MSE: quantize_nvfp4_kernel<LLNV_RULE_MSE><<<grid, 256, 0, stream>>>(xp, M, K, ldx, amax, cp, sp); break;
    default: quantize_nvfp4_kernel<LLNV_RULE_ABS_MAX><<<grid, 256, 0, stream>>>(xp, M, K, ldx, amax, cp, sp); break;
  }
  return launch_status("quantize_nvfp4_kernel");
}
