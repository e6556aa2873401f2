// Pieces shared by the 1-CTA and the 2-CTA W4A4 GEMM kernels: launch parameters, epilogue math.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "quant_block.cuh"
#include "sm100.cuh"

namespace llnv {
namespace gemm {

struct GemmParams {
  const uint8_t* sfa;
  const uint8_t* sfb;
  const float* a_amax;
  const float* b_amax;
  float alpha_denom;       // 6*Ea*6*Eb
  int64_t M, N, K;
  llnv_epilogue_t epi;
  __nv_bfloat16* d;
  int64_t ldd;
  unsigned int* status;
  // Grouped launch (1-CTA kernel): B is the concatenation along N of up to three weight matrices
  // of group_cols rows each, every one with its own tensor amax (b_amax[g]), output matrix and
  // optional output amax; 0 = one ordinary GEMM.
  int64_t group_cols;
  float* group_amax[3];
  // Requantized output (epilogue variants with kEpiQuant): NVFP4 codes [Mp, N/2] and swizzled scales of the
  // epilogue's bf16 result, quantized with the 4-over-6 MSE rule under the tensor amax *q_amax supplied by the caller.
  uint8_t* q_codes;
  uint8_t* q_sf;
  const float* q_amax;
  int store_bf16;          // 0: the bf16 result itself is not written (d may be null)
};

// Where one thread's row of a 64-column chunk goes when the epilogue requantizes (kEpiQuant).
struct QuantOut {
  quant::QuantConsts qc;
  uint8_t* codes;          // this row's 32 code bytes of the chunk
  uint32_t* sf;            // this row's 4 scale bytes of the chunk (one word of the swizzled atom)
};

struct GroupMaps {
  CUtensorMap m[2];        // output maps of groups 1 and 2 (group 0 uses the kernel's main output map)
};

// two fp32 -> packed bf16x2 (one conversion instruction, round to nearest even)
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float u = k0 * (x + k1 * x * x * x);
  return __fdividef(x, 1.f + __expf(-2.f * u));
}

// epilogue variants (compile-time, so that the plain path stays a handful of instructions per
// element and the whole epilogue fits the instruction cache)
constexpr int kEpiBias = 1, kEpiGelu = 2, kEpiRes = 4, kEpiQuant = 8;

// First step of every epilogue: alpha * accumulator, rounded to bf16 (the reference's GEMM returns
// bf16 before bias / activation / residual are applied), packed two columns per word.  After this
// step the accumulator columns are no longer needed.
__device__ __forceinline__ void drain_chunk(const uint32_t (&r)[2][32], float alpha, uint32_t (&pk)[32]) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int c0 = 2 * i, c1 = 2 * i + 1;
    pk[i] = pack2(__fmul_rn(alpha, __uint_as_float(r[c0 >> 5][c0 & 31])), __fmul_rn(alpha, __uint_as_float(r[c1 >> 5][c1 & 31])));
  }
}

// Rest of the epilogue of one 64-column chunk of one row per thread: pk holds bf16(alpha * acc) of
// columns col .. col+63 of this thread's row, the result is written as bf16 into the warp's
// swizzled staging buffer `buf` (32 rows x 128 bytes; with a residual the buffer holds the residual
// tile on entry).  grow: this row's gate vector or nullptr.
template <int EPI>
__device__ __forceinline__ void epilogue_packed(const uint32_t (&pk)[32], const uint16_t* __restrict__ bias,
                                                const uint16_t* __restrict__ grow, int64_t col, uint8_t* buf, int lane,
                                                bool want_amax, bool row_ok, float& local_amax, const QuantOut* qo = nullptr,
                                                bool store_bf16 = true) {
  constexpr bool has_res = (EPI & kEpiRes) != 0;
  constexpr bool has_quant = (EPI & kEpiQuant) != 0;
  uint32_t qw[8];                     // the 16 bf16 values of the quantization block being assembled
  uint32_t qc_words[8];               // the chunk's 32 code bytes
  uint32_t qsf = 0;                   // the chunk's 4 scale bytes
#pragma unroll
  for (int v8 = 0; v8 < 8; ++v8) {    // 8 columns (16 bytes) at a time
    uint4* slot = reinterpret_cast<uint4*>(buf + lane * 128 + ((v8 ^ (lane & 7)) << 4));
    if (EPI == 0) {
      if (want_amax && row_ok) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          local_amax = fmaxf(local_amax, fmaxf(fabsf(bf16_lo(pk[v8 * 4 + e])), fabsf(bf16_hi(pk[v8 * 4 + e]))));
        }
      }
      *slot = make_uint4(pk[v8 * 4], pk[v8 * 4 + 1], pk[v8 * 4 + 2], pk[v8 * 4 + 3]);
      continue;
    }
    float y[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      y[2 * e] = bf16_lo(pk[v8 * 4 + e]);
      y[2 * e + 1] = bf16_hi(pk[v8 * 4 + e]);
    }
    if (EPI & kEpiBias) {
      const uint4 bv = __ldg(reinterpret_cast<const uint4*>(bias + col + v8 * 8));
      const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        y[e] = y[e] + bf16_lo(bw[e >> 1]);
        y[e + 1] = y[e + 1] + bf16_hi(bw[e >> 1]);
        round_bf16x2(y[e], y[e + 1]);
      }
    }
    if (EPI & kEpiGelu) {
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        y[e] = gelu_tanh(y[e]);
        y[e + 1] = gelu_tanh(y[e + 1]);
        round_bf16x2(y[e], y[e + 1]);
      }
    }
    if (has_res) {
      const uint4 rv = *slot;
      const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
      if (grow) {
        const uint4 gv = __ldg(reinterpret_cast<const uint4*>(grow + col + v8 * 8));
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          y[e] = y[e] * bf16_lo(gw[e >> 1]);
          y[e + 1] = y[e + 1] * bf16_hi(gw[e >> 1]);
          round_bf16x2(y[e], y[e + 1]);
        }
      }
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        y[e] = bf16_lo(rw[e >> 1]) + y[e];
        y[e + 1] = bf16_hi(rw[e >> 1]) + y[e + 1];
        round_bf16x2(y[e], y[e + 1]);
      }
    }
    if (want_amax && row_ok) {
#pragma unroll
      for (int e = 0; e < 8; ++e) local_amax = fmaxf(local_amax, fabsf(y[e]));
    }
    uint4 ov;
    ov.x = pack2(y[0], y[1]);
    ov.y = pack2(y[2], y[3]);
    ov.z = pack2(y[4], y[5]);
    ov.w = pack2(y[6], y[7]);
    if (!has_quant || store_bf16) *slot = ov;
    if (has_quant) {
      // two 8-column units make one 16-element quantization block: the block quantizer of the standalone kernel,
      // on the bf16 values just produced, with the tensor amax given up front
      const int h = (v8 & 1) * 4;
      qw[h] = ov.x; qw[h + 1] = ov.y; qw[h + 2] = ov.z; qw[h + 3] = ov.w;
      if (v8 & 1) {
        uint32_t c_lo = 0, c_hi = 0, sfb = 0;
        if (row_ok) quant::quant_block<LLNV_RULE_MSE>(qw, qo->qc, c_lo, c_hi, sfb);     // rows beyond M: zero codes and scales
        qc_words[v8 - 1] = c_lo;
        qc_words[v8] = c_hi;
        qsf |= sfb << (8 * (v8 >> 1));
      }
    }
  }
  if (has_quant) {
    reinterpret_cast<uint4*>(qo->codes)[0] = make_uint4(qc_words[0], qc_words[1], qc_words[2], qc_words[3]);
    reinterpret_cast<uint4*>(qo->codes)[1] = make_uint4(qc_words[4], qc_words[5], qc_words[6], qc_words[7]);
    *qo->sf = qsf;
  }
}

// Both steps for one chunk (kernels whose accumulators rotate drain and finish chunk by chunk).
template <int EPI>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&r)[2][32], float alpha, const uint16_t* __restrict__ bias,
                                               const uint16_t* __restrict__ grow, int64_t col, uint8_t* buf, int lane,
                                               bool want_amax, bool row_ok, float& local_amax) {
  uint32_t pk[32];
  drain_chunk(r, alpha, pk);
  epilogue_packed<EPI>(pk, bias, grow, col, buf, lane, want_amax, row_ok, local_amax);
}

}  // namespace gemm
}  // namespace llnv
