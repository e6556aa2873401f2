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
#include "quant_block.cuh"

namespace llnv {

namespace {

using namespace quant;

// ---- tensor amax ----------------------------------------------------------------------------
// (F16: the 16-bit values are fp16; their magnitudes order as integers too, only the final conversion differs)
template <bool F16>
__global__ void __launch_bounds__(256) amax_16bit_kernel(const uint16_t* __restrict__ x, int64_t M, int64_t K,
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
    if (threadIdx.x == 0 && mm != 0) {
      const int bits = F16 ? __float_as_int(__half2float(__ushort_as_half((unsigned short)mm))) : (int)(mm << 16);
      atomicMax(reinterpret_cast<int*>(amax), bits);
    }
  }
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
  // sequence-parallel group whose ranks' amax values are MAX-reduced inside the quantize kernel before its first block
  // (world <= 1: none): on entry *amax is this rank's value, on return the group's
  PeerReduce peer;
};

// y of two adjacent channels (packed bf16 in, packed bf16 out) with the rounding points listed at Prologue.  Packed
// two-lane fp32 instructions: every lane rounds as the scalar instruction does, at half the issue slots.
__device__ __forceinline__ void round_f2(F2& v) { round_bf16x2(v.x, v.y); }
template <int MODE>
__device__ __forceinline__ uint32_t ln_pair(uint32_t xw, uint32_t aw, uint32_t bw, F2 mean2, F2 rstd2, int add_one) {
  F2 xn = f2_mul(f2_sub(F2{bf16_lo(xw), bf16_hi(xw)}, mean2), rstd2);
  const F2 a = {bf16_lo(aw), bf16_hi(aw)}, b = {bf16_lo(bw), bf16_hi(bw)};
  F2 y;
  if (MODE == kAdaLN) {
    F2 sc = a;
    if (add_one) {
      sc = f2_add(a, f2_splat(1.f));
      round_f2(sc);
    }
    round_f2(xn);
    F2 m = f2_mul(xn, sc);
    round_f2(m);
    y = f2_add(m, b);
  } else {
    y = f2_fma(xn, a, b);
  }
  return pack_bf16x2(y.x, y.y);
}

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
  const F2 mean2 = f2_splat(mean), rstd2 = f2_splat(rstd);
#pragma unroll
  for (int j = 0; j < 8; ++j) w[j] = ln_pair<MODE>(w[j], aw[j], bw[j], mean2, rstd2, pr.add_one);
}

template <int RULE, int MODE, bool F16 = false>
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
  float amax_val = *amax_ptr;
  unsigned int peer_epoch = 0u;
  if (pr.peer.world > 1) {
    __shared__ float amax_sh;
    __shared__ unsigned int epoch_sh;
    if (threadIdx.x < 32) {
      const float m = peer_group_max(pr.peer, amax_val, (blockIdx.x | blockIdx.y | blockIdx.z) == 0u, &epoch_sh);
      if (threadIdx.x == 0) amax_sh = m;
    }
    __syncthreads();
    amax_val = amax_sh;
    peer_epoch = epoch_sh;
  }
  const QuantConsts qc = make_consts<RULE>(amax_val);

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
    if (codes == nullptr) continue;          // transform-only call (y_out): nothing to quantize
    uint32_t c_lo, c_hi, s;
    if (F16) quant_block_f16<RULE>(cur, qc, c_lo, c_hi, s);      // the words hold fp16 values
    else quant_block<RULE>(cur, qc, c_lo, c_hi, s);
    if (col_ok) *reinterpret_cast<uint2*>(codes + r * (K >> 1) + (col >> 1)) = make_uint2(c_lo, c_hi);
    my_sf |= s << (8 * i);
  }
  if (codes == nullptr) return;

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
  if (pr.peer.world > 1 && threadIdx.x == 0) {
    // The last CTA to get here closes the exchange: every CTA has read the epoch and this rank's value by now, so the
    // scalar can take the group maximum (the GEMM that consumes this tensor scales with it) and the epoch can advance.
    const unsigned int total = gridDim.x * gridDim.y * gridDim.z;
    __threadfence();
    if (atomicAdd(pr.peer.epoch + 1, 1u) == total - 1u) {
      *const_cast<float*>(amax_ptr) = amax_val;
      pr.peer.epoch[1] = 0u;
      __threadfence();
      pr.peer.epoch[0] = peer_epoch;
    }
  }
}

// ---- row statistics + amax of the transformed activation ----------------------------------------
// One warp per row: mean and rstd in fp32 (two-pass over registers), then the row's transformed
// values are formed once to find max|y|; nothing but the 8-byte statistics is stored.
// WPR warps share one row (each takes C / WPR channels): with one warp per row a chunk of 2640
// tokens is only 2640 warps and the kernel is bound by the latency of each warp's dependent steps.
template <int MODE, int WPR>
__global__ void __launch_bounds__(256, WPR > 1 ? 8 : 1) ln_stats_amax_kernel(const uint16_t* __restrict__ x, int64_t M, int64_t C, int64_t ldx,
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
  uint4 v[kVec];
  float sum = 0.f;
  // parameter row of this token (WPR > 1: its vectors are fetched where they are used, after the statistics; the few
  // rows of a frame are shared by hundreds of tokens and stay in L1 / L2, and not holding them across the two
  // reductions keeps the kernel at 40 registers, i.e. half as many waves of CTAs)
  const int64_t prow = (MODE == kAdaLN && live) ? ((row + pr.row_offset) / pr.frame_rows) * pr.stride : 0;
  if (live) {
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const int li = lane + 32 * i;
      if (li < pvec) {
        v[i] = __ldg(reinterpret_cast<const uint4*>(x + row * ldx) + vbase + li);
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
    const F2 mean2 = f2_splat(mean), rstd2 = f2_splat(rstd);
    uint32_t ymax2 = 0u;                       // packed running maximum of |y| (two bf16 magnitudes)
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const int li = lane + 32 * i;
      if (li < pvec) {
        const int idx = vbase + li;
        const uint4 a4 = WPR > 1 ? __ldg(reinterpret_cast<const uint4*>(pr.p0 + prow) + idx) : pa_sh[fsel][idx];
        const uint4 b4 = WPR > 1 ? __ldg(reinterpret_cast<const uint4*>(pr.p1 + prow) + idx) : pb_sh[fsel][idx];
        const uint32_t ws[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
        const uint32_t aw[4] = {a4.x, a4.y, a4.z, a4.w};
        const uint32_t bw[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) ymax2 = __vmaxu2(ymax2, ln_pair<MODE>(ws[j], aw[j], bw[j], mean2, rstd2, pr.add_one) & 0x7FFF7FFFu);
      }
    }
    wmax = __uint_as_float(max(ymax2 & 0xFFFFu, ymax2 >> 16) << 16);      // bf16 magnitudes order as integers
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
                     int64_t row_offset, int phase, const PeerReduce* peer) {
  LLNV_REQUIRE(x && p0 && p1 && amax && row_stats, "%s: null pointer", who);
  if (peer) LLNV_REQUIRE(phase == 0 && codes && M > 0, "%s: the group form runs both passes on a non-empty shard and writes codes", who);
  LLNV_REQUIRE((codes && sf) || (!codes && !sf && y_out), "%s: codes and sf go together; both may be null only when y_out is wanted", who);
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
  if (phase != 2 && !amax_accumulate(1)) LLNV_CUDA(cudaMemsetAsync(amax, 0, sizeof(float), stream));
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
  if (peer) pr.peer = *peer;
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
  launch_k(amax_16bit_kernel<false>, (unsigned)blocks, 256, 0, stream, (const uint16_t*)x, M, K, ldx, amax);
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

namespace {
// Group description of the C ABI -> PeerReduce.
int fill_peer(PeerReduce* out, const void* const* slot_ptrs, const void* const* signal_ptrs, int rank, int world, void* epoch, const char* who) {
  LLNV_REQUIRE(slot_ptrs && signal_ptrs && epoch, "%s: null group pointer", who);
  LLNV_REQUIRE(world >= 2 && world <= kMaxPeers && rank >= 0 && rank < world, "%s: need 2 <= world <= 8 and 0 <= rank < world", who);
  LLNV_REQUIRE(((uintptr_t)epoch & 7) == 0, "%s: epoch must be an 8-byte aligned pair of device words", who);
  *out = PeerReduce{};
  for (int r = 0; r < world; ++r) {
    LLNV_REQUIRE(slot_ptrs[r] && signal_ptrs[r] && ((uintptr_t)slot_ptrs[r] & 3) == 0 && ((uintptr_t)signal_ptrs[r] & 3) == 0, "%s: bad pointer of rank %d", who, r);
    out->slots[r] = const_cast<void*>(slot_ptrs[r]);
    out->signals[r] = const_cast<void*>(signal_ptrs[r]);
  }
  out->rank = rank;
  out->world = world;
  out->epoch = (unsigned int*)epoch;
  out->max_polls = peer_poll_limit();
  out->status = device_status_word();
  return LLNV_OK;
}
}  // namespace

extern "C" int llnv_quantize_nvfp4_group(const void* x, int64_t M, int64_t K, int64_t ldx, int rule, void* codes, void* sf, float* amax,
                                         int shards, const void* const* slot_ptrs, const void* const* signal_ptrs, int rank, int world,
                                         void* epoch, llnv_stream_t stream_) {
  const char* who = "llnv_quantize_nvfp4_group";
  cudaStream_t stream = (cudaStream_t)stream_;
  LLNV_REQUIRE(x && codes && sf && amax, "%s: null pointer", who);
  LLNV_REQUIRE(M > 0 && K > 0 && K % 64 == 0, "%s: M must be positive and K a positive multiple of 64", who);
  LLNV_REQUIRE(shards >= 1 && K % shards == 0 && (K / shards) % 16 == 0, "%s: shards must divide K into multiples of 16 columns", who);
  const int64_t Ks = K / shards;
  LLNV_REQUIRE(ldx >= Ks && ldx % 8 == 0, "%s: ldx must be >= K / shards and a multiple of 8", who);
  LLNV_REQUIRE(rule >= 0 && rule <= 4, "%s: unknown scale rule %d", who, rule);
  LLNV_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)codes & 7) == 0 && ((uintptr_t)sf & 3) == 0, "%s: x must be 16-byte, codes 8-byte, sf 4-byte aligned", who);
  const int64_t mp = (M + 127) / 128 * 128;
  LLNV_REQUIRE(mp / 128 <= 65535, "%s: too many rows (%lld)", who, (long long)M);
  Prologue pr = {};
  if (shards > 1) {
    pr.shard_cols = Ks;
    pr.shard_stride = M * ldx;
  }
  const int rc = fill_peer(&pr.peer, slot_ptrs, signal_ptrs, rank, world, epoch, who);
  if (rc != LLNV_OK) return rc;
  dim3 grid((unsigned)((K + 127) / 128), (unsigned)(mp / 128));
  return launch_quantize<kPlain>(rule, grid, stream, (const uint16_t*)x, M, K, ldx, amax, (uint8_t*)codes, (uint8_t*)sf, pr, nullptr, 0);
}

extern "C" int llnv_adaln_quantize_nvfp4_group(const void* x, int64_t M, int64_t C, int64_t ldx, const void* scale, const void* shift,
                                               int64_t mod_stride, int frame_rows, float eps, int add_one, int rule, void* codes, void* sf,
                                               float* amax, float* row_stats, int64_t row_offset, const void* const* slot_ptrs,
                                               const void* const* signal_ptrs, int rank, int world, void* epoch, llnv_stream_t stream) {
  PeerReduce peer;
  const int rc = fill_peer(&peer, slot_ptrs, signal_ptrs, rank, world, epoch, "llnv_adaln_quantize_nvfp4_group");
  if (rc != LLNV_OK) return rc;
  return ln_quantize_impl(kAdaLN, x, M, C, ldx, scale, shift, mod_stride, frame_rows, eps, add_one, rule, codes, sf, amax, nullptr, 0,
                          row_stats, (cudaStream_t)stream, "llnv_adaln_quantize_nvfp4_group", row_offset, 0, &peer);
}

extern "C" int llnv_layernorm_quantize_nvfp4_group(const void* x, int64_t M, int64_t C, int64_t ldx, const void* weight, const void* bias,
                                                   float eps, int rule, void* codes, void* sf, float* amax, float* row_stats,
                                                   const void* const* slot_ptrs, const void* const* signal_ptrs, int rank, int world,
                                                   void* epoch, llnv_stream_t stream) {
  PeerReduce peer;
  const int rc = fill_peer(&peer, slot_ptrs, signal_ptrs, rank, world, epoch, "llnv_layernorm_quantize_nvfp4_group");
  if (rc != LLNV_OK) return rc;
  return ln_quantize_impl(kAffineLN, x, M, C, ldx, weight, bias, 0, 1, eps, 0, rule, codes, sf, amax, nullptr, 0, row_stats,
                          (cudaStream_t)stream, "llnv_layernorm_quantize_nvfp4_group", 0, 0, &peer);
}

// fp16 input (the reference's CUDA backend accepts it beside bf16, fouroversix/src/fouroversix/quantize/cuda/backend.py:45-51):
// same outputs and layouts; every block goes through the reference's fp32 arithmetic one operation at a time.
extern "C" int llnv_quantize_nvfp4_f16(const void* x, int64_t M, int64_t K, int64_t ldx, int rule, void* codes, void* sf,
                                       float* amax, int amax_given, llnv_stream_t stream_) {
  const char* who = "llnv_quantize_nvfp4_f16";
  cudaStream_t stream = (cudaStream_t)stream_;
  LLNV_REQUIRE(x && codes && sf && amax, "%s: null pointer", who);
  LLNV_REQUIRE(M >= 0 && K > 0 && K % 64 == 0, "%s: K must be a positive multiple of 64 (got %lld)", who, (long long)K);
  LLNV_REQUIRE(ldx >= K && ldx % 8 == 0, "%s: ldx must be >= K and a multiple of 8 (got %lld)", who, (long long)ldx);
  LLNV_REQUIRE(rule >= 0 && rule <= 4, "%s: unknown scale rule %d", who, rule);
  LLNV_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)codes & 7) == 0 && ((uintptr_t)sf & 3) == 0, "%s: x must be 16-byte, codes 8-byte, sf 4-byte aligned", who);
  if (!amax_given) LLNV_CUDA(cudaMemsetAsync(amax, 0, sizeof(float), stream));
  if (M == 0) return LLNV_OK;
  if (!amax_given) {
    int64_t blocks = (M * (K / 8) + 256 * 4 - 1) / (256 * 4);
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    launch_k(amax_16bit_kernel<true>, (unsigned)blocks, 256, 0, stream, (const uint16_t*)x, M, K, ldx, amax);
    const int rc = launch_status("amax_f16_kernel");
    if (rc != LLNV_OK) return rc;
  }
  const int64_t mp = (M + 127) / 128 * 128;
  LLNV_REQUIRE(mp / 128 <= 65535, "%s: too many rows (%lld)", who, (long long)M);
  dim3 grid((unsigned)((K + 63) / 64), (unsigned)(mp / 128));          // 128 threads per CTA: 128 rows x 64 columns
  const Prologue pr = {};
  const uint16_t* xp = (const uint16_t*)x;
  uint8_t* cp = (uint8_t*)codes;
  uint8_t* sp = (uint8_t*)sf;
  uint16_t* none = nullptr;
  const int64_t zero = 0;
  switch (rule) {
    case LLNV_RULE_STATIC_6: launch_k(quantize_nvfp4_kernel<LLNV_RULE_STATIC_6, kPlain, true>, grid, 128, 0, stream, xp, M, K, ldx, amax, cp, sp, pr, none, zero); break;
    case LLNV_RULE_STATIC_4: launch_k(quantize_nvfp4_kernel<LLNV_RULE_STATIC_4, kPlain, true>, grid, 128, 0, stream, xp, M, K, ldx, amax, cp, sp, pr, none, zero); break;
    case LLNV_RULE_MAE: launch_k(quantize_nvfp4_kernel<LLNV_RULE_MAE, kPlain, true>, grid, 128, 0, stream, xp, M, K, ldx, amax, cp, sp, pr, none, zero); break;
    case LLNV_RULE_MSE: launch_k(quantize_nvfp4_kernel<LLNV_RULE_MSE, kPlain, true>, grid, 128, 0, stream, xp, M, K, ldx, amax, cp, sp, pr, none, zero); break;
    default: launch_k(quantize_nvfp4_kernel<LLNV_RULE_ABS_MAX, kPlain, true>, grid, 128, 0, stream, xp, M, K, ldx, amax, cp, sp, pr, none, zero); break;
  }
  return launch_status("quantize_nvfp4_kernel<f16>");
}
