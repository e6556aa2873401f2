// RMSNorm over the full channel dimension -> per-head 3-D RoPE -> (optionally) k_smooth and the
// amax of the rotated tensor, in one pass: the Q / K prologue of the chunk attention and of the
// KV-cache write.
//
//   y   = bf16(bf16(x * rsqrt(mean(x^2) + eps)) * weight)          wan_5b/modules/model.py:82-98
//   out = bf16(rotate pairs (2d, 2d+1) of every head by (cos, sin)[token, d])  utils/rope_triton.py:36-81
//   out_smooth = bf16(out - bf16(mean over the head's channels))   utils/quant.py:797-798
//   amax = max |out|  (tensor scale of the NVFP4 cache block the rotated keys are written to)
//
// One warp per token row: a lane holds 16-byte vectors v = lane + 32*i; vector v covers channels
// 8v..8v+7, i.e. four rotation pairs of head v/16, so a head's 128 channels live in 16 adjacent
// lanes and the per-head mean is a 4-step shuffle reduction.
#include "common.cuh"

namespace llnv {
namespace {

constexpr int kMaxVec = 16;      // C <= 4096
constexpr int kMaxShards = 8;

// Base address of every head shard of the two outputs (one entry when the output is a plain
// [S, C] matrix).  The entries may point into other GPUs' memory: they are only stored to.
struct ShardOut {
  uint16_t* out[kMaxShards];
  uint16_t* smooth[kMaxShards];
};

// One tensor to process; a launch takes up to two (blockIdx.y), e.g. the q and the k projection of
// a block, which share the token count, the channel count and the rotary tables.
struct RopeJob {
  const uint16_t* x;
  const uint16_t* weight;
  ShardOut dst;
  int64_t ldx, ldo, lds;
  float* amax_out;
  int want_smooth;
};
struct RopeJobs {
  RopeJob job[2];
};

// WPR warps share one token row (each takes C / WPR channels, a whole number of heads): a row is
// short (6 KB), so with one warp per row a chunk of 2640 tokens would put only 2640 warps on the
// device and the kernel would be bound by the latency of each warp's single pass.
template <int WPR>
__global__ void __launch_bounds__(256) rmsnorm_rope_kernel(const __grid_constant__ RopeJobs jobs, int64_t S, int64_t C, float eps,
                                                           const float* __restrict__ cosv, const float* __restrict__ sinv,
                                                           int shard_vecs) {
  pdl_wait();
  const RopeJob& jb = jobs.job[blockIdx.y];
  const uint16_t* __restrict__ x = jb.x;
  const uint16_t* __restrict__ weight = jb.weight;
  const ShardOut& dst = jb.dst;
  const int64_t ldx = jb.ldx, ldo = jb.ldo, lds = jb.lds;
  const bool want_smooth = jb.want_smooth != 0;
  float* __restrict__ amax_out = jb.amax_out;
  constexpr int kVec = kMaxVec / WPR;        // 16-byte vectors per lane
  constexpr int kRows = 8 / WPR;             // rows per CTA
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int part = warp % WPR;
  const int64_t row = (int64_t)blockIdx.x * kRows + warp / WPR;
  // the norm weight is shared by all rows: one cooperative load per CTA instead of a dependent
  // global load in every step of the per-row loop
  __shared__ uint4 w_sh[4096 / 8];
  __shared__ float ss_sh[8];
  const int nvec = (int)(C >> 3);
  const int pvec = nvec / WPR;               // vectors of this warp's part
  const int vbase = part * pvec;
  if (weight) {
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) w_sh[i] = __ldg(reinterpret_cast<const uint4*>(weight) + i);
  }
  // this lane needs the same 4 cos / 4 sin values in every step (pair index depends on lane only:
  // a part starts on a head boundary)
  float cc[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
  uint4 v[kVec];
  float ss = 0.f;
  if (row < S) {
    if (cosv) {
      const int pair0 = (lane & 15) * 4;
      const float4 c4 = __ldg(reinterpret_cast<const float4*>(cosv + row * 64 + pair0));
      const float4 s4 = __ldg(reinterpret_cast<const float4*>(sinv + row * 64 + pair0));
      cc[0] = c4.x; cc[1] = c4.y; cc[2] = c4.z; cc[3] = c4.w;
      sn[0] = s4.x; sn[1] = s4.y; sn[2] = s4.z; sn[3] = s4.w;
    }
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const int li = lane + 32 * i;
      if (li < pvec) {
        v[i] = __ldg(reinterpret_cast<const uint4*>(x + row * ldx) + vbase + li);
        const uint32_t w4[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a = bf16_lo(w4[j]), b = bf16_hi(w4[j]);
          ss += a * a + b * b;
        }
      }
    }
  }
  if (weight) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    if (lane == 0) ss_sh[warp] = ss;
  }
  __syncthreads();                           // weight staged, partial sums of squares published
  float wmax = 0.f;
  if (row < S) {
    float rinv = 1.f;
    if (weight) {
      float tot = ss_sh[warp - part];
#pragma unroll
      for (int k = 1; k < WPR; ++k) tot += ss_sh[warp - part + k];
      rinv = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)C), eps)));
    }
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const int li = lane + 32 * i;
      if (li >= pvec) continue;           // uniform per (i, lane half): a part is a whole number of heads, so 16-lane groups stay whole
      const int idx = vbase + li;
      uint32_t w4[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
      float y[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        y[2 * j] = bf16_lo(w4[j]);
        y[2 * j + 1] = bf16_hi(w4[j]);
      }
      if (weight) {
        const uint4 wv = w_sh[idx];
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          float a = __fmul_rn(y[2 * p], rinv), b = __fmul_rn(y[2 * p + 1], rinv);
          round_bf16x2(a, b);
          a = __fmul_rn(a, bf16_lo(ww[p]));
          b = __fmul_rn(b, bf16_hi(ww[p]));
          round_bf16x2(a, b);
          y[2 * p] = a;
          y[2 * p + 1] = b;
        }
      }
      if (cosv) {
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const float a = y[2 * p], b = y[2 * p + 1];
          y[2 * p] = __fsub_rn(__fmul_rn(a, cc[p]), __fmul_rn(b, sn[p]));
          y[2 * p + 1] = __fadd_rn(__fmul_rn(a, sn[p]), __fmul_rn(b, cc[p]));
          round_bf16x2(y[2 * p], y[2 * p + 1]);
        }
      }
      float hsum = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        wmax = fmaxf(wmax, fabsf(y[e]));
        hsum += y[e];
      }
      uint4 o;
      o.x = pack_bf16x2(y[0], y[1]); o.y = pack_bf16x2(y[2], y[3]);
      o.z = pack_bf16x2(y[4], y[5]); o.w = pack_bf16x2(y[6], y[7]);
      // head-sharded outputs: 16-byte vector idx lives in shard idx / shard_vecs (a whole number of heads)
      const int sh = shard_vecs ? idx / shard_vecs : 0;
      const int vi = shard_vecs ? idx - sh * shard_vecs : idx;
      reinterpret_cast<uint4*>(dst.out[sh] + row * ldo)[vi] = o;
      if (want_smooth) {
#pragma unroll
        for (int sft = 8; sft > 0; sft >>= 1) hsum += __shfl_xor_sync(0xFFFFFFFFu, hsum, sft, 16);
        const float mean = round_bf16(hsum * (1.f / 128.f));
        uint4 s;
        s.x = pack_bf16x2(__fsub_rn(y[0], mean), __fsub_rn(y[1], mean));
        s.y = pack_bf16x2(__fsub_rn(y[2], mean), __fsub_rn(y[3], mean));
        s.z = pack_bf16x2(__fsub_rn(y[4], mean), __fsub_rn(y[5], mean));
        s.w = pack_bf16x2(__fsub_rn(y[6], mean), __fsub_rn(y[7], mean));
        reinterpret_cast<uint4*>(dst.smooth[sh] + row * lds)[vi] = s;
      }
    }
  }
  if (amax_out) {
    wmax = warp_max(wmax);
    __shared__ float smax[8];
    if (lane == 0) smax[warp] = wmax;
    __syncthreads();
    if (threadIdx.x == 0) {
      float m = smax[0];
#pragma unroll
      for (int i = 1; i < 8; ++i) m = fmaxf(m, smax[i]);
      if (m > 0.f) atomic_max_nonneg(amax_out, m);
    }
  }
}

}  // namespace
}  // namespace llnv

using namespace llnv;

extern "C" int llnv_rmsnorm_rope(const void* x, int64_t S, int64_t C, int64_t ldx, const void* weight, float eps,
                                 const float* cos, const float* sin, void* out, int64_t ldo, void* out_smooth, int64_t lds,
                                 float* amax_out, llnv_stream_t stream) {
  return llnv_rmsnorm_rope_ex(x, S, C, ldx, weight, eps, cos, sin, out, ldo, out_smooth, lds, amax_out, 1, stream);
}

namespace {

int check_job(const RopeJob& jb, int64_t C, int shards) {
  const int64_t Cs = C / shards;
  LLNV_REQUIRE(jb.x != nullptr, "llnv_rmsnorm_rope: null pointer");
  LLNV_REQUIRE(jb.ldx >= C && jb.ldx % 8 == 0 && jb.ldo >= Cs && jb.ldo % 8 == 0, "llnv_rmsnorm_rope: row strides must be >= the row width and multiples of 8");
  LLNV_REQUIRE(((uintptr_t)jb.x & 15) == 0 && ((uintptr_t)jb.weight & 15) == 0, "llnv_rmsnorm_rope: pointers must be 16-byte aligned");
  if (jb.want_smooth) LLNV_REQUIRE(jb.lds >= Cs && jb.lds % 8 == 0, "llnv_rmsnorm_rope: out_smooth row stride must be >= the row width and a multiple of 8");
  for (int r = 0; r < shards; ++r) {
    LLNV_REQUIRE(jb.dst.out[r] != nullptr && ((uintptr_t)jb.dst.out[r] & 15) == 0, "llnv_rmsnorm_rope: output %d must be a 16-byte aligned pointer", r);
    if (jb.want_smooth) LLNV_REQUIRE(jb.dst.smooth[r] != nullptr && ((uintptr_t)jb.dst.smooth[r] & 15) == 0, "llnv_rmsnorm_rope: out_smooth %d must be a 16-byte aligned pointer", r);
  }
  return LLNV_OK;
}

int rope_launch_jobs(const RopeJobs& jobs, int njobs, int64_t S, int64_t C, float eps, const float* cos, const float* sin, int shards,
                     cudaStream_t stream) {
  LLNV_REQUIRE((cos == nullptr) == (sin == nullptr), "llnv_rmsnorm_rope: cos and sin must be given together");
  LLNV_REQUIRE(S >= 0 && C > 0 && C % 128 == 0 && C <= 4096, "llnv_rmsnorm_rope: C must be a multiple of 128 (head_dim 128) and at most 4096 (got %lld)", (long long)C);
  LLNV_REQUIRE(shards >= 1 && shards <= kMaxShards && C % shards == 0 && (C / shards) % 128 == 0,
               "llnv_rmsnorm_rope: shards must divide the channels into whole heads, at most 8 (C=%lld shards=%d)", (long long)C, shards);
  LLNV_REQUIRE(((uintptr_t)cos & 15) == 0 && ((uintptr_t)sin & 15) == 0, "llnv_rmsnorm_rope: pointers must be 16-byte aligned");
  for (int j = 0; j < njobs; ++j) {
    int rc = check_job(jobs.job[j], C, shards);
    if (rc != LLNV_OK) return rc;
    if (jobs.job[j].amax_out && !amax_accumulate(2)) LLNV_CUDA(cudaMemsetAsync(jobs.job[j].amax_out, 0, sizeof(float), stream));
  }
  if (S == 0) return LLNV_OK;
  const int sv = shards > 1 ? (int)(C / shards / 8) : 0;
  // warps per row: as many as leave every warp a whole number of heads and every lane some work
  if (C % 512 == 0 && C >= 2048)
    launch_k(rmsnorm_rope_kernel<4>, dim3((unsigned)((S + 1) / 2), (unsigned)njobs), 256, 0, stream, jobs, S, C, eps, cos, sin, sv);
  else if (C % 256 == 0 && C >= 1024)
    launch_k(rmsnorm_rope_kernel<2>, dim3((unsigned)((S + 3) / 4), (unsigned)njobs), 256, 0, stream, jobs, S, C, eps, cos, sin, sv);
  else
    launch_k(rmsnorm_rope_kernel<1>, dim3((unsigned)((S + 7) / 8), (unsigned)njobs), 256, 0, stream, jobs, S, C, eps, cos, sin, sv);
  return launch_status("rmsnorm_rope_kernel");
}

int rope_launch(const void* x, int64_t S, int64_t C, int64_t ldx, const void* weight, float eps, const float* cos, const float* sin,
                const ShardOut& dst, int64_t ldo, int64_t lds, bool want_smooth, float* amax_out, int shards, cudaStream_t stream) {
  RopeJobs jobs = {};
  jobs.job[0] = RopeJob{(const uint16_t*)x, (const uint16_t*)weight, dst, ldx, ldo, lds, amax_out, want_smooth ? 1 : 0};
  return rope_launch_jobs(jobs, 1, S, C, eps, cos, sin, shards, stream);
}

}  // namespace

extern "C" int llnv_rmsnorm_rope_ex(const void* x, int64_t S, int64_t C, int64_t ldx, const void* weight, float eps,
                                    const float* cos, const float* sin, void* out, int64_t ldo, void* out_smooth, int64_t lds,
                                    float* amax_out, int shards, llnv_stream_t stream) {
  LLNV_REQUIRE(out != nullptr, "llnv_rmsnorm_rope: null pointer");
  LLNV_REQUIRE(shards >= 1 && shards <= kMaxShards, "llnv_rmsnorm_rope: at most 8 shards");
  ShardOut dst = {};
  for (int r = 0; r < shards; ++r) {
    dst.out[r] = (uint16_t*)out + (int64_t)r * S * ldo;
    dst.smooth[r] = out_smooth ? (uint16_t*)out_smooth + (int64_t)r * S * lds : nullptr;
  }
  return rope_launch(x, S, C, ldx, weight, eps, cos, sin, dst, ldo, lds, out_smooth != nullptr, amax_out, shards, (cudaStream_t)stream);
}

extern "C" int llnv_rmsnorm_rope_scatter(const void* x, int64_t S, int64_t C, int64_t ldx, const void* weight, float eps,
                                         const float* cos, const float* sin, void* const* out_ptrs, int64_t ldo,
                                         void* const* smooth_ptrs, int64_t lds, float* amax_out, int shards, llnv_stream_t stream) {
  LLNV_REQUIRE(out_ptrs != nullptr, "llnv_rmsnorm_rope_scatter: null pointer table");
  LLNV_REQUIRE(shards >= 1 && shards <= kMaxShards, "llnv_rmsnorm_rope: at most 8 shards");
  ShardOut dst = {};
  for (int r = 0; r < shards; ++r) {
    dst.out[r] = (uint16_t*)out_ptrs[r];
    dst.smooth[r] = smooth_ptrs ? (uint16_t*)smooth_ptrs[r] : nullptr;
  }
  return rope_launch(x, S, C, ldx, weight, eps, cos, sin, dst, ldo, lds, smooth_ptrs != nullptr, amax_out, shards, (cudaStream_t)stream);
}

extern "C" int llnv_rmsnorm_rope_qk(const void* xq, int64_t ldxq, const void* wq, void* const* q_ptrs, int64_t ldq, const void* xk,
                                    int64_t ldxk, const void* wk, void* const* k_ptrs, int64_t ldk, void* const* k_smooth_ptrs,
                                    int64_t lds, float* k_amax, int64_t S, int64_t C, float eps, const float* cos, const float* sin,
                                    int shards, llnv_stream_t stream) {
  LLNV_REQUIRE(q_ptrs != nullptr && k_ptrs != nullptr, "llnv_rmsnorm_rope_qk: null pointer table");
  LLNV_REQUIRE(shards >= 1 && shards <= kMaxShards, "llnv_rmsnorm_rope: at most 8 shards");
  RopeJobs jobs = {};
  ShardOut dq = {}, dk = {};
  for (int r = 0; r < shards; ++r) {
    dq.out[r] = (uint16_t*)q_ptrs[r];
    dk.out[r] = (uint16_t*)k_ptrs[r];
    dk.smooth[r] = k_smooth_ptrs ? (uint16_t*)k_smooth_ptrs[r] : nullptr;
  }
  jobs.job[0] = RopeJob{(const uint16_t*)xq, (const uint16_t*)wq, dq, ldxq, ldq, 0, nullptr, 0};
  jobs.job[1] = RopeJob{(const uint16_t*)xk, (const uint16_t*)wk, dk, ldxk, ldk, lds, k_amax, k_smooth_ptrs ? 1 : 0};
  return rope_launch_jobs(jobs, 2, S, C, eps, cos, sin, shards, (cudaStream_t)stream);
}
