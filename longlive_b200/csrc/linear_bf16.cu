// bf16 Linear for the layers the reference leaves unquantized: D[M, N] = act(A[M, K] . W[N, K]^T + bias).
//
// The NVFP4 filter of the reference keeps the edges of the DiT in bf16 (patch embedding, time and
// text embeddings, time projection, head: wan_5b/modules/causal_model.py:1052-1071, 1535-1573,
// 1648-1651; utils/quant.py filters them out of quantize_model).  They are small GEMMs with one
// long and one short dimension (2640 x 3072 x 192 and 2640 x 192 x 3072 per forward), so this is a
// plain tile kernel, not a persistent one: one CTA per 128 x BN output tile, a TMA ring of
// 128-byte-swizzled K-major tiles of A and W (two 64-channel blocks per stage, so that 256
// contiguous bytes of every operand row are fetched together), tcgen05.mma kind::f16 with
// the fp32 accumulator in TMEM, and an epilogue that adds the bias in fp32, rounds to bf16 (the
// rounding point of the reference's fused-bias GEMM), applies the activation on the rounded value
// (the reference's activation is a separate bf16 op), writes 32 x 64 blocks into shared memory in
// the 128-byte swizzle and hands them to TMA stores.  Rows beyond M and channels beyond K are
// zero-filled by the TMA loads; the TMA stores clip rows beyond M and columns beyond N.  The ring
// depth is chosen per launch: about 100 KB of ring for grids that cover the SMs more than once (two
// CTAs per SM), 192 KB for grids of fewer CTAs than SMs (long K, short N), where each CTA has to
// keep its SM's share of HBM bandwidth busy alone.
//
// Warps: 0 = TMA producer, 1 = TMEM allocation + MMA issue, 2..5 = epilogue (TMEM lane quarter
// warp % 4).  Every wait is bounded (mbar_wait): on a timeout the kernel records where it gave up
// in the status word, the other roles drain, TMEM is freed and the kernel returns.
#include <cuda.h>

#include "common.cuh"
#include "sm100.cuh"

namespace llnv {
namespace {

using namespace sm100;

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float u = k0 * (x + k1 * x * x * x);
  return __fdividef(x, 1.f + __expf(-2.f * u));
}

constexpr int kBM = 128, kBK = 64, kMaxStagesLin = 8, kThreadsLin = 192;
// a stage holds `sub` (1 or 2) consecutive 64-channel blocks of both operands; with 2, 256 contiguous
// bytes of every row are fetched together, which halves the DRAM pages a tile touches per byte (long K)
constexpr int kATile = kBM * kBK * 2;                       // 16 KB per 64-channel block

struct LinParams {
  int64_t M, N, K;
  const uint16_t* bias;
  uint16_t* d;
  int64_t ldd;
  int act;                                                  // 0 none, 1 GELU(tanh), 2 SiLU
  int stages;                                               // ring depth, 1 .. kMaxStagesLin
  int sub;                                                  // 64-channel blocks per stage, 1 or 2
  unsigned int* status;
};

template <int BN>
struct LinCfg {
  static constexpr int kBTile = BN * kBK * 2;
  static constexpr int kBlockBytes = kATile + kBTile;
  // the epilogue reuses the first stage: 4 warps x (BN / 64) blocks of 32 rows x 128 bytes
  static_assert(4 * (BN / 64) * 4096 <= kBlockBytes, "epilogue staging must fit one block of a stage");
  static constexpr int smem_bytes(int blocks) { return blocks * kBlockBytes + 256 + 1024; }   // + barriers + alignment slack
};

__device__ __forceinline__ float silu(float x) { return __fdividef(x, 1.f + __expf(-x)); }

template <int BN>
__global__ void __launch_bounds__(kThreadsLin, 1)
linear_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmD, const LinParams p) {
  pdl_wait();
  using Cfg = LinCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int stages = p.stages, sub = p.sub;
  const int stage_bytes = sub * Cfg::kBlockBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + stages * stage_bytes);
  uint64_t* empty = full + kMaxStagesLin;
  uint64_t* acc_full = empty + kMaxStagesLin;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN;
  const int m0 = blockIdx.y * kBM;
  const int nk = (int)((p.K + sub * kBK - 1) / (sub * kBK));     // stages of `sub` blocks; channels beyond K are zero-filled

  if (threadIdx.x == 0) {
    for (int i = 0; i < stages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0u;
    fence_barrier_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
    prefetch_tensormap(&tmD);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      for (int ks = 0; ks < nk; ++ks) {
        const int s = ks % stages;
        const uint32_t ph = (uint32_t)((ks / stages) & 1);
        if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, p.status, 1100u)) break;
        mbar_arrive_expect_tx(&full[s], stage_bytes);
        for (int u = 0; u < sub; ++u) {
          tma_load_2d(smem + s * stage_bytes + u * Cfg::kBlockBytes, &tmA, (ks * sub + u) * kBK, m0, &full[s]);
          tma_load_2d(smem + s * stage_bytes + u * Cfg::kBlockBytes + kATile, &tmB, (ks * sub + u) * kBK, n0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(kBM, BN, 0, 0);
      bool ok = true;
      for (int ks = 0; ks < nk && ok; ++ks) {
        const int s = ks % stages;
        const uint32_t ph = (uint32_t)((ks / stages) & 1);
        ok = mbar_wait(&full[s], ph, abort_flag, p.status, 1101u);
        if (!ok) break;
        tc_fence_after();
        for (int u = 0; u < sub; ++u) {
          const uint32_t a_addr = smem_u32(smem + s * stage_bytes + u * Cfg::kBlockBytes);
          const uint32_t b_addr = a_addr + kATile;
#pragma unroll
          for (int j = 0; j < 4; ++j)        // 16 channels per MMA = 32 bytes along the swizzled row
            mma_f16_ss(tmem_base, make_kmajor_sw128_desc(a_addr + j * 32), make_kmajor_sw128_desc(b_addr + j * 32), idesc,
                       (uint32_t)((ks | u | j) != 0));
        }
        tc_commit(&empty[s]);
      }
      if (ok) tc_commit(acc_full);
    }
  } else {
    const int q = warp & 3;                                  // TMEM lanes 32 q .. 32 q + 31
    const int row0 = m0 + q * 32;
    if (mbar_wait(acc_full, 0u, abort_flag, p.status, 1102u)) {
      tc_fence_after();
      // every load of the ring has been consumed by now: stage 0 is free for the output blocks
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        uint32_t r[2][32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 64), r[0]);
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 64 + 32), r[1]);
        tmem_ld_wait();
        const int64_t col = (int64_t)n0 + c * 64;
        uint8_t* buf = smem + (q * (BN / 64) + c) * 4096;     // 32 rows x 128 bytes, 128-byte swizzle
#pragma unroll
        for (int v8 = 0; v8 < 8; ++v8) {
          uint32_t w4[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int cc = v8 * 8 + 2 * e;
            float y0 = __uint_as_float(r[cc >> 5][cc & 31]), y1 = __uint_as_float(r[(cc + 1) >> 5][(cc + 1) & 31]);
            if (p.bias) {
              if (col + cc < p.N) y0 += __uint_as_float((uint32_t)__ldg(p.bias + col + cc) << 16);
              if (col + cc + 1 < p.N) y1 += __uint_as_float((uint32_t)__ldg(p.bias + col + cc + 1) << 16);
            }
            if (p.act) {
              round_bf16x2(y0, y1);
              if (p.act == 1) {
                y0 = gelu_tanh(y0);
                y1 = gelu_tanh(y1);
              } else {
                y0 = silu(y0);
                y1 = silu(y1);
              }
            }
            w4[e] = pack_bf16x2(y0, y1);
          }
          *reinterpret_cast<uint4*>(buf + lane * 128 + ((v8 ^ (lane & 7)) << 4)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0 && row0 < p.M && col < p.N) {
          tma_store_2d(&tmD, buf, (int)col, row0);
          bulk_commit();
        }
      }
      if (lane == 0) bulk_wait<0>();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);         // let copies in flight land before the CTA exits
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, BN);
  }
}

template <int BN>
int launch_linear(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD, const LinParams& p, cudaStream_t stream) {
  using Cfg = LinCfg<BN>;
  static bool attr_set[64] = {};
  int dev = 0;
  LLNV_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    LLNV_CUDA(cudaFuncSetAttribute(linear_bf16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::smem_bytes(BN == 128 ? 6 : 8)));
    attr_set[dev] = true;
  }
  const dim3 grid((unsigned)((p.N + BN - 1) / BN), (unsigned)((p.M + kBM - 1) / kBM));
  launch_k(linear_bf16_kernel<BN>, grid, kThreadsLin, (size_t)Cfg::smem_bytes(p.stages * p.sub), stream, tmA, tmB, tmD, p);
  return launch_status("linear_bf16_kernel");
}

}  // namespace
}  // namespace llnv

using namespace llnv;

extern "C" int llnv_linear_bf16(const void* a, int64_t lda, const void* w, int64_t ldw, const void* bias, int act, int64_t M, int64_t N,
                                int64_t K, void* d, int64_t ldd, llnv_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  LLNV_REQUIRE(M >= 0 && N > 0 && K > 0, "llnv_linear_bf16: bad sizes M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
  LLNV_REQUIRE(act >= 0 && act <= 2, "llnv_linear_bf16: act is 0 (none), 1 (GELU tanh) or 2 (SiLU), got %d", act);
  if (M == 0) return LLNV_OK;
  LLNV_REQUIRE(a && w && d, "llnv_linear_bf16: null tensor");
  LLNV_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && lda >= K && ldw >= K,
               "llnv_linear_bf16: K and the row strides of a and w must be multiples of 8 elements (16 bytes)");
  LLNV_REQUIRE(ldd % 8 == 0 && ldd >= N && N % 8 == 0, "llnv_linear_bf16: N and the row stride of d must be multiples of 8 elements");
  LLNV_REQUIRE((((uintptr_t)a | (uintptr_t)w | (uintptr_t)d) & 15) == 0 && ((uintptr_t)bias & 1) == 0,
               "llnv_linear_bf16: a, w and d must be 16-byte aligned");
  LinParams p;
  p.M = M, p.N = N, p.K = K;
  p.bias = (const uint16_t*)bias;
  p.d = (uint16_t*)d;
  p.ldd = ldd;
  p.act = act;
  p.status = device_status_word();

  // narrow tiles when the wide ones would leave most SMs without a CTA
  const int64_t row_tiles = (M + kBM - 1) / kBM;
  const bool narrow = N <= 64 || row_tiles * ((N + 127) / 128) < 2 * (int64_t)sm_count();
  const int64_t ctas = row_tiles * ((N + (narrow ? 63 : 127)) / (narrow ? 64 : 128));
  p.sub = K >= 512 ? 2 : 1;
  const int64_t nk = (K + p.sub * kBK - 1) / (p.sub * kBK);
  const int64_t blocks = ctas <= sm_count() ? (narrow ? 8 : 6) : 4;       // 64-channel blocks the ring may hold (192 KB / 96-128 KB)
  const int64_t deep = blocks / p.sub;
  p.stages = (int)(nk < deep ? nk : deep);
  CUtensorMap tmA, tmB, tmD;
  int rc = cached_tensor_map(&tmA, 1, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, kBM, kBK, 3);
  if (rc != LLNV_OK) return rc;
  rc = cached_tensor_map(&tmB, 1, w, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, narrow ? 64 : 128, kBK, 3);
  if (rc != LLNV_OK) return rc;
  rc = cached_tensor_map(&tmD, 1, d, (uint64_t)M, (uint64_t)N, (uint64_t)ldd, 32, 64, 3);
  if (rc != LLNV_OK) return rc;
  return narrow ? launch_linear<64>(tmA, tmB, tmD, p, stream) : launch_linear<128>(tmA, tmB, tmD, p, stream);
}
