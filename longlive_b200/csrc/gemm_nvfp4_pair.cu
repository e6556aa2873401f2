// W4A4 GEMM on CTA pairs (tcgen05 cta_group::2): one 256 x 256 output tile per pair of SMs.
//
// Why pairs: with one CTA per tile the kernel is limited by the L2 -> shared-memory operand stream
// (a 128 x 256 tile needs 54 KB per 256-element K block).  In a pair each CTA loads its own 128 rows
// of A but only half of the B tile, and the tensor cores of both SMs read both halves, so the
// operand stream per CTA drops to 38 KB per K block for the same work.  Every CTA loads its own
// tiles with plain TMA loads; the only cross-CTA traffic is the B operand fetch done by the MMA
// hardware and mbarrier arrivals.
//
// Each 256-column tile is computed as two 128-column halves with separate accumulators, and three
// 128-column accumulator buffers rotate (3 x 128 + 48 scale columns <= 512 TMEM columns), so the
// epilogue of a half overlaps the MMAs that follow it.
//
// Roles per CTA (6 warps): warp 0 TMA producer (both CTAs), warp 1 MMA issuer (leader CTA only;
// owns the TMEM allocation in both), warps 2-5 epilogue (both CTAs, own 128 rows each).
// Barriers: full[s] lives in the leader and collects the transaction bytes of both CTAs' loads;
// empty[s] and tmem_full[b] exist in both CTAs and are signalled by tcgen05.commit from the leader
// (one commit per CTA, addressed through the cluster window); tmem_empty[b] lives in the leader and
// counts the eight epilogue warps of the pair.  All waits are bounded.
#include "gemm_common.cuh"

namespace llnv {
namespace {

using namespace sm100;
using namespace gemm;

constexpr int kThreads = 192;
constexpr int kStages = 5;
constexpr uint32_t kABytes = 128 * 128;          // 128 rows x 256 E2M1
constexpr uint32_t kBBytes = 128 * 128;          // two halves of 64 rows
constexpr uint32_t kSfaBytes = 2048;             // 4 atoms (one per K = 64 step)
constexpr uint32_t kSfbBytes = 4096;             // 2 column halves x 4 atoms
constexpr uint32_t kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;     // 38912
constexpr uint32_t kStagingOff = kStages * kStageBytes;
constexpr uint32_t kStagingBytes = 4 * 2 * 4096;
constexpr uint32_t kBarOff = kStagingOff + kStagingBytes;
constexpr uint32_t kSmemBytes = kBarOff + 1024;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccBufs = 3;
constexpr uint32_t kSfaCol = 384, kSfbCol = 400;
static_assert(kStageBytes % 1024 == 0, "stage must keep 1024-byte alignment");
static_assert(kSmemBytes <= 232448, "more shared memory than one CTA may use");

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_nvfp4_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB,
                       const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmR, const GemmParams p) {
  pdl_wait();
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kBarOff);     // used in the leader only
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tfull_bar = empty_bar + kStages;                            // [3]
  uint64_t* tempty_bar = tfull_bar + kAccBufs;                          // [3], used in the leader only
  uint64_t* res_bar = tempty_bar + kAccBufs;                            // [4 warps][2 buffers]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(res_bar + 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();            // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  const int num_m = (int)((p.M + 255) / 256);
  const int num_n = (int)(p.N / 256);
  const int num_tiles = num_m * num_n;
  const int num_kb = (int)(p.K / 256);
  const int64_t k_atoms = p.K / 64;

  if ((smem_u32(smem) & 1023u) != 0) {
    // both CTAs of a pair see the same alignment, so both leave here and nobody waits for the other
    if (threadIdx.x == 0 && p.status && atomicCAS(p.status, 0u, 2u) == 0u) p.status[1] = 902u;
    return;
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < (int)kAccBufs; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 8);
    }
    for (int i = 0; i < 8; ++i) mbar_init(&res_bar[i], 1);
    *abort_flag = 0u;
    fence_barrier_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
    prefetch_tensormap(&tmSFA);
    prefetch_tensormap(&tmSFB);
    prefetch_tensormap(&tmD);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();                                     // the peer's barriers are initialised from here on
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = pair; tile < num_tiles; tile += num_pairs) {
        const int mt = tile % num_m, nt = tile / num_m;
        const int a_row = mt * 256 + (int)rank * 128;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_spin(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, 100u);
          uint8_t* st = smem + stage * kStageBytes;
          // the leader posts the byte count of both CTAs' loads of this stage
          if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * kStageBytes);
          tma_load_2d_pair(st, &tmA, kb * 128, a_row, &full_bar[stage]);
#pragma unroll
          for (int h = 0; h < 2; ++h)     // my 64 rows of each 128-column half of the B tile
            tma_load_2d_pair(st + kABytes + h * 8192, &tmB, kb * 128, nt * 256 + h * 128 + (int)rank * 64, &full_bar[stage]);
          // scale atoms: 2 KB runs of 4 atoms, addressed as rows of 256 bytes
          tma_load_2d_pair(st + kABytes + kBBytes, &tmSFA, 0, (int)((((int64_t)mt * 2 + rank) * k_atoms + kb * 4) * 2), &full_bar[stage]);
#pragma unroll
          for (int h = 0; h < 2; ++h)
            tma_load_2d_pair(st + kABytes + kBBytes + kSfaBytes + h * 2048, &tmSFB, 0,
                             (int)((((int64_t)nt * 2 + h) * k_atoms + kb * 4) * 2), &full_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (rank == 0 && elect_one()) {
      constexpr uint32_t idesc = make_idesc_nvf4(256, 128);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t use = 0;                                // running count of accumulator uses (2 per tile)
      for (int tile = pair; tile < num_tiles; tile += num_pairs) {
        const uint32_t b0 = use % kAccBufs, b1 = (use + 1) % kAccBufs;
        const uint32_t ph0 = (use / kAccBufs) & 1u, ph1 = ((use + 1) / kAccBufs) & 1u;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_spin(&full_bar[stage], phase, abort_flag, p.status, 201u);
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * kStageBytes);
          const uint32_t b_addr = a_addr + kABytes;
          const uint32_t sfa_addr = b_addr + kBBytes;
          const uint32_t sfb_addr = sfa_addr + kSfaBytes;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            tmem_cp_sf_pair(tmem_base + kSfaCol + 4 * g, make_sf_desc(sfa_addr + g * 512));
#pragma unroll
            for (int h = 0; h < 2; ++h)
              tmem_cp_sf_pair(tmem_base + kSfbCol + 16 * h + 4 * g, make_sf_desc(sfb_addr + h * 2048 + g * 512));
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (kb == 0) {
              // the accumulator buffer of this half must have been drained by both CTAs' epilogues
              mbar_wait(&tempty_bar[h ? b1 : b0], (h ? ph1 : ph0) ^ 1u, abort_flag, p.status, 200u);
              tc_fence_after();
            }
            const uint32_t d_tmem = tmem_base + (h ? b1 : b0) * 128;
            const uint64_t a_desc = make_kmajor_sw128_desc(a_addr);
            const uint64_t b_desc = make_kmajor_sw128_desc(b_addr + h * 8192);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_nvf4_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, tmem_base + kSfaCol + 4 * k,
                            tmem_base + kSfbCol + 16 * h + 4 * k, (kb | k) != 0 ? 1u : 0u);
            if (kb == num_kb - 1) {
              // this half is complete: hand its accumulator to the epilogue warps of both CTAs
              tc_commit_pair_addr(mapa_u32(&tfull_bar[h ? b1 : b0], 0));
              tc_commit_pair_addr(mapa_u32(&tfull_bar[h ? b1 : b0], 1));
            }
          }
          // release the shared-memory stage in both CTAs
          tc_commit_pair_addr(mapa_u32(&empty_bar[stage], 0));
          tc_commit_pair_addr(mapa_u32(&empty_bar[stage], 1));
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        use += 2;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int q = warp & 3;
    float alpha;
    if (p.epi.alpha) alpha = __ldg(p.epi.alpha);
    else alpha = __fdiv_rn(__fmul_rn(__ldg(p.a_amax), __ldg(p.b_amax)), p.alpha_denom);
    const uint16_t* bias = reinterpret_cast<const uint16_t*>(p.epi.bias);
    constexpr bool has_res = (EPI & kEpiRes) != 0;
    const uint16_t* gate = reinterpret_cast<const uint16_t*>(p.epi.gate);
    uint8_t* my_stage = smem + kStagingOff + q * 8192;
    uint64_t* my_res_bar = res_bar + q * 2;
    uint32_t res_phase = 0u;
    float local_amax = 0.f;
    uint32_t use = 0, chunk = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs) {
      const int mt = tile % num_m, nt = tile / num_m;
      const int row0 = mt * 256 + (int)rank * 128 + q * 32;
      const int64_t row = (int64_t)row0 + lane;
      const bool row_ok = row < p.M;
      const uint16_t* grow = nullptr;
      if (gate && row_ok) grow = gate + ((row + p.epi.row_offset) / p.epi.frame_rows) * p.epi.gate_stride;
      for (int h = 0; h < 2; ++h, ++use) {
        const uint32_t b = use % kAccBufs;
        if (has_res && row0 < p.M && lane == 0) {
          const uint32_t b0 = chunk & 1u;
          bulk_wait_read<1>();
          mbar_arrive_expect_tx(&my_res_bar[b0], 4096);
          tma_load_2d(my_stage + b0 * 4096, &tmR, nt * 256 + h * 128, row0, &my_res_bar[b0]);
        }
        mbar_wait(&tfull_bar[b], (use / kAccBufs) & 1u, abort_flag, p.status, 300u);
        tc_fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 64, ++chunk) {
          const uint32_t sb = chunk & 1u;
          uint8_t* buf = my_stage + sb * 4096;
          uint32_t r[2][32];
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + b * 128 + c0, r[0]);
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + b * 128 + c0 + 32, r[1]);
          tmem_ld_wait();
          if (c0 + 64 == 128) {
            // buffer fully read: report to the leader's tmem_empty barrier
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster_addr(mapa_u32(&tempty_bar[b], 0));
          }
          if (row0 < p.M) {
            if (has_res) {
              if (c0 + 64 < 128 && lane == 0) {
                bulk_wait_read<0>();
                mbar_arrive_expect_tx(&my_res_bar[sb ^ 1u], 4096);
                tma_load_2d(my_stage + (sb ^ 1u) * 4096, &tmR, nt * 256 + h * 128 + c0 + 64, row0, &my_res_bar[sb ^ 1u]);
              }
              mbar_wait(&my_res_bar[sb], (res_phase >> sb) & 1u, abort_flag, p.status, 301u);
              res_phase ^= 1u << sb;
            } else {
              if (lane == 0) bulk_wait_read<1>();
              __syncwarp();
            }
            const int64_t col = (int64_t)nt * 256 + h * 128 + c0;
            epilogue_chunk<EPI>(r, alpha, bias, grow, col, buf, lane, p.epi.out_amax != nullptr, row_ok, local_amax);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmD, buf, (int)col, row0);
              bulk_commit();
            }
          }
        }
      }
    }
    if (lane == 0) bulk_wait<0>();
    if (p.epi.out_amax) {
      local_amax = warp_max(local_amax);
      if (lane == 0 && local_amax > 0.f) atomic_max_nonneg(p.epi.out_amax, local_amax);
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  cluster_sync();                                     // nobody leaves while the peer may still signal its barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <int EPI>
int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmSFA, const CUtensorMap& tmSFB,
                const CUtensorMap& tmD, const CUtensorMap& tmR, const GemmParams& p, cudaStream_t stream) {
  static bool attr_set[64] = {};
  int dev = 0;
  LLNV_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    LLNV_CUDA(cudaFuncSetAttribute(gemm_nvfp4_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
    attr_set[dev] = true;
  }
  const int64_t tiles = ((p.M + 255) / 256) * (p.N / 256);
  int64_t pairs = sm_count() / 2;
  if (tiles < pairs) pairs = tiles;
  launch_k(gemm_nvfp4_pair_kernel<EPI>, (unsigned)(2 * pairs), kThreads, kSmemBytes, stream, tmA, tmB, tmSFA, tmSFB, tmD, tmR, p);
  return launch_status("gemm_nvfp4_pair_kernel");
}

}  // namespace

// Called by llnv_gemm_nvfp4 (gemm_nvfp4.cu) when the shape suits the pair kernel.
int gemm_nvfp4_pair(const void* a_codes, const void* a_sf, const void* b_codes, const void* b_sf, const gemm::GemmParams& p,
                    const CUtensorMap& tmD, const CUtensorMap& tmR, int variant, cudaStream_t stream) {
  const uint64_t mp = (uint64_t)((p.M + 127) / 128 * 128);
  CUtensorMap tmA, tmB, tmSFA, tmSFB;
  int rc = cached_tensor_map(&tmA, 0, a_codes, mp, (uint64_t)p.K / 2, (uint64_t)p.K / 2, 128, 128, 3);
  if (rc != LLNV_OK) return rc;
  rc = cached_tensor_map(&tmB, 0, b_codes, (uint64_t)p.N, (uint64_t)p.K / 2, (uint64_t)p.K / 2, 64, 128, 3);
  if (rc != LLNV_OK) return rc;
  // scale arrays as rows of 256 bytes (a 512-byte atom = 2 rows), box = 8 rows = the 4 atoms of one K block
  rc = cached_tensor_map(&tmSFA, 0, a_sf, mp * (uint64_t)p.K / 16 / 256, 256, 256, 8, 256, 0);
  if (rc != LLNV_OK) return rc;
  rc = cached_tensor_map(&tmSFB, 0, b_sf, (uint64_t)p.N * (uint64_t)p.K / 16 / 256, 256, 256, 8, 256, 0);
  if (rc != LLNV_OK) return rc;
#define LLNV_PAIR_CASE(V) \
  case V: return launch_pair<V>(tmA, tmB, tmSFA, tmSFB, tmD, tmR, p, stream);
  switch (variant) {
    LLNV_PAIR_CASE(0)
    LLNV_PAIR_CASE(1)
    LLNV_PAIR_CASE(2)
    LLNV_PAIR_CASE(3)
    LLNV_PAIR_CASE(4)
    LLNV_PAIR_CASE(5)
    LLNV_PAIR_CASE(6)
    LLNV_PAIR_CASE(7)
  }
#undef LLNV_PAIR_CASE
  set_error("gemm_nvfp4_pair: internal dispatch error");
  return LLNV_E_INVALID;
}

}  // namespace llnv
