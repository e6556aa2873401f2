// W4A4 GEMM on tcgen05 block-scaled tensor cores (kind::mxf4nvf4, E2M1 operands, UE4M3 scale per
// 16 elements, fp32 accumulators in tensor memory) with a fused epilogue.
//
//   D[M, N] = epilogue(alpha * A[M, K] * B[N, K]^T)
//
// One persistent CTA per SM, 6 warps:
//   warp 0      TMA producer: per 256-element K block it loads the A tile (128 rows x 128 bytes of
//               packed codes), the B tile (BN rows x 128 bytes) with the 128-byte swizzle, and the
//               scale factors of both tiles (already stored as 512-byte 128x4 atoms, so a tile's
//               scales are contiguous runs fetched with untiled bulk copies).
//   warp 1      MMA issuer (one elected lane): copies the scale atoms shared -> tensor memory with
//               tcgen05.cp, then issues four K=64 MMAs per stage; tcgen05.commit releases the
//               stage to the producer and, after the last K block, hands the accumulator to the
//               epilogue.  Warp 1 also owns the TMEM allocation.
//   warps 2-5   epilogue: tcgen05.ld of the fp32 accumulator (32 lanes x 32 columns per load),
//               alpha / bias / GELU / gate*y + residual / amax, bf16 stores.
// BN = 128 and BN = 192 keep two accumulators in tensor memory so the epilogue of a tile overlaps
// the main loop of the next one; BN = 256 has one accumulator (2 x 256 columns + scales exceed the
// 512 columns) but the least shared-memory traffic per flop.  A 192-row B tile starts 0 or 64 rows
// into a 128-row scale atom: both atoms it touches are copied to tensor memory and the MMA's scale
// address starts 0 or 2 columns (32 rows per column) into them.
//
// Every mbarrier wait is bounded (see sm100.cuh); no CTA waits on another CTA.
#include <cuda.h>

#include "gemm_common.cuh"

namespace llnv {
namespace {

using namespace sm100;
using namespace gemm;

constexpr int BM = 128;
constexpr int BK_BYTES = 128;            // 256 E2M1 elements
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;

template <int BN>
struct Cfg {
  static constexpr int kAcc = BN == 256 ? 1 : 2;
  static constexpr int kStages = BN == 128 ? 5 : (BN == 192 ? 4 : 3);
  static constexpr int kSfbAtoms = (BN + 127) / 128;     // 128-row scale atoms a B tile touches (192 rows: always two)
  static constexpr uint32_t kABytes = BM * BK_BYTES;
  static constexpr uint32_t kBBytes = BN * BK_BYTES;
  static constexpr uint32_t kSfaBytes = 2048;
  static constexpr uint32_t kSfbBytes = kSfbAtoms * 2048;
  static constexpr uint32_t kSfbColsPerK = 4 * kSfbAtoms;  // TMEM columns of B scales per K=64 MMA
  static constexpr uint32_t kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  // epilogue staging: per epilogue warp two buffers of 32 rows x 64 bf16 columns (128-byte rows,
  // 128-byte swizzle) that TMA stores drain; the same buffers receive the residual tile first
  // (the single-accumulator tile has one buffer per 64-column chunk, so that the residual of a whole
  // tile can be fetched while its main loop still runs)
  static constexpr int kBufs = kAcc == 1 ? BN / 64 : 2;
  static constexpr uint32_t kStagingBytes = 4 * kBufs * 4096;
  static constexpr uint32_t kStagingOff = kStages * kStageBytes;
  static constexpr uint32_t kBarOff = kStagingOff + kStagingBytes;
  static constexpr uint32_t kSmemBytes = kBarOff + 1024;
  static constexpr uint32_t kSfaCol = kAcc * BN;          // first TMEM column of the A scales
  static constexpr uint32_t kSfbCol = kSfaCol + 16;       // 4 MMAs x 4 columns
  static_assert(kStageBytes % 1024 == 0, "stage must keep 1024-byte alignment");
  static_assert(BN == 128 || BN == 192 || BN == 256, "unsupported tile width");
  static_assert(kSfbCol + 4 * kSfbColsPerK <= kTmemCols, "tensor memory overflow");
};

// GELU, tanh form: 0.5 x (1 + tanh(u)) = x / (1 + exp(-2u)), u = sqrt(2/pi) (x + 0.044715 x^3)
template <int BN, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmR,
                  const __grid_constant__ GroupMaps gmaps, const GemmParams p) {
  pdl_wait();
  using C = Cfg<BN>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::kBarOff);
  uint64_t* empty_bar = full_bar + C::kStages;
  uint64_t* tfull_bar = empty_bar + C::kStages;
  uint64_t* tempty_bar = tfull_bar + C::kAcc;
  uint64_t* res_bar = tempty_bar + C::kAcc;                 // [4 warps][2 buffers]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(res_bar + 16);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int num_m = (int)((p.M + BM - 1) / BM);
  const int num_n = (int)(p.N / BN);
  const int num_tiles = num_m * num_n;
  const int num_kb = (int)(p.K / 256);
  const int64_t k_atoms = p.K / 64;       // 512-byte scale atoms per 128-row tile

  if ((smem_u32(smem) & 1023u) != 0) {    // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0 && p.status && atomicCAS(p.status, 0u, 2u) == 0u) p.status[1] = 900u;
    return;
  }

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < C::kAcc; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 4);
    }
    for (int i = 0; i < 16; ++i) mbar_init(&res_bar[i], 1);
    *abort_flag = 0u;
    fence_barrier_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
    prefetch_tensormap(&tmD);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // Both pipeline threads walk the K blocks in groups of kStages with the stage index a
    // compile-time constant (and one phase bit per stage), so that every shared-memory address,
    // barrier address and descriptor below is loop-invariant: the single issuing thread of each
    // role is on the critical path of every K block.
    if (elect_one()) {
      uint32_t phases = 0;                   // bit s: parity the stage's empty barrier completed last
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int mt = tile % num_m, nt = tile / num_m;
        const uint8_t* sfa_src = p.sfa + (int64_t)mt * k_atoms * 512;
        const uint8_t* sfb_src = p.sfb + (((int64_t)nt * BN) / 128) * k_atoms * 512;      // first scale atom row of the B tile
        for (int kb0 = 0; kb0 < num_kb; kb0 += C::kStages) {
#pragma unroll
          for (int s = 0; s < C::kStages; ++s) {
            const int kb = kb0 + s;
            if (kb >= num_kb) break;
            mbar_wait(&empty_bar[s], ((phases >> s) & 1u) ^ 1u, abort_flag, p.status, 100u);
            phases ^= 1u << s;
            uint8_t* st = smem + s * C::kStageBytes;
            mbar_arrive_expect_tx(&full_bar[s], C::kStageBytes);
            tma_load_2d(st, &tmA, kb * BK_BYTES, mt * BM, &full_bar[s]);
            tma_load_2d(st + C::kABytes, &tmB, kb * BK_BYTES, nt * BN, &full_bar[s]);
            bulk_load(st + C::kABytes + C::kBBytes, sfa_src + (int64_t)kb * 2048, 2048, &full_bar[s]);
#pragma unroll
            for (int h = 0; h < C::kSfbAtoms; ++h)
              bulk_load(st + C::kABytes + C::kBBytes + C::kSfaBytes + h * 2048, sfb_src + ((int64_t)h * k_atoms + kb * 4) * 512, 2048,
                        &full_bar[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_nvf4(BM, BN);
      // upper words of the shared-memory descriptors (stride between 8-row groups, version, layout) are constants;
      // the lower word is (address >> 4) | (leading-dimension field << 16)
      constexpr uint32_t kOpHi = (uint32_t)(make_smem_desc(0, 16, 1024, 2) >> 32);
      constexpr uint32_t kSfHi = (uint32_t)(make_smem_desc(0, 0, 128, 0) >> 32);
      const uint32_t smem_base = smem_u32(smem);
      int acc = 0;
      uint32_t phases = 0, acc_phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_flag, p.status, 200u);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int nt = tile / num_m;
        const uint32_t sfb_col0 = (uint32_t)((((int64_t)nt * BN) % 128) / 32);     // tile start inside its first scale atom
        for (int kb0 = 0; kb0 < num_kb; kb0 += C::kStages) {
#pragma unroll
          for (int s = 0; s < C::kStages; ++s) {
            const int kb = kb0 + s;
            if (kb >= num_kb) break;
            mbar_wait(&full_bar[s], (phases >> s) & 1u, abort_flag, p.status, 201u);
            phases ^= 1u << s;
            tc_fence_after();
            const uint32_t a_lo = ((smem_base + s * C::kStageBytes) >> 4) | (1u << 16);
            const uint32_t b_lo = a_lo + (C::kABytes >> 4);
            const uint32_t sfa_lo = (smem_base + s * C::kStageBytes + C::kABytes + C::kBBytes) >> 4;
            const uint32_t sfb_lo = sfa_lo + (C::kSfaBytes >> 4);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              tmem_cp_sf(tmem_base + C::kSfaCol + 4 * g, ((uint64_t)kSfHi << 32) | (sfa_lo + 32 * g));
#pragma unroll
              for (int h = 0; h < C::kSfbAtoms; ++h)
                tmem_cp_sf(tmem_base + C::kSfbCol + C::kSfbColsPerK * g + 4 * h, ((uint64_t)kSfHi << 32) | (sfb_lo + 128 * h + 32 * g));
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              // 64 E2M1 elements = 32 bytes further along K inside the 128-byte swizzled row
              mma_nvf4(d_tmem, ((uint64_t)kOpHi << 32) | (a_lo + 2 * k), ((uint64_t)kOpHi << 32) | (b_lo + 2 * k), idesc,
                       tmem_base + C::kSfaCol + 4 * k, tmem_base + C::kSfbCol + C::kSfbColsPerK * k + sfb_col0, (kb | k) != 0 ? 1u : 0u);
            }
            tc_commit(&empty_bar[s]);
          }
        }
        tc_commit(&tfull_bar[acc]);
        if (++acc == C::kAcc) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;                           // TMEM lane quarter this warp may access
    float alpha0, alpha1 = 0.f, alpha2 = 0.f;           // per weight group (one group unless p.group_cols)
    if (p.epi.alpha) alpha0 = __ldg(p.epi.alpha);
    else alpha0 = __fdiv_rn(__fmul_rn(__ldg(p.a_amax), __ldg(p.b_amax)), p.alpha_denom);
    if (p.group_cols) {
      alpha1 = __fdiv_rn(__fmul_rn(__ldg(p.a_amax), __ldg(p.b_amax + 1)), p.alpha_denom);
      if (p.N >= 3 * p.group_cols) alpha2 = __fdiv_rn(__fmul_rn(__ldg(p.a_amax), __ldg(p.b_amax + 2)), p.alpha_denom);
    }
    float amax0 = 0.f, amax1 = 0.f, amax2 = 0.f;
    quant::QuantConsts qconsts = {};
    if constexpr ((EPI & kEpiQuant) != 0) qconsts = quant::make_consts<LLNV_RULE_MSE>(__ldg(p.q_amax));
    const uint16_t* bias = reinterpret_cast<const uint16_t*>(p.epi.bias);
    constexpr bool has_res = (EPI & kEpiRes) != 0;
    const uint16_t* gate = reinterpret_cast<const uint16_t*>(p.epi.gate);
    uint8_t* my_stage = smem + C::kStagingOff + q * C::kBufs * 4096;
    uint64_t* my_res_bar = res_bar + q * C::kBufs;
    uint32_t res_phase = 0u;                          // bit b = parity to wait for on buffer b
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t chunk = 0;                               // running chunk counter -> staging buffer
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const int mt = tile % num_m, nt = tile / num_m;
      const int row0 = mt * BM + q * 32;              // first row of this warp
      const int64_t row = (int64_t)row0 + lane;
      const bool row_ok = row < p.M;
      const uint16_t* grow = nullptr;
      if (gate && row_ok) grow = gate + ((row + p.epi.row_offset) / p.epi.frame_rows) * p.epi.gate_stride;
      // weight group of this tile: its scale, its output matrix, its amax target
      const int grp = p.group_cols ? (int)(((int64_t)nt * BN) / p.group_cols) : 0;
      const int64_t gcol0 = (int64_t)grp * p.group_cols;
      const float alpha = grp == 0 ? alpha0 : (grp == 1 ? alpha1 : alpha2);
      const CUtensorMap* tm_out = grp == 0 ? &tmD : &gmaps.m[grp - 1];
      const float* amax_dst = grp == 0 ? p.group_amax[0] : (grp == 1 ? p.group_amax[1] : p.group_amax[2]);
      const bool want_amax = p.group_cols ? amax_dst != nullptr : p.epi.out_amax != nullptr;
      float local_amax = 0.f;
      if (C::kAcc == 1) {
        // one buffer per chunk: once the previous tile's stores have read them, the residual of the
        // whole tile is fetched while the main loop is still running
        if (row0 < p.M && lane == 0) {
          bulk_wait_read<0>();
          if (has_res) {
#pragma unroll
            for (int ci = 0; ci < C::kBufs; ++ci) {
              mbar_arrive_expect_tx(&my_res_bar[ci], 4096);
              tma_load_2d(my_stage + ci * 4096, &tmR, nt * BN + ci * 64, row0, &my_res_bar[ci]);
            }
          }
        }
        __syncwarp();
      } else if (has_res && row0 < p.M) {
        // residual tile of the first chunk can be fetched while the main loop is still running
        const uint32_t b0 = chunk & 1u;
        if (lane == 0) {
          bulk_wait_read<1>();                        // the store that used this buffer two chunks ago has read it
          mbar_arrive_expect_tx(&my_res_bar[b0], 4096);
          tma_load_2d(my_stage + b0 * 4096, &tmR, nt * BN, row0, &my_res_bar[b0]);
        }
      }
      mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, 300u);
      tc_fence_after();
      // everything after the accumulator has been drained: residual wait, epilogue math, staging, store
      auto finish_chunk = [&](int c0, const uint32_t (&pkc)[32]) {
        const uint32_t b = C::kAcc == 1 ? (uint32_t)(c0 >> 6) : (chunk & 1u);
        uint8_t* buf = my_stage + b * 4096;
        if (row0 < p.M) {
          if (C::kAcc == 1) {
            if (has_res) {
              mbar_wait(&my_res_bar[b], (res_phase >> b) & 1u, abort_flag, p.status, 301u);
              res_phase ^= 1u << b;
            }
          } else if (has_res) {
            // prefetch the residual of the next chunk of this tile into the other buffer
            if (c0 + 64 < BN && lane == 0) {
              bulk_wait_read<0>();
              mbar_arrive_expect_tx(&my_res_bar[b ^ 1u], 4096);
              tma_load_2d(my_stage + (b ^ 1u) * 4096, &tmR, nt * BN + c0 + 64, row0, &my_res_bar[b ^ 1u]);
            }
            mbar_wait(&my_res_bar[b], (res_phase >> b) & 1u, abort_flag, p.status, 301u);
            res_phase ^= 1u << b;
          } else {
            if (lane == 0) bulk_wait_read<1>();       // buffer b was last used two chunks ago
            __syncwarp();
          }
          const int64_t col = (int64_t)nt * BN + c0;
          if constexpr ((EPI & kEpiQuant) != 0) {
            // codes [Mp, N/2] row-major; scales in 512-byte atoms of 128 rows x 4 scale columns (64 elements)
            QuantOut qo;
            qo.qc = qconsts;
            qo.codes = p.q_codes + row * (p.N >> 1) + (col >> 1);
            qo.sf = reinterpret_cast<uint32_t*>(p.q_sf + ((int64_t)mt * (p.N >> 6) + (col >> 6)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4);
            epilogue_packed<EPI>(pkc, bias, grow, col, buf, lane, want_amax, row_ok, local_amax, &qo, p.store_bf16 != 0);
          } else {
            epilogue_packed<EPI>(pkc, bias, grow, col, buf, lane, want_amax, row_ok, local_amax);
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0 && ((EPI & kEpiQuant) == 0 || p.store_bf16)) {
            tma_store_2d(tm_out, buf, (int)(col - gcol0), row0);  // rows beyond M are clipped by the tensor map
            bulk_commit();
          }
        } else if constexpr ((EPI & kEpiQuant) != 0) {
          // a group of 32 padding rows (M..Mp-1): zero codes and zero scales, as the standalone quantizer writes them
          const int64_t col = (int64_t)nt * BN + c0;
          uint4* cz = reinterpret_cast<uint4*>(p.q_codes + row * (p.N >> 1) + (col >> 1));
          cz[0] = make_uint4(0u, 0u, 0u, 0u);
          cz[1] = make_uint4(0u, 0u, 0u, 0u);
          *reinterpret_cast<uint32_t*>(p.q_sf + ((int64_t)mt * (p.N >> 6) + (col >> 6)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4) = 0u;
        }
      };
      const uint32_t acc_tmem = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      if constexpr (C::kAcc == 1) {
        // Single accumulator: drain all of it first (alpha, round to bf16, pack: 32 registers per 64
        // columns) and hand it back to the MMA warp, so that the next tile's main loop runs while
        // this tile's epilogue math, residual waits and stores are still in progress.
        constexpr int kChunks = BN / 64;
        uint32_t pk[kChunks][32];
#pragma unroll
        for (int ci = 0; ci < kChunks; ++ci) {
          uint32_t r[2][32];
          tmem_ld32(acc_tmem + ci * 64, r[0]);
          tmem_ld32(acc_tmem + ci * 64 + 32, r[1]);
          tmem_ld_wait();
          drain_chunk(r, alpha, pk[ci]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[acc]);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 64, ++chunk) {
          finish_chunk(c0, pk[0]);
          // rotate the packed chunks so that the rolled loop always reads pk[0] (static register indices)
#pragma unroll
          for (int ci = 0; ci + 1 < kChunks; ++ci)
#pragma unroll
            for (int i = 0; i < 32; ++i) pk[ci][i] = pk[ci + 1][i];
        }
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 64, ++chunk) {
          uint32_t r[2][32];
          tmem_ld32(acc_tmem + c0, r[0]);
          tmem_ld32(acc_tmem + c0 + 32, r[1]);
          tmem_ld_wait();
          if (c0 + 64 == BN) {
            // accumulator fully read: hand it back to the MMA warp before the math and the stores
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty_bar[acc]);
          }
          uint32_t pkc[32];
          drain_chunk(r, alpha, pkc);
          finish_chunk(c0, pkc);
        }
      }
      if (grp == 0) amax0 = fmaxf(amax0, local_amax);
      else if (grp == 1) amax1 = fmaxf(amax1, local_amax);
      else amax2 = fmaxf(amax2, local_amax);
      if (++acc == C::kAcc) { acc = 0; acc_phase ^= 1u; }
    }
    if (lane == 0) bulk_wait<0>();
    if (p.group_cols) {
      const float am[3] = {warp_max(amax0), warp_max(amax1), warp_max(amax2)};
#pragma unroll
      for (int g = 0; g < 3; ++g)
        if (lane == 0 && p.group_amax[g] && am[g] > 0.f) atomic_max_nonneg(p.group_amax[g], am[g]);
    } else if (p.epi.out_amax) {
      amax0 = warp_max(amax0);
      if (lane == 0 && amax0 > 0.f) atomic_max_nonneg(p.epi.out_amax, amax0);
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // a wait gave up: give copies that may still be in flight time to land before shared memory
    // and tensor memory are released
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host side ------------------------------------------------------------------------------

int get_codes_map(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
  return cached_tensor_map(out, 0, ptr, rows, row_bytes, row_bytes, box_rows, BK_BYTES, 3);
}

int get_out_map(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t pitch) {
  return cached_tensor_map(out, 1, ptr, rows, cols, pitch, 32, 64, 3);
}

template <int BN, int EPI>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD, const CUtensorMap& tmR,
           const GemmParams& p, cudaStream_t stream, const GroupMaps& gmaps) {
  static bool attr_set[64] = {};
  int dev = 0;
  LLNV_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    LLNV_CUDA(cudaFuncSetAttribute(gemm_nvfp4_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<BN>::kSmemBytes));
    attr_set[dev] = true;
  }
  const int64_t tiles = ((p.M + BM - 1) / BM) * (p.N / BN);
  const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  launch_k(gemm_nvfp4_kernel<BN, EPI>, grid, kThreads, Cfg<BN>::kSmemBytes, stream, tmA, tmB, tmD, tmR, gmaps, p);
  return launch_status("gemm_nvfp4_kernel");
}

}  // namespace

int gemm_nvfp4_pair(const void* a_codes, const void* a_sf, const void* b_codes, const void* b_sf, const gemm::GemmParams& p,
                    const CUtensorMap& tmD, const CUtensorMap& tmR, int variant, cudaStream_t stream);
}  // namespace llnv

using namespace llnv;

namespace {

// groups == 1: one GEMM into d.  groups == 2 or 3: B holds that many weight matrices of N / groups rows
// each, b_amax one tensor amax per matrix; matrix g is written to d_groups[g] (row stride ldd_groups[g])
// and its output amax, if wanted, to amax_groups[g].
int gemm_run(const void* a_codes, const void* a_sf, const float* a_amax, int a_rule, const void* b_codes, const void* b_sf,
             const float* b_amax, int b_rule, int64_t M, int64_t N, int64_t K, const llnv_epilogue_t* epilogue, void* d, int64_t ldd,
             cudaStream_t stream, int groups, void* const* d_groups, const int64_t* ldd_groups, float* const* amax_groups, int tile) {
  LLNV_REQUIRE(a_codes && a_sf && b_codes && b_sf, "llnv_gemm_nvfp4: null pointer");
  LLNV_REQUIRE(M >= 0 && N > 0 && K > 0, "llnv_gemm_nvfp4: bad shape M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
  LLNV_REQUIRE(N % 128 == 0, "llnv_gemm_nvfp4: N must be a multiple of 128 (got %lld)", (long long)N);
  LLNV_REQUIRE(K % 256 == 0, "llnv_gemm_nvfp4: K must be a multiple of 256 (got %lld)", (long long)K);
  LLNV_REQUIRE(d == nullptr || (ldd >= N / groups && ldd % 8 == 0 && ((uintptr_t)d & 15) == 0), "llnv_gemm_nvfp4: d must be 16-byte aligned with ldd a multiple of 8");
  LLNV_REQUIRE(((uintptr_t)a_sf & 15) == 0 && ((uintptr_t)b_sf & 15) == 0, "llnv_gemm_nvfp4: scale arrays must be 16-byte aligned");
  LLNV_REQUIRE(a_rule >= 0 && a_rule <= 4 && b_rule >= 0 && b_rule <= 4, "llnv_gemm_nvfp4: unknown scale rule");
  LLNV_REQUIRE(tile == LLNV_GEMM_TILE_AUTO || tile == LLNV_GEMM_TILE_PAIR || tile == 128 || tile == 192 || tile == 256,
               "llnv_gemm_nvfp4: tile must be 0 (automatic), 128, 192, 256 or LLNV_GEMM_TILE_PAIR (got %d)", tile);
  
  llnv_epilogue_t epi;
  memset(&epi, 0, sizeof(epi));
  if (epilogue) epi = *epilogue;
  LLNV_REQUIRE(epi.alpha || (a_amax && b_amax), "llnv_gemm_nvfp4: need alpha or both amax pointers");
  LLNV_REQUIRE(epi.act == 0 || epi.act == 1, "llnv_gemm_nvfp4: unknown activation %d", epi.act);
  if (epi.residual) LLNV_REQUIRE(epi.ldr >= N, "llnv_gemm_nvfp4: residual row stride smaller than N");
  if (epi.bias) LLNV_REQUIRE(((uintptr_t)epi.bias & 15) == 0, "llnv_gemm_nvfp4: bias must be 16-byte aligned");
  if (epi.gate) LLNV_REQUIRE(((uintptr_t)epi.gate & 15) == 0 && epi.gate_stride % 8 == 0, "llnv_gemm_nvfp4: gate must be 16-byte aligned with a stride that is a multiple of 8");
  if (epi.gate) LLNV_REQUIRE(epi.residual && epi.frame_rows > 0 && epi.gate_stride >= N, "llnv_gemm_nvfp4: gate needs residual, frame_rows > 0 and gate_stride >= N");
  const bool requant = epi.q_codes != nullptr;
  if (requant) {
    LLNV_REQUIRE(epi.q_sf && epi.q_amax, "llnv_gemm_nvfp4: requantized output needs q_codes, q_sf and q_amax");
    LLNV_REQUIRE(epi.q_rule == LLNV_RULE_MSE, "llnv_gemm_nvfp4: the epilogue requantizes with the 4-over-6 MSE rule only (got rule %d)", epi.q_rule);
    LLNV_REQUIRE(!epi.residual && groups == 1, "llnv_gemm_nvfp4: requantized output cannot be combined with a residual or a grouped launch");
    LLNV_REQUIRE(((uintptr_t)epi.q_codes & 15) == 0 && ((uintptr_t)epi.q_sf & 3) == 0, "llnv_gemm_nvfp4: q_codes must be 16-byte, q_sf 4-byte aligned");
    LLNV_REQUIRE(N % 64 == 0, "llnv_gemm_nvfp4: requantized output needs N %% 64 == 0");
  }
  LLNV_REQUIRE(d != nullptr || requant, "llnv_gemm_nvfp4: null output pointer");
  if (M == 0) return LLNV_OK;

  const int64_t group_cols = groups > 1 ? N / groups : 0;
  int bn = (N % 256 == 0 && (groups == 1 || group_cols % 256 == 0)) ? 256 : 128;
  // few tokens (a sequence-parallel shard): 256-wide tiles would leave SMs idle, 128-wide tiles double the grid
  if (bn == 256 && ((M + 127) / 128) * (N / 256) * 2 <= (int64_t)sm_count() + 8) bn = 128;
  // less than one wave of 256-wide tiles: 192-wide ones fill more SMs (and overlap their epilogue
  // with the next main loop); with more tiles the lower operand traffic of the 256-wide tile wins
  else if (bn == 256 && N % 192 == 0 && (groups == 1 || group_cols % 192 == 0) && ((M + 127) / 128) * (N / 256) <= (int64_t)sm_count()) bn = 192;
  if (tile == 128) bn = 128;
  if (tile == 192 && N % 192 == 0 && (groups == 1 || group_cols % 192 == 0)) bn = 192;
  if (tile == 256 && N % 256 == 0 && (groups == 1 || group_cols % 256 == 0)) bn = 256;

  const uint64_t mp = (uint64_t)((M + 127) / 128 * 128);
  CUtensorMap tmA, tmB;
  int rc = get_codes_map(&tmA, a_codes, mp, (uint64_t)K / 2, BM);
  if (rc != LLNV_OK) return rc;
  rc = get_codes_map(&tmB, b_codes, (uint64_t)N, (uint64_t)K / 2, (uint32_t)bn);
  if (rc != LLNV_OK) return rc;

  GemmParams p;
  p.sfa = (const uint8_t*)a_sf;
  p.sfb = (const uint8_t*)b_sf;
  p.a_amax = a_amax;
  p.b_amax = b_amax;
  p.alpha_denom = rule_e2m1_max(a_rule) * rule_e4m3_max(a_rule) * rule_e2m1_max(b_rule) * rule_e4m3_max(b_rule);
  p.M = M;
  p.N = N;
  p.K = K;
  p.epi = epi;
  p.d = (__nv_bfloat16*)d;
  p.ldd = ldd;
  p.status = device_status_word();
  p.q_codes = (uint8_t*)epi.q_codes;
  p.q_sf = (uint8_t*)epi.q_sf;
  p.q_amax = epi.q_amax;
  p.store_bf16 = d != nullptr ? 1 : 0;
  if (d == nullptr) {           // the output map is never used; describe the codes buffer so that the encode succeeds
    d = epi.q_codes;
    ldd = N;
  }
  CUtensorMap tmD, tmR;
  GroupMaps gmaps;
  memset(&gmaps, 0, sizeof(gmaps));
  p.group_cols = group_cols;
  for (int g = 0; g < 3; ++g) p.group_amax[g] = (groups > 1 && g < groups && amax_groups) ? amax_groups[g] : nullptr;
  rc = get_out_map(&tmD, d, (uint64_t)M, (uint64_t)(groups > 1 ? group_cols : N), (uint64_t)ldd);
  if (rc != LLNV_OK) return rc;
  gmaps.m[0] = tmD;
  gmaps.m[1] = tmD;
  for (int g = 1; g < groups; ++g) {
    rc = get_out_map(&gmaps.m[g - 1], d_groups[g], (uint64_t)M, (uint64_t)group_cols, (uint64_t)ldd_groups[g]);
    if (rc != LLNV_OK) return rc;
  }
  tmR = tmD;
  if (epi.residual) {
    LLNV_REQUIRE(((uintptr_t)epi.residual & 15) == 0 && epi.ldr % 8 == 0, "llnv_gemm_nvfp4: residual must be 16-byte aligned with ldr a multiple of 8");
    rc = get_out_map(&tmR, epi.residual, (uint64_t)M, (uint64_t)N, (uint64_t)epi.ldr);
    if (rc != LLNV_OK) return rc;
  }
  const int variant = (epi.bias ? kEpiBias : 0) | (epi.act == 1 ? kEpiGelu : 0) | (epi.residual ? kEpiRes : 0) | (requant ? kEpiQuant : 0);
  // CTA pairs pay off when the K loop dominates (measured: +13..17 % at K = 14336, no gain at K = 3072)
  const bool pair_ok = N % 256 == 0 && !requant;
  const bool pair_auto = tile == 0 && K >= 8192 && M >= 1024 && groups == 1;
  if (pair_ok && groups == 1 && (tile == 2 || pair_auto)) return gemm_nvfp4_pair(a_codes, a_sf, b_codes, b_sf, p, tmD, tmR, variant, stream);
#define LLNV_GEMM_CASE(V)                                                                   \
  case V:                                                                                   \
    return bn == 256   ? launch<256, V>(tmA, tmB, tmD, tmR, p, stream, gmaps)                     \
           : bn == 192 ? launch<192, V>(tmA, tmB, tmD, tmR, p, stream, gmaps)                     \
                       : launch<128, V>(tmA, tmB, tmD, tmR, p, stream, gmaps);
  switch (variant) {
    LLNV_GEMM_CASE(0)
    LLNV_GEMM_CASE(1)
    LLNV_GEMM_CASE(2)
    LLNV_GEMM_CASE(3)
    LLNV_GEMM_CASE(4)
    LLNV_GEMM_CASE(5)
    LLNV_GEMM_CASE(6)
    LLNV_GEMM_CASE(7)
    LLNV_GEMM_CASE(8)       // requantized output: plain, + bias, + GELU, + bias + GELU
    LLNV_GEMM_CASE(9)
    LLNV_GEMM_CASE(10)
    LLNV_GEMM_CASE(11)
  }
#undef LLNV_GEMM_CASE
  set_error("llnv_gemm_nvfp4: internal dispatch error");
  return LLNV_E_INVALID;
}

}  // namespace

extern "C" int llnv_gemm_nvfp4(const void* a_codes, const void* a_sf, const float* a_amax, int a_rule, const void* b_codes,
                               const void* b_sf, const float* b_amax, int b_rule, int64_t M, int64_t N, int64_t K,
                               const llnv_epilogue_t* epilogue, void* d, int64_t ldd, llnv_stream_t stream) {
  return gemm_run(a_codes, a_sf, a_amax, a_rule, b_codes, b_sf, b_amax, b_rule, M, N, K, epilogue, d, ldd, (cudaStream_t)stream, 1, nullptr,
                  nullptr, nullptr, LLNV_GEMM_TILE_AUTO);
}

extern "C" int llnv_gemm_nvfp4_ex(const void* a_codes, const void* a_sf, const float* a_amax, int a_rule, const void* b_codes,
                                  const void* b_sf, const float* b_amax, int b_rule, int64_t M, int64_t N, int64_t K,
                                  const llnv_epilogue_t* epilogue, void* d, int64_t ldd, int tile, llnv_stream_t stream) {
  return gemm_run(a_codes, a_sf, a_amax, a_rule, b_codes, b_sf, b_amax, b_rule, M, N, K, epilogue, d, ldd, (cudaStream_t)stream, 1, nullptr,
                  nullptr, nullptr, tile);
}

extern "C" int llnv_gemm_nvfp4_grouped(const void* a_codes, const void* a_sf, const float* a_amax, int a_rule, const void* b_codes,
                                       const void* b_sf, const float* b_amax, int b_rule, int64_t M, int64_t N_each, int64_t K, int groups,
                                       const llnv_epilogue_t* epilogue, void* const* d, const int64_t* ldd, float* const* out_amax,
                                       llnv_stream_t stream) {
  LLNV_REQUIRE(groups >= 2 && groups <= 3, "llnv_gemm_nvfp4_grouped: 2 or 3 weight groups (got %d)", groups);
  LLNV_REQUIRE(d && ldd && a_amax && b_amax, "llnv_gemm_nvfp4_grouped: null pointer");
  LLNV_REQUIRE(N_each > 0 && N_each % 128 == 0, "llnv_gemm_nvfp4_grouped: rows per weight matrix must be a multiple of 128");
  for (int g = 0; g < groups; ++g)
    LLNV_REQUIRE(d[g] != nullptr && ldd[g] >= N_each && ldd[g] % 8 == 0 && ((uintptr_t)d[g] & 15) == 0,
                 "llnv_gemm_nvfp4_grouped: output %d must be 16-byte aligned with a row stride >= N_each that is a multiple of 8", g);
  if (epilogue) LLNV_REQUIRE(!epilogue->residual && !epilogue->gate && !epilogue->alpha && !epilogue->out_amax,
                             "llnv_gemm_nvfp4_grouped: residual, gate, alpha and out_amax belong to the single-matrix call");
  if (out_amax) {
    for (int g = 0; g < groups; ++g)
      if (out_amax[g] && !amax_accumulate(2)) LLNV_CUDA(cudaMemsetAsync(out_amax[g], 0, sizeof(float), (cudaStream_t)stream));
  }
  return gemm_run(a_codes, a_sf, a_amax, a_rule, b_codes, b_sf, b_amax, b_rule, M, N_each * groups, K, epilogue, d[0], ldd[0],
                  (cudaStream_t)stream, groups, d, ldd, out_amax, LLNV_GEMM_TILE_AUTO);
}
