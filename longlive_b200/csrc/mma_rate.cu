// Tensor-core issue rate of the block-scaled FP4 MMA with nothing else in the way: the denominator
// the W4A4 GEMM's tensor roofline is quoted against.
//
// One CTA per SM.  The CTA fills one A tile (128 rows x 256 E2M1) and one B tile (256 rows x 256
// E2M1) in shared memory with pseudo-random codes in the canonical 128-byte-swizzled K-major layout,
// puts unit scales (UE4M3 1.0) into tensor memory, and then a single thread issues `k_blocks` x 4
// tcgen05.mma (128 x 256 x 64 each, kind::mxf4nvf4) into one accumulator.  No operand is refilled, no
// accumulator is read back: the launch time is the MMA pipe's time for 2 * 128 * 256 * 256 * k_blocks
// flop per SM, i.e. what a GEMM main loop could reach if loads, scale copies and the epilogue were free.
// The wait for the last commit is bounded like every other wait of the library.
#include "common.cuh"
#include "sm100.cuh"

namespace llnv {
namespace {

using namespace sm100;

constexpr uint32_t kABytes = 128 * 128, kBBytes = 256 * 128, kSfBytes = 2048;
constexpr uint32_t kSmem = kABytes + kBBytes + kSfBytes + 1024 + 64;

__global__ void __launch_bounds__(128, 1) mma_rate_kernel(int k_blocks, unsigned int* status) {
  pdl_wait();
  extern __shared__ __align__(1024) uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* done_bar = reinterpret_cast<uint64_t*>(smem + kABytes + kBBytes + kSfBytes);
  uint64_t* step_bar = done_bar + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  const int warp = threadIdx.x >> 5;

  uint32_t h = 0x9E3779B9u * (blockIdx.x * 128 + threadIdx.x + 1);
  for (uint32_t i = threadIdx.x; i < (kABytes + kBBytes) / 4; i += 128) {
    h = h * 1664525u + 1013904223u;
    reinterpret_cast<uint32_t*>(smem)[i] = h ^ (h >> 13);
  }
  for (uint32_t i = threadIdx.x; i < kSfBytes / 4; i += 128)
    reinterpret_cast<uint32_t*>(smem + kABytes + kBBytes)[i] = 0x38383838u;        // UE4M3 1.0
  if (threadIdx.x == 0) {
    mbar_init(done_bar, 1);
    mbar_init(step_bar, 1);
    *abort_flag = 0u;
    fence_barrier_init();
  }
  fence_proxy_async();
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 1 && elect_one()) {
    constexpr uint32_t idesc = make_idesc_nvf4(128, 256);
    constexpr uint32_t kOpHi = (uint32_t)(make_smem_desc(0, 16, 1024, 2) >> 32);
    constexpr uint32_t kSfHi = (uint32_t)(make_smem_desc(0, 0, 128, 0) >> 32);
    const uint32_t a_lo = (smem_u32(smem) >> 4) | (1u << 16);
    const uint32_t b_lo = a_lo + (kABytes >> 4);
    const uint32_t sf_lo = (smem_u32(smem) + kABytes + kBBytes) >> 4;
    // scale columns: A scales at 256..271 (4 per K=64 step), B scales at 272..303 (8 per step)
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      tmem_cp_sf(tmem_base + 256 + 4 * g, ((uint64_t)kSfHi << 32) | (sf_lo + 32 * g));
      tmem_cp_sf(tmem_base + 272 + 8 * g, ((uint64_t)kSfHi << 32) | (sf_lo + 32 * g));
      tmem_cp_sf(tmem_base + 272 + 8 * g + 4, ((uint64_t)kSfHi << 32) | (sf_lo + 32 * g));
    }
    for (int kb = 0; kb < k_blocks; ++kb) {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        mma_nvf4(tmem_base, ((uint64_t)kOpHi << 32) | (a_lo + 2 * k), ((uint64_t)kOpHi << 32) | (b_lo + 2 * k), idesc,
                 tmem_base + 256 + 4 * k, tmem_base + 272 + 8 * k, (kb | k) != 0 ? 1u : 0u);
      tc_commit(step_bar);            // what a GEMM does per K block to release the stage; nobody waits on it here
    }
    tc_commit(done_bar);
    mbar_wait(done_bar, 0u, abort_flag, status, 950u);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

}  // namespace
}  // namespace llnv

extern "C" int llnv_fp4_mma_rate(int k_blocks, double* flop_out, void* stream) {
  using namespace llnv;
  LLNV_REQUIRE(k_blocks > 0 && k_blocks <= (1 << 22), "llnv_fp4_mma_rate: k_blocks must be in 1..4194304 (got %d)", k_blocks);
  LLNV_CUDA(cudaFuncSetAttribute(mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem));
  const int ctas = sm_count();
  if (flop_out) *flop_out = 2.0 * 128 * 256 * 256 * (double)k_blocks * ctas;
  LLNV_CUDA(launch_k(mma_rate_kernel, dim3(ctas), dim3(128), kSmem, (cudaStream_t)stream, k_blocks, device_status_word()));
  return LLNV_OK;
}
