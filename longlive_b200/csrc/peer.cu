// Sequence-parallel exchange over NVLink peer memory: kernels that write their results straight
// into the other ranks' buffers, and the barrier that orders them.
//
// The two all-to-alls of Ulysses sequence parallelism (tokens -> heads before attention, heads ->
// tokens after it; wan_5b/distributed/sp_ulysses_inference.py:122-154) move every value exactly
// once, from the kernel that produces it to the kernel that consumes it on another GPU.  With all
// exchange buffers in symmetric memory (the same allocation mapped on every rank of the node) a
// producer can store each shard directly at its final address on the destination GPU with plain
// st.global over NVLink, instead of writing a send buffer that a communication kernel copies again:
//   * llnv_rmsnorm_rope_scatter (rope_norm.cu) writes q / rotated k / smoothed k per head shard,
//   * llnv_scatter_2d (here) pushes a [rows, cols] matrix as P row blocks or P column blocks,
//   * llnv_peer_barrier (here) makes every rank's pushes visible to the others before the consumers
//     start, and keeps a rank from overwriting a buffer another rank is still reading.
// Only plain loads and stores touch peer memory: no TMA multicast, no library kernel gets a peer
// pointer.
//
// Barrier protocol.  Each rank owns `world` 32-bit flags in its symmetric signal area, flag s
// written only by rank s.  Barrier number e (counted per rank in device memory, so a captured graph
// replays correctly): thread r of the single CTA stores e into flag[my_rank] of rank r
// (st.release.sys), then polls its own flag[r] until it is >= e (ld.acquire.sys).  Epochs only
// grow, so a rank that is already one barrier ahead cannot be missed.  The poll is bounded: after
// max_polls polls (a launch parameter; llnv_set_peer_poll_limit, default a few seconds) the kernel
// records a timeout in the status word (read by llnv_check_status) and returns; it never traps and
// never spins forever.  What a consumer reads after a timed-out barrier is undefined, so callers
// check the status before they use a step's results (CausalDiT.run_chunk does, once per chunk).
#include "common.cuh"

namespace llnv {
namespace {

constexpr uint32_t kDefaultPeerPolls = 1u << 22;     // a few seconds of polling before giving up
uint32_t g_peer_polls = kDefaultPeerPolls;

struct PeerPtrs {
  void* p[kMaxPeers];
};

__global__ void __launch_bounds__(32) peer_barrier_kernel(PeerPtrs signals, int rank, int world, unsigned int* epoch,
                                                          unsigned int* status, uint32_t max_polls) {
  pdl_wait();
  __shared__ unsigned int e_sh;
  if (threadIdx.x == 0) e_sh = *epoch + 1u;
  __syncwarp();
  const unsigned int e = e_sh;
  const int r = threadIdx.x;
  bool ok = true;
  if (r < world) {
    unsigned int* theirs = reinterpret_cast<unsigned int*>(signals.p[r]) + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(e) : "memory");
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(signals.p[rank]) + r;
    ok = false;
    for (uint32_t i = 0; i < max_polls; ++i) {
      unsigned int v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if ((int)(v - e) >= 0) {
        ok = true;
        break;
      }
    }
  }
  if (!ok && status && atomicCAS(status, 0u, 3u) == 0u) {
    status[1] = 700u;
    status[2] = (unsigned int)r;
    status[3] = e;
  }
  __syncwarp();
  if (threadIdx.x == 0) *epoch = e;
}

// MAX all-reduce of up to 32 floats over the group, fused with the barrier: thread r stores this
// rank's values into rank r's slot array (slots[epoch parity][my rank][i]), signals and waits as
// peer_barrier_kernel does, then thread i takes the maximum of slot i over all ranks.  Two slot
// arrays alternate with the epoch, so a rank that is already in the next reduction cannot overwrite
// values a slower rank has not read yet (it cannot be two reductions ahead: each one is a barrier).
__global__ void __launch_bounds__(32) peer_allreduce_max_kernel(float* __restrict__ vals, int n, PeerPtrs slots, PeerPtrs signals,
                                                                int rank, int world, unsigned int* epoch, unsigned int* status,
                                                                uint32_t max_polls) {
  pdl_wait();
  __shared__ unsigned int e_sh;
  if (threadIdx.x == 0) e_sh = *epoch + 1u;
  __syncwarp();
  const unsigned int e = e_sh;
  const int r = threadIdx.x;
  const int par = (int)(e & 1u);
  bool ok = true;
  if (r < world) {
    float* theirs = reinterpret_cast<float*>(slots.p[r]) + ((int64_t)par * kMaxPeers + rank) * 32;
    for (int i = 0; i < n; ++i) theirs[i] = vals[i];
    unsigned int* flag = reinterpret_cast<unsigned int*>(signals.p[r]) + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(e) : "memory");
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(signals.p[rank]) + r;
    ok = false;
    for (uint32_t i = 0; i < max_polls; ++i) {
      unsigned int v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if ((int)(v - e) >= 0) {
        ok = true;
        break;
      }
    }
  }
  if (!ok && status && atomicCAS(status, 0u, 3u) == 0u) {
    status[1] = 701u;
    status[2] = (unsigned int)r;
    status[3] = e;
  }
  __syncwarp();
  if (threadIdx.x < n) {
    const float* mine = reinterpret_cast<const float*>(slots.p[rank]) + (int64_t)par * kMaxPeers * 32 + threadIdx.x;
    float m = -INFINITY;
    for (int q = 0; q < world; ++q) {
      float v;
      asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(mine + q * 32) : "memory");
      m = fmaxf(m, v);
    }
    vals[threadIdx.x] = m;
  }
  __syncwarp();
  if (threadIdx.x == 0) *epoch = e;
}

// dst[r][i][0:row_bytes] = src[r * src_shard_bytes + i * src_pitch : ... + row_bytes], 16-byte vectors.
__global__ void __launch_bounds__(256) scatter_2d_kernel(const uint8_t* __restrict__ src, int64_t src_shard_bytes, int64_t src_pitch,
                                                         PeerPtrs dst, int64_t dst_pitch, int64_t rows, int vec_per_row) {
  pdl_wait();
  const int r = blockIdx.y;
  const uint8_t* s = src + (int64_t)r * src_shard_bytes;
  uint8_t* d = reinterpret_cast<uint8_t*>(dst.p[r]);
  const int64_t total = rows * vec_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / vec_per_row;
    const int v = (int)(i - row * vec_per_row);
    const uint4 val = __ldg(reinterpret_cast<const uint4*>(s + row * src_pitch) + v);
    reinterpret_cast<uint4*>(d + row * dst_pitch)[v] = val;
  }
}

}  // namespace

unsigned int peer_poll_limit() { return g_peer_polls; }
}  // namespace llnv

using namespace llnv;

extern "C" int llnv_set_peer_poll_limit(unsigned int max_polls) {
  const unsigned int before = g_peer_polls;
  g_peer_polls = max_polls ? max_polls : kDefaultPeerPolls;
  return (int)(before > 0x7FFFFFFFu ? 0x7FFFFFFFu : before);
}

extern "C" int llnv_peer_barrier(void* const* signal_ptrs, int rank, int world, void* epoch, llnv_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  LLNV_REQUIRE(signal_ptrs && epoch, "llnv_peer_barrier: null pointer");
  LLNV_REQUIRE(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, "llnv_peer_barrier: need 1 <= world <= 8 and 0 <= rank < world");
  PeerPtrs sp = {};
  for (int r = 0; r < world; ++r) {
    LLNV_REQUIRE(signal_ptrs[r] != nullptr && ((uintptr_t)signal_ptrs[r] & 3) == 0, "llnv_peer_barrier: bad signal pointer of rank %d", r);
    sp.p[r] = signal_ptrs[r];
  }
  launch_k(peer_barrier_kernel, 1, 32, 0, stream, sp, rank, world, (unsigned int*)epoch, device_status_word(), g_peer_polls);
  return launch_status("peer_barrier_kernel");
}

extern "C" int llnv_peer_allreduce_max(float* vals, int n, void* const* slot_ptrs, void* const* signal_ptrs, int rank, int world,
                                       void* epoch, llnv_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  LLNV_REQUIRE(vals && slot_ptrs && signal_ptrs && epoch, "llnv_peer_allreduce_max: null pointer");
  LLNV_REQUIRE(n >= 1 && n <= 32, "llnv_peer_allreduce_max: 1 to 32 values (got %d)", n);
  LLNV_REQUIRE(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, "llnv_peer_allreduce_max: need 1 <= world <= 8 and 0 <= rank < world");
  PeerPtrs sl = {}, sg = {};
  for (int r = 0; r < world; ++r) {
    LLNV_REQUIRE(slot_ptrs[r] != nullptr && signal_ptrs[r] != nullptr && ((uintptr_t)slot_ptrs[r] & 3) == 0 && ((uintptr_t)signal_ptrs[r] & 3) == 0,
                 "llnv_peer_allreduce_max: bad pointer of rank %d", r);
    sl.p[r] = slot_ptrs[r];
    sg.p[r] = signal_ptrs[r];
  }
  launch_k(peer_allreduce_max_kernel, 1, 32, 0, stream, vals, n, sl, sg, rank, world, (unsigned int*)epoch, device_status_word(), g_peer_polls);
  return launch_status("peer_allreduce_max_kernel");
}

extern "C" int llnv_scatter_2d(const void* src, int64_t src_shard_bytes, int64_t src_pitch, void* const* dst_ptrs, int64_t dst_pitch,
                               int64_t rows, int64_t row_bytes, int shards, llnv_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  LLNV_REQUIRE(src && dst_ptrs, "llnv_scatter_2d: null pointer");
  LLNV_REQUIRE(shards >= 1 && shards <= kMaxPeers, "llnv_scatter_2d: need 1 <= shards <= 8");
  LLNV_REQUIRE(rows >= 0 && row_bytes > 0 && row_bytes % 16 == 0 && src_pitch % 16 == 0 && dst_pitch % 16 == 0 && src_shard_bytes % 16 == 0 &&
                   src_pitch >= row_bytes && dst_pitch >= row_bytes && ((uintptr_t)src & 15) == 0,
               "llnv_scatter_2d: sizes, pitches and pointers must be multiples of 16 bytes");
  PeerPtrs dp = {};
  for (int r = 0; r < shards; ++r) {
    LLNV_REQUIRE(dst_ptrs[r] != nullptr && ((uintptr_t)dst_ptrs[r] & 15) == 0, "llnv_scatter_2d: bad destination pointer %d", r);
    dp.p[r] = dst_ptrs[r];
  }
  if (rows == 0) return LLNV_OK;
  const int vec = (int)(row_bytes / 16);
  const int64_t total = rows * vec;
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 8 / shards + 1;
  if (blocks > cap) blocks = cap;
  launch_k(scatter_2d_kernel, dim3((unsigned)blocks, (unsigned)shards), 256, 0, stream, (const uint8_t*)src, src_shard_bytes, src_pitch, dp,
                                                                                 dst_pitch, rows, vec);
  return launch_status("scatter_2d_kernel");
}
