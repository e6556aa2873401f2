// Shared host/device helpers of the llnvfp4 library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/llnvfp4.h"

namespace llnv {

// ---- error reporting -------------------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define LLNV_REQUIRE(cond, ...)          \
  do {                                   \
    if (!(cond)) {                       \
      ::llnv::set_error(__VA_ARGS__);    \
      return LLNV_E_INVALID;             \
    }                                    \
  } while (0)

#define LLNV_CUDA(call)                                     \
  do {                                                      \
    cudaError_t e__ = (call);                               \
    if (e__ != cudaSuccess) return ::llnv::cuda_fail(e__, #call); \
  } while (0)

inline int launch_status(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, what);
  return LLNV_OK;
}

// Device status word written by kernels whose bounded waits give up.
unsigned int* device_status_word();   // lazily allocated per device (never freed)

// SM count of the current device (cached).
int sm_count();

// ---- programmatic dependent launch ---------------------------------------------------------
// Every kernel of the library is launched through launch_k and starts with pdl_wait().  When the
// "programmatic stream serialization" attribute is switched on (llnv_set_pdl(1) or LLNV_PDL=1) a
// grid may be scheduled while the preceding kernel of the stream is still draining; pdl_wait()
// then blocks until that grid has completed and its writes are visible, so the memory semantics
// are those of an ordinary in-stream launch.  No kernel triggers its dependents early: a dependent
// grid starts only when every CTA of its predecessor has exited, so a waiting grid never holds SM
// resources a running grid needs.  It is OFF by default: on a B200 the 30-layer chunk replayed as
// CUDA graphs measured 145.5 ms with it and 145.6 ms without -- kernel boundaries inside a graph
// are already back to back -- so the default stays the plain launch.  Without the attribute
// pdl_wait() returns at once.
bool pdl_enabled();                    // llnv_set_pdl / environment LLNV_PDL=0 turn the attribute off
void count_launch();                   // llnv_launch_count(): kernels launched by the library since it was loaded
bool amax_accumulate(int which);       // llnv_set_amax_accumulate: bit 1 attention + LN quantizers, bit 2 grouped GEMM + RoPE

template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  count_launch();
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- group maximum over NVLink peer memory, for kernels that consume a tensor amax --------------
// A sequence-parallel group that wants the single-GPU codes needs the MAX of every tensor amax over its ranks before the
// quantizer's first block.  Instead of a separate one-warp all-reduce kernel in front of it, the quantize kernel does the
// exchange itself (quantize.cu): its first CTA publishes this rank's value into every rank's slot array and raises this
// rank's flag there, one warp of every CTA waits (bounded; lane r on rank r's flag) until all ranks' flags show the current
// epoch, and takes the maximum of the slots.  Flags, slots and the epoch counter are those of llnv_peer_barrier / llnv_peer_allreduce_max
// (peer.cu), so the fused form counts as one barrier of the same sequence.  epoch[1] counts the CTAs that are done:
// the last one stores the group maximum back to the amax scalar, resets the counter and advances the epoch.
constexpr int kMaxPeers = 8;
struct PeerReduce {
  void* slots[kMaxPeers];
  void* signals[kMaxPeers];
  int rank, world;             // world <= 1: no exchange
  unsigned int* epoch;         // [2] device words of this rank: epoch, finished-CTA counter
  unsigned int max_polls;
  unsigned int* status;
};
unsigned int peer_poll_limit();        // llnv_set_peer_poll_limit

// LayerNorm-family transform fused into the quantizer (quantize.cu).  mode: 1 = adaLN modulation,
// 2 = affine LayerNorm.  row_stats is a scratch array of 2*M floats; nothing is allocated.
// row_offset shifts the frame lookup (token shards); phase 0 = statistics + amax + quantize,
// 1 = statistics + amax only, 2 = quantize only (amax and row_stats as left by phase 1).
// peer (phase 0 only): MAX-reduce the tensor amax over a sequence-parallel group inside the quantize kernel.
int ln_quantize_impl(int mode, const void* x, int64_t M, int64_t C, int64_t ldx, const void* p0, const void* p1,
                     int64_t mod_stride, int frame_rows, float eps, int add_one, int rule, void* codes, void* sf,
                     float* amax, void* y_out, int64_t ldy, float* row_stats, cudaStream_t stream, const char* who,
                     int64_t row_offset, int phase, const struct PeerReduce* peer = nullptr);

// ---- scale rule constants -----------------------------------------------------------------
__host__ __device__ inline float rule_e2m1_max(int rule) { return rule == LLNV_RULE_STATIC_4 ? 4.f : 6.f; }
__host__ __device__ inline float rule_e4m3_max(int rule) {
  return (rule == LLNV_RULE_STATIC_6 || rule == LLNV_RULE_STATIC_4) ? 448.f : 256.f;
}

// ---- device helpers -------------------------------------------------------------------------
#ifdef __CUDACC__

// First statement of every kernel: wait for the preceding grid of the stream (see launch_k).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// See PeerReduce.  Called by the 32 lanes of ONE warp per CTA (lane r talks to rank r, so that the waits on the `world`
// flags overlap instead of queueing behind one another); `publish` is true in exactly one CTA of the grid.  Every lane
// returns the group maximum; lane 0 also returns the epoch of the exchange through epoch_out.
__device__ inline float peer_group_max(const PeerReduce& pr, float local, bool publish, unsigned int* epoch_out) {
  const int r = (int)(threadIdx.x & 31u);
  const unsigned int e = *reinterpret_cast<volatile unsigned int*>(pr.epoch) + 1u;
  if (r == 0) *epoch_out = e;
  const int par = (int)(e & 1u);
  float m = local;
  if (r < pr.world) {
    if (publish) {
      float* theirs = reinterpret_cast<float*>(pr.slots[r]) + ((int64_t)par * kMaxPeers + pr.rank) * 32;
      asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(theirs), "f"(local) : "memory");
      unsigned int* flag = reinterpret_cast<unsigned int*>(pr.signals[r]) + pr.rank;
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(e) : "memory");
    }
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(pr.signals[pr.rank]) + r;
    bool ok = false;
    for (unsigned int i = 0; i < pr.max_polls; ++i) {
      unsigned int v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if ((int)(v - e) >= 0) {
        ok = true;
        break;
      }
      // another CTA (or an earlier kernel) has already recorded a failed wait: do not wait it out again
      if ((i & 1023u) == 1023u && pr.status && *reinterpret_cast<volatile unsigned int*>(pr.status) != 0u) break;
    }
    if (!ok && pr.status && atomicCAS(pr.status, 0u, 3u) == 0u) {
      pr.status[1] = 702u;
      pr.status[2] = (unsigned int)r;
      pr.status[3] = e;
    }
    // rank r's value in my slot area (its flag, acquired above, was raised after the value was stored)
    const float* slot = reinterpret_cast<const float*>(pr.slots[pr.rank]) + ((int64_t)par * kMaxPeers + r) * 32;
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(slot) : "memory");
    m = fmaxf(m, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
  return m;
}

// fp32 -> bf16 bits, round to nearest even (finite inputs).
__device__ __forceinline__ uint32_t f2bf(float f) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}
// two fp32 -> packed bf16x2 with ONE paired conversion (the scalar conversion issues on the slow
// special-function pipe; the paired form does not)
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&p);
}
// round two fp32 values to bf16 precision in place (kept in fp32)
__device__ __forceinline__ void round_bf16x2(float& a, float& b) {
  const uint32_t p = pack_bf16x2(a, b);
  a = __uint_as_float(p << 16);
  b = __uint_as_float(p & 0xFFFF0000u);
}
// round an fp32 value to bf16 precision, keep it in fp32
__device__ __forceinline__ float round_bf16(float f) { return __uint_as_float(f2bf(f) << 16); }

// Packed two-lane fp32 arithmetic (sm_100): each lane is the correctly rounded IEEE operation, so a
// packed instruction gives bit for bit what the two scalar ones give, at half the issue slots.
struct F2 {
  float x, y;
};
__device__ __forceinline__ F2 f2_fma(F2 a, F2 b, F2 c) {
  F2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ F2 f2_mul(F2 a, F2 b) {
  F2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ F2 f2_add(F2 a, F2 b) {
  F2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ F2 f2_sub(F2 a, F2 b) {
  F2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "sub.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ F2 f2_splat(float v) { return F2{v, v}; }

// e4m3 byte -> fp32 (exact)
__device__ __forceinline__ float e4m3_to_float(uint32_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)(b & 0xFF), __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
// fp32 -> e4m3 byte, round to nearest even (inputs here never exceed 448)
__device__ __forceinline__ uint32_t float_to_e4m3(float f) {
  return (uint32_t)__nv_cvt_float_to_fp8(f, __NV_SATFINITE, __NV_E4M3);
}

// Offset of scale (row r, scale column c) in the 128x4-swizzled layout; cols = scale columns per row.
__host__ __device__ __forceinline__ int64_t sf_offset(int64_t r, int64_t c, int64_t cols) {
  int64_t tile = (r >> 7) * (cols >> 2) + (c >> 2);
  return tile * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (c & 3);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}

// atomic max for non-negative floats (bit pattern order == value order)
__device__ __forceinline__ void atomic_max_nonneg(float* addr, float v) {
  atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
}

#endif  // __CUDACC__

}  // namespace llnv
