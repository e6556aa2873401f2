// Allocation-free variant of the adaLN + quantize entry point.
//
// llnv_adaln_quantize_nvfp4 needs a scratch array (mean and 1/std of every row, written by its
// first kernel and read by its second) that the caller normally allocates.  Some hosts of this
// library cannot do that at the point of the call: a serving process that has handed all device
// memory to its own arena and forbids further allocations, or a latency-critical loop in which
// the device-wide synchronisation a cudaMalloc implies would stall every other stream.  For those
// callers the scratch lives in a fixed array that is part of the library image, so the entry
// point below performs no cudaMalloc / cudaFree and calls no allocating library routine.
//
// Consequences of the fixed array, all part of the contract:
//   * capacity: at most LLNV_STATIC_MAX_ROWS rows per call (128 KiB of device memory that every
//     GPU which loads the library holds until the process exits); larger M is rejected;
//   * every call on a device shares the one array.  Its contents are whatever the previous call
//     left there; this entry point needs no zero-initialised state (each call overwrites the
//     statistics of rows 0..M-1 before reading them).  Two calls that may run concurrently on the
//     same GPU (different streams) race on the array and must not be issued;
//   * the device address of the array is looked up with cudaGetSymbolAddress on every call (a host-side table
//     lookup once the library's device code is loaded, no stream operation) and never cached: a cached address
//     would dangle after cudaDeviceReset() or any other teardown of the primary context, whereas the lookup
//     follows the context that is current.  The array's contents do not survive such a teardown and need not.
//     The first call on each device may load the device code; make it during start-up, before any stream
//     capture begins.
#include "common.cuh"

namespace llnv {
namespace {

constexpr int64_t kStaticMaxRows = 16384;

// Device-side storage.  In host code this name is only a handle for the symbol, never a device
// address: the address kernels receive comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_static_row_stats[2 * kStaticMaxRows];

// Device address of the scratch array in the current context.
int static_row_stats(float** out) {
  float* p = nullptr;
  cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_row_stats);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_static_row_stats)");
  LLNV_REQUIRE(p != nullptr, "static scratch: cudaGetSymbolAddress returned a null address");
  *out = p;
  return LLNV_OK;
}

}  // namespace
}  // namespace llnv

using namespace llnv;

extern "C" int64_t llnv_static_max_rows(void) { return kStaticMaxRows; }

extern "C" int llnv_adaln_quantize_nvfp4_static(const void* x, int64_t M, int64_t C, int64_t ldx, const void* scale,
                                                const void* shift, int64_t mod_stride, int frame_rows, float eps,
                                                int add_one, int rule, void* codes, void* sf, float* amax, void* y_out,
                                                int64_t ldy, llnv_stream_t stream) {
  LLNV_REQUIRE(M <= kStaticMaxRows,
               "llnv_adaln_quantize_nvfp4_static: M = %lld exceeds the built-in scratch capacity of %lld rows; "
               "use llnv_adaln_quantize_nvfp4 with a caller-provided row_stats array",
               (long long)M, (long long)kStaticMaxRows);
  float* row_stats = nullptr;
  const int rc = static_row_stats(&row_stats);
  if (rc != LLNV_OK) return rc;
  return ln_quantize_impl(1, x, M, C, ldx, scale, shift, mod_stride, frame_rows, eps, add_one, rule, codes, sf, amax, y_out,
                          ldy, row_stats, (cudaStream_t)stream, "llnv_adaln_quantize_nvfp4_static", 0, 0);
}
