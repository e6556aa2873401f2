// Host-side construction of TMA tensor maps.  cuTensorMapEncodeTiled is resolved through the
// runtime's driver entry point query so the library links against cudart only.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "sm100.cuh"

namespace llnv {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

static int encode(CUtensorMap* out, CUtensorMapDataType dt, size_t esize, const void* base, uint64_t rows, uint64_t cols,
                  uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols, int swizzle) {
  EncodeTiledFn fn = get_encode();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return LLNV_E_CUDA;
  }
  if (((uintptr_t)base & 15) != 0 || (pitch_bytes & 15) != 0) {
    set_error("tensor map: base address and row pitch must be multiples of 16 bytes");
    return LLNV_E_INVALID;
  }
  if (box_rows == 0 || box_rows > 256 || box_cols == 0 || box_cols * esize > 256 * esize || (box_cols * esize) % 16 != 0) {
    set_error("tensor map: unsupported box %u x %u", box_rows, box_cols);
    return LLNV_E_INVALID;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapSwizzle sw = swizzle == 3 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                          : swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_32B
                                         : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (rows=%llu cols=%llu pitch=%llu box=%ux%u)", (int)r,
              (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)pitch_bytes, box_rows, box_cols);
    return LLNV_E_CUDA;
  }
  return LLNV_OK;
}

int make_tensor_map_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes, uint64_t pitch_bytes,
                       uint32_t box_rows, uint32_t box_bytes, int swizzle) {
  return encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, base, rows, row_bytes, pitch_bytes, box_rows, box_bytes, swizzle);
}

int make_tensor_map_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_elems,
                            uint32_t box_rows, uint32_t box_cols, int swizzle) {
  return encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, rows, cols, pitch_elems * 2, box_rows, box_cols, swizzle);
}

// ---- small cache: encoding a tensor map costs a few microseconds of host time ----------------
namespace {
struct MapKey {
  const void* ptr;
  uint64_t rows, cols, pitch;
  uint32_t box_rows, box_cols;
  int kind, swizzle;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && pitch == o.pitch && box_rows == o.box_rows &&
           box_cols == o.box_cols && kind == o.kind && swizzle == o.swizzle;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = (uint64_t)(uintptr_t)k.ptr * 0x9e3779b97f4a7c15ull;
    h ^= k.rows * 1315423911ull + k.cols * 2654435761ull + k.pitch * 40503ull + k.box_rows * 97ull + k.box_cols * 13ull +
         (uint64_t)k.kind * 7ull + (uint64_t)k.swizzle;
    return (size_t)(h ^ (h >> 29));
  }
};
std::mutex g_map_mu;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
}  // namespace

int cached_tensor_map(CUtensorMap* out, int kind, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch,
                      uint32_t box_rows, uint32_t box_cols, int swizzle) {
  MapKey key{base, rows, cols, pitch, box_rows, box_cols, kind, swizzle};
  std::lock_guard<std::mutex> lock(g_map_mu);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return LLNV_OK;
  }
  CUtensorMap m;
  int rc = kind == 0 ? make_tensor_map_2d(&m, base, rows, cols, pitch, box_rows, box_cols, swizzle)
                     : make_tensor_map_2d_bf16(&m, base, rows, cols, pitch, box_rows, box_cols, swizzle);
  if (rc != LLNV_OK) return rc;
  if (g_maps.size() > 8192) g_maps.clear();
  g_maps.emplace(key, m);
  *out = m;
  return LLNV_OK;
}

}  // namespace llnv
