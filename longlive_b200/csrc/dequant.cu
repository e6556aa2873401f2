// NVFP4 -> bf16/fp16/fp32 dequantize: a general matrix form and the multi-block KV-cache form
// (one launch for all cache blocks of a layer, pointer table passed as launch parameters).
// Each thread decodes one 16-element block: one 8-byte code load, one scale byte, 32 bytes out.
#include <cuda_fp4.h>

#include "common.cuh"

namespace llnv {
namespace {

constexpr int kMaxBlocks = 32;

struct BlockTable {
  const uint8_t* codes[kMaxBlocks];
  const uint8_t* sf[kMaxBlocks];
  const float* amax[kMaxBlocks];
};

template <int ROUNDING>
__device__ __forceinline__ float deq_scale(float vs, float amax, float g, float denom) {
  if (ROUNDING == LLNV_DEQ_PYTORCH) return __fdiv_rn(__fmul_rn(vs, amax), denom);
  return __fmul_rn(vs, g);   // FUSED: g = amax * fp32(1/denom);  TRITON: g = amax / denom
}

template <typename T>
__device__ __forceinline__ void store16(T* out, const float (&v)[16]);

template <>
__device__ __forceinline__ void store16<__nv_bfloat16>(__nv_bfloat16* out, const float (&v)[16]) {
  uint4 a, b;
  a.x = pack_bf16x2(v[0], v[1]);   a.y = pack_bf16x2(v[2], v[3]);
  a.z = pack_bf16x2(v[4], v[5]);   a.w = pack_bf16x2(v[6], v[7]);
  b.x = pack_bf16x2(v[8], v[9]);   b.y = pack_bf16x2(v[10], v[11]);
  b.z = pack_bf16x2(v[12], v[13]); b.w = pack_bf16x2(v[14], v[15]);
  reinterpret_cast<uint4*>(out)[0] = a;
  reinterpret_cast<uint4*>(out)[1] = b;
}
template <>
__device__ __forceinline__ void store16<__half>(__half* out, const float (&v)[16]) {
  __half2 h[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
  reinterpret_cast<uint4*>(out)[0] = *reinterpret_cast<uint4*>(&h[0]);
  reinterpret_cast<uint4*>(out)[1] = *reinterpret_cast<uint4*>(&h[4]);
}
template <>
__device__ __forceinline__ void store16<float>(float* out, const float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
    reinterpret_cast<float4*>(out)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
}

// decode 8 packed bytes (16 codes) and scale them
template <int ROUNDING>
__device__ __forceinline__ void decode16(uint2 packed, float s, float amax, float g, float denom, float (&v)[16]) {
  const uint32_t words[2] = {packed.x, packed.y};
#pragma unroll
  for (int wi = 0; wi < 2; ++wi) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const uint8_t byte = (uint8_t)(words[wi] >> (8 * b));
      const __half2_raw h2 = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)byte, __NV_E2M1);
      const float lo = __half2float(__ushort_as_half(h2.x));
      const float hi = __half2float(__ushort_as_half(h2.y));
      v[wi * 8 + b * 2] = deq_scale<ROUNDING>(__fmul_rn(lo, s), amax, g, denom);
      v[wi * 8 + b * 2 + 1] = deq_scale<ROUNDING>(__fmul_rn(hi, s), amax, g, denom);
    }
  }
}

__device__ __forceinline__ float global_scale(int rounding, float amax, float denom) {
  if (rounding == LLNV_DEQ_FUSED) return __fmul_rn(amax, (float)(1.0 / (double)denom));
  return __fdiv_rn(amax, denom);
}

// rows x cols logical matrix; codes row stride = cols_padded/2 bytes; scales swizzled with
// cols_padded/16 scale columns.
template <typename T, int ROUNDING>
__global__ void __launch_bounds__(256) dequant_matrix_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ sf,
                                                             const float* __restrict__ amax_ptr, int64_t rows, int64_t cols,
                                                             int64_t cols_padded, float denom, T* __restrict__ out, int64_t ldo) {
  pdl_wait();
  const int64_t groups_per_row = cols >> 4;
  const int64_t total = rows * groups_per_row;
  const float amax = *amax_ptr;
  const float g = global_scale(ROUNDING, amax, denom);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / groups_per_row, c = i - r * groups_per_row;
    const uint2 p = __ldg(reinterpret_cast<const uint2*>(codes + r * (cols_padded >> 1) + c * 8));
    const float s = e4m3_to_float(__ldg(sf + sf_offset(r, c, cols_padded >> 4)));
    float v[16];
    decode16<ROUNDING>(p, s, amax, g, denom, v);
    store16<T>(out + r * ldo + c * 16, v);
  }
}

// KV cache: block b holds `rows` logical rows of 128 columns; out row = b*rows + r.
template <typename T, int ROUNDING>
__global__ void __launch_bounds__(256) dequant_kv_kernel(BlockTable tab, int num_blocks, int64_t rows, float denom,
                                                         T* __restrict__ out) {
  pdl_wait();
  const int64_t per_block = rows * 8;
  const int64_t total = per_block * num_blocks;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int b = (int)(i / per_block);
    const int64_t j = i - (int64_t)b * per_block;
    const int64_t r = j >> 3, c = j & 7;
    const float amax = __ldg(tab.amax[b]);
    const float g = global_scale(ROUNDING, amax, denom);
    const uint2 p = __ldg(reinterpret_cast<const uint2*>(tab.codes[b] + r * 64 + c * 8));
    const float s = e4m3_to_float(__ldg(tab.sf[b] + sf_offset(r, c, 8)));
    float v[16];
    decode16<ROUNDING>(p, s, amax, g, denom, v);
    store16<T>(out + ((int64_t)b * rows + r) * 128 + c * 16, v);
  }
}

template <typename T>
int launch_matrix(const uint8_t* codes, const uint8_t* sf, const float* amax, int64_t rows, int64_t cols, int64_t cols_padded,
                  float denom, int rounding, void* out, int64_t ldo, cudaStream_t stream) {
  const int64_t total = rows * (cols / 16);
  if (total == 0) return LLNV_OK;
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  T* o = (T*)out;
  switch (rounding) {
    case LLNV_DEQ_FUSED: launch_k(dequant_matrix_kernel<T, LLNV_DEQ_FUSED>, (unsigned)blocks, 256, 0, stream, codes, sf, amax, rows, cols, cols_padded, denom, o, ldo); break;
    case LLNV_DEQ_PYTORCH: launch_k(dequant_matrix_kernel<T, LLNV_DEQ_PYTORCH>, (unsigned)blocks, 256, 0, stream, codes, sf, amax, rows, cols, cols_padded, denom, o, ldo); break;
    default: launch_k(dequant_matrix_kernel<T, LLNV_DEQ_TRITON>, (unsigned)blocks, 256, 0, stream, codes, sf, amax, rows, cols, cols_padded, denom, o, ldo); break;
  }
  return launch_status("dequant_matrix_kernel");
}

template <typename T>
int launch_kv(const BlockTable& tab, int n, int64_t rows, float denom, int rounding, T* out, cudaStream_t stream) {
  const int64_t total = rows * 8 * n;
  if (total == 0) return LLNV_OK;
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  switch (rounding) {
    case LLNV_DEQ_FUSED: launch_k(dequant_kv_kernel<T, LLNV_DEQ_FUSED>, (unsigned)blocks, 256, 0, stream, tab, n, rows, denom, out); break;
    case LLNV_DEQ_PYTORCH: launch_k(dequant_kv_kernel<T, LLNV_DEQ_PYTORCH>, (unsigned)blocks, 256, 0, stream, tab, n, rows, denom, out); break;
    default: launch_k(dequant_kv_kernel<T, LLNV_DEQ_TRITON>, (unsigned)blocks, 256, 0, stream, tab, n, rows, denom, out); break;
  }
  return launch_status("dequant_kv_kernel");
}

}  // namespace
}  // namespace llnv

using namespace llnv;

extern "C" int llnv_dequantize_nvfp4(const void* codes, const void* sf, const float* amax, int64_t rows, int64_t cols,
                                     int64_t cols_padded, int dtype_code, float e2m1_max, float e4m3_max, int rounding,
                                     void* out, int64_t ldo, llnv_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  LLNV_REQUIRE(codes && sf && amax && out, "llnv_dequantize_nvfp4: null pointer");
  LLNV_REQUIRE(rows >= 0 && cols >= 0 && cols % 16 == 0 && cols_padded % 64 == 0 && cols_padded >= cols,
               "llnv_dequantize_nvfp4: cols must be a multiple of 16 and cols_padded a multiple of 64 (cols=%lld padded=%lld)",
               (long long)cols, (long long)cols_padded);
  LLNV_REQUIRE(rounding >= 0 && rounding <= 2, "llnv_dequantize_nvfp4: unknown rounding %d", rounding);
  LLNV_REQUIRE(e2m1_max > 0 && e4m3_max > 0, "llnv_dequantize_nvfp4: e2m1_max and e4m3_max must be positive");
  LLNV_REQUIRE(ldo >= cols && ldo % 8 == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)codes & 7) == 0,
               "llnv_dequantize_nvfp4: out must be 16-byte aligned with ldo a multiple of 8, codes 8-byte aligned");
  const float denom = e2m1_max * e4m3_max;
  const uint8_t* c = (const uint8_t*)codes;
  const uint8_t* s = (const uint8_t*)sf;
  switch (dtype_code) {
    case LLNV_DTYPE_BF16: return launch_matrix<__nv_bfloat16>(c, s, amax, rows, cols, cols_padded, denom, rounding, out, ldo, stream);
    case LLNV_DTYPE_FP16: return launch_matrix<__half>(c, s, amax, rows, cols, cols_padded, denom, rounding, out, ldo, stream);
    case LLNV_DTYPE_FP32: return launch_matrix<float>(c, s, amax, rows, cols, cols_padded, denom, rounding, out, ldo, stream);
    default: set_error("llnv_dequantize_nvfp4: unsupported dtype code %d", dtype_code); return LLNV_E_INVALID;
  }
}

extern "C" int llnv_kv_dequant(const void* const* codes, const void* const* sf, const float* const* amax, int num_blocks,
                               int num_heads, int block_token_size, int dtype_code, float e2m1_max, float e4m3_max,
                               int rounding, void* out, llnv_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  LLNV_REQUIRE(codes && sf && amax && out, "llnv_kv_dequant: null pointer");
  LLNV_REQUIRE(num_blocks > 0, "llnv_kv_dequant: values must contain at least one cache block");
  LLNV_REQUIRE(num_heads > 0, "llnv_kv_dequant: num_heads must be positive");
  LLNV_REQUIRE(block_token_size > 0, "llnv_kv_dequant: block_token_size must be positive");
  LLNV_REQUIRE(e2m1_max > 0 && e4m3_max > 0, "llnv_kv_dequant: e2m1_max and e4m3_max must be positive");
  LLNV_REQUIRE(rounding >= 0 && rounding <= 2, "llnv_kv_dequant: unknown rounding %d", rounding);
  LLNV_REQUIRE(((uintptr_t)out & 15) == 0, "llnv_kv_dequant: out must be 16-byte aligned");
  const int64_t rows = (int64_t)num_heads * block_token_size;
  const float denom = e2m1_max * e4m3_max;
  const size_t esize = dtype_code == LLNV_DTYPE_FP32 ? 4 : 2;
  LLNV_REQUIRE(dtype_code >= 0 && dtype_code <= 2, "llnv_kv_dequant: unsupported dtype code %d", dtype_code);
  for (int base = 0; base < num_blocks; base += kMaxBlocks) {
    const int n = num_blocks - base < kMaxBlocks ? num_blocks - base : kMaxBlocks;
    BlockTable tab;
    for (int i = 0; i < n; ++i) {
      LLNV_REQUIRE(codes[base + i] && sf[base + i] && amax[base + i], "llnv_kv_dequant: null pointer in block %d", base + i);
      LLNV_REQUIRE(((uintptr_t)codes[base + i] & 7) == 0, "llnv_kv_dequant: codes of block %d must be 8-byte aligned", base + i);
      tab.codes[i] = (const uint8_t*)codes[base + i];
      tab.sf[i] = (const uint8_t*)sf[base + i];
      tab.amax[i] = amax[base + i];
    }
    char* o = (char*)out + (size_t)base * rows * 128 * esize;
    int rc;
    if (dtype_code == LLNV_DTYPE_BF16) rc = launch_kv<__nv_bfloat16>(tab, n, rows, denom, rounding, (__nv_bfloat16*)o, stream);
    else if (dtype_code == LLNV_DTYPE_FP16) rc = launch_kv<__half>(tab, n, rows, denom, rounding, (__half*)o, stream);
    else rc = launch_kv<float>(tab, n, rows, denom, rounding, (float*)o, stream);
    if (rc != LLNV_OK) return rc;
  }
  return LLNV_OK;
}
