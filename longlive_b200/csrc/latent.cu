// Latent <-> token layout of a chunk: patchify (what the patch-embedding Conv3d with kernel and
// stride (1, 2, 2) sees) and unpatchify (wan_5b/modules/causal_model.py:1835-1858) as one pass.
//
//   latent [C, F, 2h, 2w] (strides for C and F free, the two image axes contiguous)
//   tokens [F * h * w, 4 * C]: token (f, hh, ww), features ordered (c, kh, kw)
//   latent[c][f][2 hh + kh][2 ww + kw] == tokens[(f * h + hh) * w + ww][(c * 2 + kh) * 2 + kw]
//
// The model keeps a chunk's latents patchified between its forwards (the head's rows are stored
// in this feature order); the latent layout is needed where a chunk enters (noise) and where it
// leaves (the hand-off to the VAE, pipeline/causal_diffusion_inference.py:666-695).  One CTA moves
// one row of tokens (f, hh) through shared memory, so both the token side (w * 4C contiguous
// values) and the latent side (2C image rows of 2w contiguous values) are accessed coalesced.
// A shared row is padded to an odd number of 32-bit words: lanes that walk along ww hit
// different banks.
#include "common.cuh"

namespace llnv {
namespace {

template <bool TO_TOKENS>
__global__ void __launch_bounds__(256) latent_tokens_kernel(uint16_t* __restrict__ tokens, int64_t ldt, uint16_t* __restrict__ latent,
                                                            int64_t stride_c, int64_t stride_f, int C, int h, int w) {
  pdl_wait();
  extern __shared__ uint32_t sm[];                            // [w][2C + 1] words: (kw = 0, kw = 1) pairs
  const int hh = blockIdx.x, f = blockIdx.y;
  const int pairs = 2 * C;                                    // (c, kh) pairs per token
  const int pitch = pairs + 1;
  uint16_t* trow = tokens + ((int64_t)f * h + hh) * w * ldt;
  const int total = w * pairs;
  if (TO_TOKENS) {
    // latent -> shared: thread walks (c, kh) slowly, ww fast: 2w contiguous values per image row
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
      const int ww = i % w, ck = i / w;
      const uint16_t* src = latent + (int64_t)(ck >> 1) * stride_c + (int64_t)f * stride_f + (int64_t)(2 * hh + (ck & 1)) * (2 * w);
      sm[ww * pitch + ck] = reinterpret_cast<const uint32_t*>(src)[ww];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
      const int ck = i % pairs, ww = i / pairs;
      reinterpret_cast<uint32_t*>(trow + (int64_t)ww * ldt)[ck] = sm[ww * pitch + ck];
    }
  } else {
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
      const int ck = i % pairs, ww = i / pairs;
      sm[ww * pitch + ck] = reinterpret_cast<const uint32_t*>(trow + (int64_t)ww * ldt)[ck];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
      const int ww = i % w, ck = i / w;
      uint16_t* dst = latent + (int64_t)(ck >> 1) * stride_c + (int64_t)f * stride_f + (int64_t)(2 * hh + (ck & 1)) * (2 * w);
      reinterpret_cast<uint32_t*>(dst)[ww] = sm[ww * pitch + ck];
    }
  }
}

int run(bool to_tokens, void* tokens, int64_t ldt, void* latent, int64_t stride_c, int64_t stride_f, int C, int F, int h, int w,
        cudaStream_t stream, const char* who) {
  LLNV_REQUIRE(C > 0 && F >= 0 && h > 0 && w > 0, "%s: bad sizes C=%d F=%d h=%d w=%d", who, C, F, h, w);
  if (F == 0) return LLNV_OK;
  LLNV_REQUIRE(tokens && latent, "%s: null tensor", who);
  LLNV_REQUIRE(ldt >= 4 * (int64_t)C && ldt % 2 == 0 && ((uintptr_t)tokens & 3) == 0, "%s: token rows must be 4-byte aligned and hold 4*C values", who);
  LLNV_REQUIRE(stride_c % 2 == 0 && stride_f % 2 == 0 && ((uintptr_t)latent & 3) == 0, "%s: latent strides must be even and the base 4-byte aligned", who);
  LLNV_REQUIRE(F <= 65535, "%s: at most 65535 frames per call", who);
  const size_t smem = (size_t)w * (2 * C + 1) * 4;
  LLNV_REQUIRE(smem <= 200 * 1024, "%s: one row of tokens (%zu bytes) does not fit shared memory", who, smem);
  auto kernel = to_tokens ? latent_tokens_kernel<true> : latent_tokens_kernel<false>;
  if (smem > 48 * 1024) LLNV_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  launch_k(kernel, dim3((unsigned)h, (unsigned)F), 256, smem, stream, (uint16_t*)tokens, ldt, (uint16_t*)latent, stride_c, stride_f, C, h, w);
  return launch_status(who);
}

}  // namespace
}  // namespace llnv

using namespace llnv;

extern "C" int llnv_patchify(const void* latent, int64_t stride_c, int64_t stride_f, void* tokens, int64_t ldt, int C, int F, int h, int w,
                             llnv_stream_t stream) {
  return run(true, tokens, ldt, const_cast<void*>(latent), stride_c, stride_f, C, F, h, w, (cudaStream_t)stream, "llnv_patchify");
}

extern "C" int llnv_unpatchify(const void* tokens, int64_t ldt, void* latent, int64_t stride_c, int64_t stride_f, int C, int F, int h, int w,
                               llnv_stream_t stream) {
  return run(false, const_cast<void*>(tokens), ldt, latent, stride_c, stride_f, C, F, h, w, (cudaStream_t)stream, "llnv_unpatchify");
}
