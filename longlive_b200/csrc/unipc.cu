// One step of the flow-matching UniPC scheduler as a single elementwise pass.
//
// The reference's scheduler.step (wan_5b/utils/fm_solvers_unipc.py:657-741) is about twenty
// PyTorch calls on the chunk's latents: convert the flow prediction to an x0 prediction
// (:320-323), correct the current sample with it (UniC, :488-628), then predict the next sample
// (UniP, :352-486).  Every call reads and writes whole tensors; here each element is loaded once
// (flow prediction, sample, the two older x0 predictions, the sample the previous prediction
// started from), goes through the same sequence of operations in registers, and the three results
// (x0 prediction, corrected sample, next sample) are stored once.
//
// Rounding follows PyTorch's CUDA kernels, so results are bit-identical to the reference running on
// a GPU: every tensor operation is computed in fp32 and rounded to the latents' dtype (bf16 or
// fp32) before the next one uses it; fp32 scalars stay fp32; a division by a scalar is a
// multiplication by its fp32 reciprocal; the corrector / predictor weights (rho) arrive already
// rounded to the latents' dtype.  Products and sums use the non-contracting intrinsics so that no
// multiply-add is fused; values are processed in pairs so that a bf16 rounding is half a paired conversion.  The scalar coefficients are computed on the host.
#include "common.cuh"

namespace llnv {
namespace {

struct Coef {
  float sigma;                                    // sigma of this step: x0 = sample - sigma * flow
  int use_corrector, corrector_order;
  float cc1, cc2, cc3, c_inv_rk, c_rho0, c_rho1;  // UniC: sigma ratio, alpha_t * h_phi_1, alpha_t * B(h), 1 / r_1, weights
  int predictor_order;
  float pc1, pc2, pc3, p_inv_rk, p_zero;          // UniP; p_zero = alpha_t * B(h) * 0 (order 1 subtracts it)
};

template <bool BF16>
__device__ __forceinline__ float rnd(float x) {
  if constexpr (BF16) return round_bf16(x);
  return x;
}

// Two values per call: the bf16 rounding of a pair is one cvt.rn.bf16x2.f32 (the scalar conversion
// issues on the quarter-rate XU pipe and made the kernel instruction-bound).
struct P2 {
  float a, b;
};
template <bool BF16>
__device__ __forceinline__ P2 R(P2 v) {
  if constexpr (BF16) round_bf16x2(v.a, v.b);
  return v;
}
__device__ __forceinline__ P2 mul_s(float s, P2 v) { return {__fmul_rn(s, v.a), __fmul_rn(s, v.b)}; }
__device__ __forceinline__ P2 sub2(P2 x, P2 y) { return {__fsub_rn(x.a, y.a), __fsub_rn(x.b, y.b)}; }
__device__ __forceinline__ P2 add2(P2 x, P2 y) { return {__fadd_rn(x.a, y.a), __fadd_rn(x.b, y.b)}; }

template <bool BF16>
__device__ __forceinline__ void step_pair(const Coef& c, P2 v, P2 x, P2 m0p, P2 m1p, P2 last, P2& x0_out, P2& xs_out, P2& next_out) {
  const P2 x0 = R<BF16>(sub2(x, R<BF16>(mul_s(c.sigma, v))));
  P2 xs = x;
  if (c.use_corrector) {
    const P2 xt = R<BF16>(sub2(R<BF16>(mul_s(c.cc1, last)), R<BF16>(mul_s(c.cc2, m0p))));
    P2 res = R<BF16>(mul_s(c.c_rho1, R<BF16>(sub2(x0, m0p))));
    if (c.corrector_order == 2) {
      const P2 d1 = R<BF16>(mul_s(c.c_inv_rk, R<BF16>(sub2(m1p, m0p))));
      res = R<BF16>(add2(R<BF16>(mul_s(c.c_rho0, d1)), res));
    }
    xs = R<BF16>(sub2(xt, R<BF16>(mul_s(c.cc3, res))));
  }
  const P2 xt = R<BF16>(sub2(R<BF16>(mul_s(c.pc1, xs)), R<BF16>(mul_s(c.pc2, x0))));
  P2 next;
  if (c.predictor_order == 2) {
    const P2 d1 = R<BF16>(mul_s(c.p_inv_rk, R<BF16>(sub2(m0p, x0))));
    next = R<BF16>(sub2(xt, R<BF16>(mul_s(c.pc3, R<BF16>(mul_s(0.5f, d1))))));
  } else {
    next = R<BF16>(sub2(xt, P2{c.p_zero, c.p_zero}));
  }
  x0_out = x0;
  xs_out = xs;
  next_out = next;
}

template <bool BF16>
__device__ __forceinline__ void step_element(const Coef& c, float v, float x, float m0p, float m1p, float last, float& x0_out,
                                             float& xs_out, float& next_out) {
  P2 o0, o1, o2;
  step_pair<BF16>(c, {v, v}, {x, x}, {m0p, m0p}, {m1p, m1p}, {last, last}, o0, o1, o2);
  x0_out = o0.a;
  xs_out = o1.a;
  next_out = o2.a;
}

template <bool BF16>
struct Elem;
template <>
struct Elem<true> {
  using T = uint16_t;
  static constexpr int kVec = 8;
  static __device__ __forceinline__ float load(const T* p) { return __uint_as_float((uint32_t)*p << 16); }
  static __device__ __forceinline__ void store(T* p, float f) { *p = (T)f2bf(f); }
  static __device__ __forceinline__ void store2(T* p, P2 v) { *reinterpret_cast<uint32_t*>(p) = pack_bf16x2(v.a, v.b); }
};
template <>
struct Elem<false> {
  using T = float;
  static constexpr int kVec = 4;
  static __device__ __forceinline__ float load(const T* p) { return *p; }
  static __device__ __forceinline__ void store(T* p, float f) { *p = f; }
  static __device__ __forceinline__ void store2(T* p, P2 v) {
    p[0] = v.a;
    p[1] = v.b;
  }
};

// The output pointers may equal input pointers (the x0 history rotates in place, the next sample
// may overwrite the sample): an element is read before it is written, by the same thread.
template <bool BF16, bool VEC>
__global__ void __launch_bounds__(256) unipc_step_kernel(const void* v_, const void* x_, const void* m0_, const void* m1_, const void* last_,
                                                         void* x0_, void* xs_, void* next_, int64_t n, const __grid_constant__ Coef c) {
  pdl_wait();
  using E = Elem<BF16>;
  using T = typename E::T;
  const T* v = (const T*)v_;
  const T* x = (const T*)x_;
  const T* m0 = (const T*)m0_;
  const T* m1 = (const T*)m1_;
  const T* last = (const T*)last_;
  T* x0o = (T*)x0_;
  T* xso = (T*)xs_;
  T* nxo = (T*)next_;
  const bool need_m0 = c.use_corrector || c.predictor_order == 2;
  const bool need_m1 = c.use_corrector && c.corrector_order == 2;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if constexpr (VEC) {
    constexpr int V = E::kVec;
    const int64_t nv = n / V;
    for (int64_t i = tid; i < nv; i += stride) {
      T a[V], b[V], p[V] = {}, q[V] = {}, l[V] = {}, r0[V], r1[V], r2[V];
      *reinterpret_cast<uint4*>(a) = reinterpret_cast<const uint4*>(v)[i];
      *reinterpret_cast<uint4*>(b) = reinterpret_cast<const uint4*>(x)[i];
      if (need_m0) *reinterpret_cast<uint4*>(p) = reinterpret_cast<const uint4*>(m0)[i];
      if (need_m1) *reinterpret_cast<uint4*>(q) = reinterpret_cast<const uint4*>(m1)[i];
      if (c.use_corrector) *reinterpret_cast<uint4*>(l) = reinterpret_cast<const uint4*>(last)[i];
#pragma unroll
      for (int j = 0; j < V; j += 2) {
        P2 o0, o1, o2;
        step_pair<BF16>(c, {E::load(a + j), E::load(a + j + 1)}, {E::load(b + j), E::load(b + j + 1)}, {E::load(p + j), E::load(p + j + 1)},
                        {E::load(q + j), E::load(q + j + 1)}, {E::load(l + j), E::load(l + j + 1)}, o0, o1, o2);
        E::store2(r0 + j, o0);
        E::store2(r1 + j, o1);
        E::store2(r2 + j, o2);
      }
      reinterpret_cast<uint4*>(x0o)[i] = *reinterpret_cast<uint4*>(r0);
      reinterpret_cast<uint4*>(xso)[i] = *reinterpret_cast<uint4*>(r1);
      reinterpret_cast<uint4*>(nxo)[i] = *reinterpret_cast<uint4*>(r2);
    }
    for (int64_t i = nv * V + tid; i < n; i += stride) {
      float o0, o1, o2;
      step_element<BF16>(c, E::load(v + i), E::load(x + i), need_m0 ? E::load(m0 + i) : 0.f, need_m1 ? E::load(m1 + i) : 0.f,
                         c.use_corrector ? E::load(last + i) : 0.f, o0, o1, o2);
      E::store(x0o + i, o0);
      E::store(xso + i, o1);
      E::store(nxo + i, o2);
    }
  } else {
    for (int64_t i = tid; i < n; i += stride) {
      float o0, o1, o2;
      step_element<BF16>(c, E::load(v + i), E::load(x + i), need_m0 ? E::load(m0 + i) : 0.f, need_m1 ? E::load(m1 + i) : 0.f,
                         c.use_corrector ? E::load(last + i) : 0.f, o0, o1, o2);
      E::store(x0o + i, o0);
      E::store(xso + i, o1);
      E::store(nxo + i, o2);
    }
  }
}

}  // namespace
}  // namespace llnv

using namespace llnv;

extern "C" int llnv_unipc_step(const void* model_output, const void* sample, const void* x0_prev, const void* x0_older,
                               const void* last_sample, void* x0_out, void* sample_out, void* next_out, int64_t n, int dtype,
                               const llnv_unipc_coef* coef, llnv_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  LLNV_REQUIRE(coef != nullptr, "llnv_unipc_step: null coefficients");
  LLNV_REQUIRE(n >= 0, "llnv_unipc_step: negative size");
  LLNV_REQUIRE(dtype == 0 || dtype == 1, "llnv_unipc_step: dtype is 0 (bf16) or 1 (fp32), got %d", dtype);
  LLNV_REQUIRE(coef->predictor_order == 1 || coef->predictor_order == 2, "llnv_unipc_step: predictor order 1 or 2 (got %d)",
               coef->predictor_order);
  LLNV_REQUIRE(!coef->use_corrector || coef->corrector_order == 1 || coef->corrector_order == 2,
               "llnv_unipc_step: corrector order 1 or 2 (got %d)", coef->corrector_order);
  if (n == 0) return LLNV_OK;
  LLNV_REQUIRE(model_output && sample && x0_out && sample_out && next_out, "llnv_unipc_step: null tensor");
  const bool need_m0 = coef->use_corrector || coef->predictor_order == 2;
  const bool need_m1 = coef->use_corrector && coef->corrector_order == 2;
  LLNV_REQUIRE(!need_m0 || x0_prev, "llnv_unipc_step: this step needs the previous x0 prediction");
  LLNV_REQUIRE(!need_m1 || x0_older, "llnv_unipc_step: this step needs the x0 prediction before the previous one");
  LLNV_REQUIRE(!coef->use_corrector || last_sample, "llnv_unipc_step: the corrector needs the previous step's sample");
  Coef c;
  c.sigma = coef->sigma;
  c.use_corrector = coef->use_corrector;
  c.corrector_order = coef->corrector_order;
  c.cc1 = coef->cc1, c.cc2 = coef->cc2, c.cc3 = coef->cc3, c.c_inv_rk = coef->c_inv_rk, c.c_rho0 = coef->c_rho0, c.c_rho1 = coef->c_rho1;
  c.predictor_order = coef->predictor_order;
  c.pc1 = coef->pc1, c.pc2 = coef->pc2, c.pc3 = coef->pc3, c.p_inv_rk = coef->p_inv_rk, c.p_zero = coef->p_zero;
  const uintptr_t all = (uintptr_t)model_output | (uintptr_t)sample | (uintptr_t)x0_out | (uintptr_t)sample_out | (uintptr_t)next_out |
                        (need_m0 ? (uintptr_t)x0_prev : 0) | (need_m1 ? (uintptr_t)x0_older : 0) |
                        (coef->use_corrector ? (uintptr_t)last_sample : 0);
  const int esize = dtype == 0 ? 2 : 4;
  LLNV_REQUIRE((all & (uintptr_t)(esize - 1)) == 0, "llnv_unipc_step: tensors must be aligned to their element size");
  const bool vec = (all & 15) == 0;
  const int per_thread = vec ? 16 / esize : 1;
  int64_t blocks = (n / per_thread + 255) / 256 + 1;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  const dim3 grid((unsigned)blocks);
#define LLNV_UNIPC_LAUNCH(BF, VEC) \
  launch_k(unipc_step_kernel<BF, VEC>, grid, 256, 0, stream, model_output, sample, x0_prev, x0_older, last_sample, x0_out, sample_out, next_out, n, c)
  if (dtype == 0) {
    if (vec) LLNV_UNIPC_LAUNCH(true, true);
    else LLNV_UNIPC_LAUNCH(true, false);
  } else {
    if (vec) LLNV_UNIPC_LAUNCH(false, true);
    else LLNV_UNIPC_LAUNCH(false, false);
  }
#undef LLNV_UNIPC_LAUNCH
  return launch_status("unipc_step_kernel");
}
