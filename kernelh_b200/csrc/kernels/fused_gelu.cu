// fused_gelu: out = GELU_tanh(t), two entry points.
//
//  fused_gelu       t = 1.5*x + 0.5. Replaces the kernel the reference
//                   generates from lib/dsl/kernels/fused_gelu.cpp:73-160 (an
//                   affine loop and a GELU loop fused by its `fuse` pass), same
//                   entry symbol and parameters (x, tmp, out) as rank-1 memref
//                   descriptors, 15 parameters. `tmp` is the intermediate the
//                   fusion removes: it is accepted and never touched.
//  fused_gelu_bias  t = x + bias[i], parameters (x, bias, out): the form the
//                   benchmark configuration names. No counterpart in the
//                   reference's template set.
//
// GELU_tanh(t) = 0.5 t (1 + tanh(z)), z = 0.7978845608 (t + 0.044715 t^3).
// 1 + tanh(z) = 2 / (1 + exp(-2z)), so GELU_tanh(t) = t / (1 + exp(-2z)):
// no cancellation for negative t, one exp and one divide per element.
//
// HBM-bound: 8 bytes per element (12 for the bias form). 128-bit vector
// loads/stores with streaming hints, four vectors in flight per thread,
// persistent grid-stride; scalar path for tails and misaligned/strided data.
#include "kh_device.cuh"

#ifndef KH_GELU_UNROLL
#define KH_GELU_UNROLL 4 // float4 per thread and trip; the host sizes the grid for it
#endif

namespace {

// exp(-2z) = 2^(t (c1 + c2 t^2)) with c1 = -2 * 0.7978845608 * log2(e) and c2 = 0.044715 * c1: three
// multiply-adds, one special-function exponential, one add, one approximate divide. At the small
// benchmark size the kernel has about as many issue cycles to spare as DRAM cycles, so the lean
// form is what keeps it on the memory roofline; it stays within 1e-6 relative of the fp64 value.
__device__ __forceinline__ float gelu_tanh(float t) {
  constexpr float c1 = -2.302208198f, c2 = -0.1029432396f;
  const float e = khd::exp2_approx(t * fmaf(c2, t * t, c1));
  return __fdividef(t, 1.0f + e);
}

template <bool kBias>
__device__ __forceinline__ void gelu_body(const float *__restrict__ x, int64_t x_stride,
                                          const float *__restrict__ bias, int64_t bias_stride,
                                          float *__restrict__ out, int64_t out_stride, int64_t n) {
  khd::grid_dependency_wait(); // scheduled under the previous kernel's tail: its writes are visible from here
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  bool vec_ok = khd::is_aligned16(x) && khd::is_aligned16(out) && x_stride == 1 && out_stride == 1;
  if (kBias) vec_ok = vec_ok && khd::is_aligned16(bias) && bias_stride == 1;
  int64_t done = 0;
  if (vec_ok) {
    constexpr int kUnroll = KH_GELU_UNROLL;
    const int64_t nvec = n >> 2;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    const float4 *b4 = reinterpret_cast<const float4 *>(bias);
    float4 *o4 = reinterpret_cast<float4 *>(out);
    auto apply = [&](float4 v, float4 bv) {
      if (kBias) {
        v.x += bv.x; v.y += bv.y; v.z += bv.z; v.w += bv.w;
      } else {
        v.x = fmaf(1.5f, v.x, 0.5f); v.y = fmaf(1.5f, v.y, 0.5f);
        v.z = fmaf(1.5f, v.z, 0.5f); v.w = fmaf(1.5f, v.w, 0.5f);
      }
      return make_float4(gelu_tanh(v.x), gelu_tanh(v.y), gelu_tanh(v.z), gelu_tanh(v.w));
    };
    // Trips of kUnroll vectors per thread, all loaded before the first is used; the last trip
    // is predicated rather than peeled, so any grid the host picks does whole trips only.
    const int64_t step = kUnroll * nthreads;
#pragma unroll 1
    for (int64_t base = tid; base < nvec; base += step) {
      float4 v[kUnroll], bv[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        // clamped, never predicated: a predicated load keeps the loads from issuing back to back
        const int64_t i = min(base + u * nthreads, nvec - 1);
        v[u] = __ldcs(x4 + i);
        if (kBias) bv[u] = __ldcs(b4 + i);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t i = base + u * nthreads;
        if (i < nvec) __stcs(o4 + i, apply(v[u], bv[u]));
      }
    }
    done = nvec << 2;
  }
  for (int64_t i = done + tid; i < n; i += nthreads) {
    const float t = kBias ? x[i * x_stride] + bias[i * bias_stride] : fmaf(1.5f, x[i * x_stride], 0.5f);
    out[i * out_stride] = gelu_tanh(t);
  }
}

} // namespace

extern "C" __global__ void __launch_bounds__(256)
fused_gelu(KH_MEMREF1(const float, x), KH_MEMREF1(float, tmp), KH_MEMREF1(float, out)) {
  (void)tmp_alloc; (void)tmp_ptr; (void)tmp_off; (void)tmp_size0; (void)tmp_stride0;
  gelu_body<false>(KH_DATA(x), x_stride0, nullptr, 0, KH_DATA(out), out_stride0, out_size0);
}

extern "C" __global__ void __launch_bounds__(256)
fused_gelu_bias(KH_MEMREF1(const float, x), KH_MEMREF1(const float, bias), KH_MEMREF1(float, out)) {
  gelu_body<true>(KH_DATA(x), x_stride0, KH_DATA(bias), bias_stride0, KH_DATA(out), out_stride0,
                  out_size0);
}
