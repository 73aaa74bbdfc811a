// layernorm: y = (x - mean) / sqrt(var + 1e-5) * gamma + beta per row, fp32,
// biased variance.
//
// Replaces the kernel the reference generates from
// lib/dsl/kernels/layernorm.cpp:58-153 (each thread redundantly forms the
// row's mean and variance in two passes over global memory, 106-134; eps is
// the constant 1e-5, 102), same entry symbol and parameters: (x, gamma, beta,
// y) as rank-2, rank-1, rank-1, rank-2 memref descriptors, 24 parameters.
//
// One read of x from HBM (8 bytes per element + gamma/beta, which stay in
// L2): the row sits in registers, the mean is a shuffle reduction of the sum,
// and the variance is a second reduction of (x - mean)^2 over the SAME
// registers, which keeps the reference's two-pass numerics without a second
// global read. Same row-to-thread mapping and fallbacks as softmax.
#include "kh_device.cuh"

#ifndef KH_ROW_MAX_REGS
#define KH_ROW_MAX_REGS 72
#endif

namespace {

constexpr int kMaxVec = 8;
constexpr float kEps = 1e-5f;

template <bool kWholeBlock>
__device__ __forceinline__ float row_sum(float v, float *smem) {
  v = khd::warp_sum(v);
  if (kWholeBlock) {
    const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) smem[warp] = v;
    __syncthreads();
    float acc = smem[0];
    for (int w = 1; w < nwarps; ++w) acc += smem[w];
    v = acc;
  }
  return v;
}

// kFull: the row fills all kMaxVec vectors of every thread, so nothing is clamped or predicated.
template <bool kWholeBlock, bool kFull = false>
__device__ __forceinline__ void layernorm_row_regs(const float *__restrict__ xrow,
                                                   const float *__restrict__ gamma,
                                                   const float *__restrict__ beta,
                                                   float *__restrict__ yrow, int nvec, int cols,
                                                   int lane, int tpr, float *smem) {
  const float4 *x4 = reinterpret_cast<const float4 *>(xrow);
  const float4 *g4 = reinterpret_cast<const float4 *>(gamma);
  const float4 *b4 = reinterpret_cast<const float4 *>(beta);
  float4 *y4 = reinterpret_cast<float4 *>(yrow);
  float4 v[kMaxVec];
  // Loads are unconditional (the index is clamped into the row, the value ignored later): a
  // predicated load keeps the compiler from issuing the eight of them back to back.
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) v[i] = __ldcs(x4 + (kFull ? lane + i * tpr : min(lane + i * tpr, nvec - 1)));
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i)
    if (kFull || lane + i * tpr < nvec) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  const float mean = row_sum<kWholeBlock>(s, smem) / static_cast<float>(cols);
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i)
    if (kFull || lane + i * tpr < nvec) {
      v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
      q += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
    }
  const float var = row_sum<kWholeBlock>(q, smem) / static_cast<float>(cols);
  const float rstd = 1.0f / sqrtf(var + kEps);
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int idx = lane + i * tpr;
    // unconditional like the loads of x; the register budget (64) keeps them in the output loop
    const int gi = kFull ? idx : min(idx, nvec - 1);
    const float4 g = __ldg(g4 + gi), b = __ldg(b4 + gi);
    if (kFull || idx < nvec) {
      __stcs(y4 + idx, make_float4(fmaf(v[i].x * rstd, g.x, b.x), fmaf(v[i].y * rstd, g.y, b.y),
                                   fmaf(v[i].z * rstd, g.z, b.z), fmaf(v[i].w * rstd, g.w, b.w)));
    }
  }
}

// Block-per-row rows of at most kVec float4 per thread, with the next row's
// loads issued before the current row is reduced, so a block always has a row
// in flight (the two reductions need four block barriers per row).
template <int kVec>
__device__ __forceinline__ void layernorm_rows_block_prefetch(const float *__restrict__ x,
                                                              const float *__restrict__ gamma,
                                                              const float *__restrict__ beta, float *__restrict__ y,
                                                              int64_t rows, int64_t x_stride0, int64_t y_stride0,
                                                              int nvec, int cols, float *smem) {
  const int tid = threadIdx.x, tpr = blockDim.x;
  const float4 *g4 = reinterpret_cast<const float4 *>(gamma);
  const float4 *b4 = reinterpret_cast<const float4 *>(beta);
  float4 nxt[kVec];
  const auto load_row = [&](int64_t r) {
    const float4 *x4 = reinterpret_cast<const float4 *>(x + r * x_stride0);
#pragma unroll
    for (int i = 0; i < kVec; ++i) nxt[i] = __ldcs(x4 + min(tid + i * tpr, nvec - 1)); // clamped, never predicated
  };
  if (blockIdx.x < rows) load_row(blockIdx.x);
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    float4 v[kVec];
#pragma unroll
    for (int i = 0; i < kVec; ++i) v[i] = nxt[i];
    if (r + gridDim.x < rows) load_row(r + gridDim.x);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kVec; ++i)
      if (tid + i * tpr < nvec) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    const float mean = row_sum<true>(s, smem) / static_cast<float>(cols);
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < kVec; ++i)
      if (tid + i * tpr < nvec) {
        v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
        q += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
      }
    const float var = row_sum<true>(q, smem) / static_cast<float>(cols);
    const float rstd = 1.0f / sqrtf(var + kEps);
    float4 *y4 = reinterpret_cast<float4 *>(y + r * y_stride0);
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const int idx = tid + i * tpr;
      if (idx < nvec) {
        const float4 g = __ldg(g4 + idx), b = __ldg(b4 + idx);
        __stcs(y4 + idx, make_float4(fmaf(v[i].x * rstd, g.x, b.x), fmaf(v[i].y * rstd, g.y, b.y),
                                     fmaf(v[i].z * rstd, g.z, b.z), fmaf(v[i].w * rstd, g.w, b.w)));
      }
    }
  }
}

} // namespace

// 72 registers: the host's one-wave geometry for 1024-column rows is four resident blocks of
// 224 threads per SM (4 x 7 warps x 72 x 32 = 64512 of the 65536 registers).
extern "C" __global__ void __maxnreg__(KH_ROW_MAX_REGS)
layernorm(KH_MEMREF2(const float, x), KH_MEMREF1(const float, gamma), KH_MEMREF1(const float, beta),
          KH_MEMREF2(float, y)) {
  __shared__ float smem[32];
  khd::grid_dependency_wait(); // scheduled under the previous kernel's tail: its writes are visible from here
  const float *__restrict__ x = KH_DATA(x);
  const float *__restrict__ gamma = KH_DATA(gamma);
  const float *__restrict__ beta = KH_DATA(beta);
  float *__restrict__ y = KH_DATA(y);
  const int64_t rows = x_size0, cols = x_size1;

  const bool fast = khd::is_aligned16(x) && khd::is_aligned16(y) && khd::is_aligned16(gamma) &&
                    khd::is_aligned16(beta) && x_stride1 == 1 && y_stride1 == 1 &&
                    gamma_stride0 == 1 && beta_stride0 == 1 && (x_stride0 & 3) == 0 &&
                    (y_stride0 & 3) == 0 && (cols & 3) == 0 && (blockDim.x & 31) == 0;
  if (fast && cols <= 32 * 4 * kMaxVec) {
    const int64_t warps_per_block = blockDim.x >> 5;
    const int64_t warp0 = static_cast<int64_t>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * warps_per_block;
    if (cols == 32 * 4 * kMaxVec) {
      for (int64_t r = warp0; r < rows; r += nwarps)
        layernorm_row_regs<false, true>(x + r * x_stride0, gamma, beta, y + r * y_stride0, 32 * kMaxVec,
                                        32 * 4 * kMaxVec, threadIdx.x & 31, 32, smem);
      return;
    }
    for (int64_t r = warp0; r < rows; r += nwarps)
      layernorm_row_regs<false>(x + r * x_stride0, gamma, beta, y + r * y_stride0,
                                static_cast<int>(cols >> 2), static_cast<int>(cols),
                                threadIdx.x & 31, 32, smem);
    return;
  }
  if (fast && cols <= static_cast<int64_t>(blockDim.x) * 4 * 4) {
    layernorm_rows_block_prefetch<4>(x, gamma, beta, y, rows, x_stride0, y_stride0, static_cast<int>(cols >> 2),
                                     static_cast<int>(cols), smem);
    return;
  }
  if (fast && cols <= static_cast<int64_t>(blockDim.x) * 4 * kMaxVec) {
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x)
      layernorm_row_regs<true>(x + r * x_stride0, gamma, beta, y + r * y_stride0,
                               static_cast<int>(cols >> 2), static_cast<int>(cols), threadIdx.x,
                               blockDim.x, smem);
    return;
  }
  // generic: re-reads the row for the variance and the output; any shape,
  // stride or block size. Sums are collected through shared memory by thread 0.
  __shared__ float all[256];
  __shared__ float bcast;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const float *xr = x + r * x_stride0;
    float *yr = y + r * y_stride0;
    float s = 0.f;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) s += xr[c * x_stride1];
    __syncthreads();
    all[threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
      float acc = 0.f;
      for (unsigned i = 0; i < blockDim.x; ++i) acc += all[i];
      bcast = acc / static_cast<float>(cols);
    }
    __syncthreads();
    const float mean = bcast;
    float q = 0.f;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
      const float d = xr[c * x_stride1] - mean;
      q += d * d;
    }
    __syncthreads();
    all[threadIdx.x] = q;
    __syncthreads();
    if (threadIdx.x == 0) {
      float acc = 0.f;
      for (unsigned i = 0; i < blockDim.x; ++i) acc += all[i];
      bcast = 1.0f / sqrtf(acc / static_cast<float>(cols) + kEps);
    }
    __syncthreads();
    const float rstd = bcast;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x)
      yr[c * y_stride1] = fmaf((xr[c * x_stride1] - mean) * rstd, gamma[c * gamma_stride0],
                               beta[c * beta_stride0]);
  }
}
