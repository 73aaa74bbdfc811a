// softmax: y[r, c] = exp(x[r, c] - max_r) / sum_c exp(x[r, c] - max_r), fp32.
//
// Replaces the kernel the reference generates from
// lib/dsl/kernels/softmax.cpp:68-165 (every thread re-reads its whole row to
// form the online max/sum, 134-142), same entry symbol and parameters: (x, y)
// as rank-2 memref descriptors, 14 eight-byte parameters.
//
// One pass over HBM (8 bytes per element): a row is read once with 128-bit
// loads into registers, each lane forms its own (max, sum of exp) pair, the
// pairs are merged across lanes with the online rule
//   M = max(m1, m2);  s = s1 * exp(m1 - M) + s2 * exp(m2 - M)
// by warp shuffles (plus one shared-memory exchange when a row spans the
// block), and the row is written once. Rows up to 1024 columns take a warp
// each; rows up to 8 float4 per thread take a block; anything else (long,
// misaligned or strided rows, odd block sizes) takes a two-read generic path.
// All row loops stride over the grid, so any launch geometry is correct.
#include "kh_device.cuh"

namespace {

constexpr int kMaxVec = 8; // float4 per thread held in registers

struct MaxSum {
  float m, s;
};

__device__ __forceinline__ MaxSum merge(MaxSum a, MaxSum b) {
  const float M = fmaxf(a.m, b.m);
  if (M == -INFINITY) return {M, 0.f};
  return {M, a.s * expf(a.m - M) + b.s * expf(b.m - M)};
}

__device__ __forceinline__ MaxSum warp_merge(MaxSum v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum other{__shfl_xor_sync(0xffffffffu, v.m, o), __shfl_xor_sync(0xffffffffu, v.s, o)};
    v = merge(v, other);
  }
  return v;
}

// One row held in registers by `tpr` cooperating threads (a warp, or the block).
template <bool kWholeBlock>
__device__ __forceinline__ void softmax_row_regs(const float *__restrict__ xrow,
                                                 float *__restrict__ yrow, int nvec, int lane,
                                                 int tpr, MaxSum *smem) {
  const float4 *x4 = reinterpret_cast<const float4 *>(xrow);
  float4 *y4 = reinterpret_cast<float4 *>(yrow);
  float4 v[kMaxVec];
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int idx = lane + i * tpr;
    if (idx < nvec) v[i] = __ldcs(x4 + idx);
  }
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i)
    if (lane + i * tpr < nvec) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i)
    if (lane + i * tpr < nvec) {
      v[i].x = expf(v[i].x - m);
      v[i].y = expf(v[i].y - m);
      v[i].z = expf(v[i].z - m);
      v[i].w = expf(v[i].w - m);
      s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
  MaxSum t = warp_merge({m, s});
  if (kWholeBlock) {
    const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    __syncthreads(); // smem reuse across rows
    if ((threadIdx.x & 31) == 0) smem[warp] = t;
    __syncthreads();
    MaxSum acc = smem[0];
    for (int w = 1; w < nwarps; ++w) acc = merge(acc, smem[w]);
    t = acc;
  }
  // exp(v - M) / S = exp(v - m) * exp(m - M) / S
  const float scale = (m == -INFINITY) ? 0.f : expf(m - t.m) / t.s;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int idx = lane + i * tpr;
    if (idx < nvec)
      __stcs(y4 + idx, make_float4(v[i].x * scale, v[i].y * scale, v[i].z * scale, v[i].w * scale));
  }
}

// Block-per-row rows of at most kVec float4 per thread, with the next row's
// loads issued before the current row is reduced, so a block always has a row
// in flight (the reduce needs two block barriers per row).
template <int kVec>
__device__ __forceinline__ void softmax_rows_block_prefetch(const float *__restrict__ x, float *__restrict__ y,
                                                            int64_t rows, int64_t x_stride0, int64_t y_stride0,
                                                            int nvec, MaxSum *smem) {
  const int tid = threadIdx.x, tpr = blockDim.x, warp = tid >> 5, nwarps = tpr >> 5;
  float4 nxt[kVec];
  const auto load_row = [&](int64_t r) {
    const float4 *x4 = reinterpret_cast<const float4 *>(x + r * x_stride0);
#pragma unroll
    for (int i = 0; i < kVec; ++i)
      if (tid + i * tpr < nvec) nxt[i] = __ldcs(x4 + tid + i * tpr);
  };
  if (blockIdx.x < rows) load_row(blockIdx.x);
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    float4 v[kVec];
#pragma unroll
    for (int i = 0; i < kVec; ++i) v[i] = nxt[i];
    if (r + gridDim.x < rows) load_row(r + gridDim.x);
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < kVec; ++i)
      if (tid + i * tpr < nvec) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kVec; ++i)
      if (tid + i * tpr < nvec) {
        v[i].x = expf(v[i].x - m);
        v[i].y = expf(v[i].y - m);
        v[i].z = expf(v[i].z - m);
        v[i].w = expf(v[i].w - m);
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
      }
    MaxSum t = warp_merge({m, s});
    __syncthreads(); // smem reuse across rows
    if ((tid & 31) == 0) smem[warp] = t;
    __syncthreads();
    MaxSum acc = smem[0];
    for (int w = 1; w < nwarps; ++w) acc = merge(acc, smem[w]);
    const float scale = (m == -INFINITY) ? 0.f : expf(m - acc.m) / acc.s;
    float4 *y4 = reinterpret_cast<float4 *>(y + r * y_stride0);
#pragma unroll
    for (int i = 0; i < kVec; ++i)
      if (tid + i * tpr < nvec)
        __stcs(y4 + tid + i * tpr, make_float4(v[i].x * scale, v[i].y * scale, v[i].z * scale, v[i].w * scale));
  }
}

} // namespace

extern "C" __global__ void __launch_bounds__(256)
softmax(KH_MEMREF2(const float, x), KH_MEMREF2(float, y)) {
  __shared__ MaxSum smem[32];
  const float *__restrict__ x = KH_DATA(x);
  float *__restrict__ y = KH_DATA(y);
  const int64_t rows = x_size0, cols = x_size1;

  const bool fast = khd::is_aligned16(x) && khd::is_aligned16(y) && x_stride1 == 1 &&
                    y_stride1 == 1 && (x_stride0 & 3) == 0 && (y_stride0 & 3) == 0 &&
                    (cols & 3) == 0 && (blockDim.x & 31) == 0;
  if (fast && cols <= 32 * 4 * kMaxVec) {
    // a warp per row
    const int64_t warps_per_block = blockDim.x >> 5;
    const int64_t warp0 = static_cast<int64_t>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * warps_per_block;
    for (int64_t r = warp0; r < rows; r += nwarps)
      softmax_row_regs<false>(x + r * x_stride0, y + r * y_stride0, static_cast<int>(cols >> 2),
                              threadIdx.x & 31, 32, smem);
    return;
  }
  if (fast && cols <= static_cast<int64_t>(blockDim.x) * 4 * 4) {
    // the block per row, next row prefetched
    softmax_rows_block_prefetch<4>(x, y, rows, x_stride0, y_stride0, static_cast<int>(cols >> 2), smem);
    return;
  }
  if (fast && cols <= static_cast<int64_t>(blockDim.x) * 4 * kMaxVec) {
    // the block per row
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x)
      softmax_row_regs<true>(x + r * x_stride0, y + r * y_stride0, static_cast<int>(cols >> 2),
                             threadIdx.x, blockDim.x, smem);
    return;
  }
  // generic: two reads of the row, any shape, stride or block size
  __shared__ MaxSum part[256 / 32 + 1];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const float *xr = x + r * x_stride0;
    float *yr = y + r * y_stride0;
    MaxSum t{-INFINITY, 0.f};
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) t = merge(t, {xr[c * x_stride1], 1.f});
    // block merge without assuming full warps: lane 0 of each 32-thread group
    // collects through shared memory
    __shared__ MaxSum all[256];
    __syncthreads();
    all[threadIdx.x] = t;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) {
      MaxSum acc = t;
      for (int i = 1; i < 32 && threadIdx.x + i < blockDim.x; ++i) acc = merge(acc, all[threadIdx.x + i]);
      part[threadIdx.x >> 5] = acc;
    }
    __syncthreads();
    MaxSum acc = part[0];
    for (int w = 1; w < static_cast<int>((blockDim.x + 31) >> 5); ++w) acc = merge(acc, part[w]);
    const float inv = 1.0f / acc.s;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x)
      yr[c * y_stride1] = expf(xr[c * x_stride1] - acc.m) * inv;
  }
}
