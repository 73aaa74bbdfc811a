// softmax: y[r, c] = exp(x[r, c] - max_r) / sum_c exp(x[r, c] - max_r), fp32.
//
// Replaces the kernel the reference generates from
// lib/dsl/kernels/softmax.cpp:68-165 (every thread re-reads its whole row to
// form the online max/sum, 134-142), same entry symbol and parameters: (x, y)
// as rank-2 memref descriptors, 14 eight-byte parameters.
//
// One pass over HBM (8 bytes per element): a row is read once with 128-bit
// loads into registers; a warp takes the maximum m of its part in one redux
// instruction, forms exp(v - m) as 2^(v log2e - m log2e) (one fused
// multiply-add and one special-function instruction per element: the kernel
// has about as many instruction-issue cycles to spare as it has DRAM cycles at
// the small benchmark size, so the lean form is what keeps it on the memory
// roofline) and sums by shuffles; when a row spans the block the warps' (m, s)
// pairs are merged through shared memory with the online rule
//   M = max(m1, m2);  s = s1 * exp(m1 - M) + s2 * exp(m2 - M)
// and the row is written once. The rounding of m log2e is common to the whole
// row and cancels in the quotient. Rows up to 1024 columns take a warp
// each; rows up to 8 float4 per thread take a block; anything else (long,
// misaligned or strided rows, odd block sizes) takes a two-read generic path.
// All row loops stride over the grid, so any launch geometry is correct.
#include "kh_device.cuh"

#ifndef KH_ROW_MIN_BLOCKS
#define KH_ROW_MIN_BLOCKS 4 // resident blocks per SM the register budget is cut for
#endif

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

constexpr float kLog2e = 1.4426950408889634f;

// exp(v - m) for a lane's vectors, given mb = m * log2e; returns the lane's sum.
__device__ __forceinline__ float exp_in_place(float4 &v, float mb) {
  v.x = khd::exp2_approx(fmaf(v.x, kLog2e, -mb));
  v.y = khd::exp2_approx(fmaf(v.y, kLog2e, -mb));
  v.z = khd::exp2_approx(fmaf(v.z, kLog2e, -mb));
  v.w = khd::exp2_approx(fmaf(v.w, kLog2e, -mb));
  return (v.x + v.y) + (v.z + v.w);
}

// One row held in registers by `tpr` cooperating threads (a warp, or the block).
template <bool kWholeBlock>
__device__ __forceinline__ void softmax_row_regs(const float *__restrict__ xrow,
                                                 float *__restrict__ yrow, int nvec, int lane,
                                                 int tpr, MaxSum *smem) {
  const float4 *x4 = reinterpret_cast<const float4 *>(xrow);
  float4 *y4 = reinterpret_cast<float4 *>(yrow);
  float4 v[kMaxVec];
  // Loads are unconditional (the index is clamped into the row, the value ignored later): a
  // predicated load keeps the compiler from issuing the eight of them back to back.
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) v[i] = __ldcs(x4 + min(lane + i * tpr, nvec - 1));
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i)
    if (lane + i * tpr < nvec) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
  m = khd::warp_max_redux(m);
  const float mb = (m == -INFINITY) ? 0.f : m * kLog2e; // a part of -inf only: every exp is 0
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i)
    if (lane + i * tpr < nvec) s += exp_in_place(v[i], mb);
  MaxSum t{m, khd::warp_sum(s)};
  if (kWholeBlock) {
    const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    __syncthreads(); // smem reuse across rows
    if ((threadIdx.x & 31) == 0) smem[warp] = t;
    __syncthreads();
    MaxSum acc = smem[0];
    for (int w = 1; w < nwarps; ++w) acc = merge(acc, smem[w]);
    t = acc;
  }
  // exp(v - M) / S = exp(v - m) * exp(m - M) / S, m the warp's maximum and M the row's
  const float scale = (m == -INFINITY) ? 0.f : (kWholeBlock ? expf(m - t.m) : 1.0f) / t.s;
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
    for (int i = 0; i < kVec; ++i) nxt[i] = __ldcs(x4 + min(tid + i * tpr, nvec - 1)); // clamped, never predicated
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
    m = khd::warp_max_redux(m);
    const float mb = (m == -INFINITY) ? 0.f : m * kLog2e;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kVec; ++i)
      if (tid + i * tpr < nvec) s += exp_in_place(v[i], mb);
    MaxSum t{m, khd::warp_sum(s)};
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

// Four blocks of up to 256 threads per SM is what the host's one-wave geometry needs: 64 registers.
extern "C" __global__ void __launch_bounds__(256, KH_ROW_MIN_BLOCKS)
softmax(KH_MEMREF2(const float, x), KH_MEMREF2(float, y)) {
  __shared__ MaxSum smem[32];
  khd::grid_dependency_wait(); // scheduled under the previous kernel's tail: its writes are visible from here
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
