// gemm: C = A . B, row-major fp32, A is m x k, B is k x n, C is m x n, zero
// seeded accumulator and a plain store (no alpha/beta).
//
// Replaces the kernel the reference generates from
// lib/dsl/kernels/gemm.cpp:116-296 (32x32x32 tiles of scalar fp32 FMAs, one
// k-tile staged in 8 KiB of static shared memory). Entry symbol `gemm`; the
// first 21 parameters are the reference's: (A, B, C) as rank-2 memref
// descriptors. The TMA-fed kernel then takes four tensor maps, the k-block
// count, a status pointer and the two scale-exponent arrays.
//
// Arithmetic: fp32 results from three fp16 tensor-core products ("3xFP16").
// Every row of A and every column of B is first scaled by an exact power of
// two that brings its largest magnitude into [2^14, 2^15), so the whole row
// sits in the upper part of the fp16 range. A scaled value x is split into
// hi = fp16(x) (round to nearest) and lo = fp16(x - hi) (the difference is exact
// in fp32): 22 significand bits for every element within 2^-17 of its row's
// largest, an absolute floor of 2^-38 of the largest below that. Every k-step
// issues three tcgen05 products into one fp32 accumulator in tensor memory:
// lo.hi, hi.lo, hi.hi (lo.lo, ~2^-22 relative, is dropped), and the epilogue
// undoes the two scalings exactly with ldexp. This carries the same number of
// significand bits as a tf32 hi/lo split at twice the tensor rate, and the fp16
// array draws less power per product, so the SM clock the part sustains under
// its power cap costs less too (measured on random operands: kind::f16 holds
// 1625 TFLOP/s at 1340 MHz, kind::tf32 907-943 TFLOP/s at 1500-1560 MHz).
// The tensor core's fp32 accumulation truncates, which biases long sums (the
// error grew linearly with k when a whole k = 8192 product stayed in tensor
// memory), so only K = 256 is accumulated there at a time: two accumulators
// alternate, and each finished chunk is added into fp32 registers with
// round-to-nearest by the epilogue warps while the next chunk is running.
//
// Four launches:
//  gemm_split_a   per row of A: largest magnitude, scale exponent, then A_hi,
//      A_lo (m x kp fp16, kp = k rounded up to 32, zero padded); long rows are
//      staged whole in shared memory by bulk copies (TMA), double buffered.
//      It also clears the column maxima for the next launch.
//  gemm_colmax_b  largest magnitude of every column of B (atomic max on the
//      bit patterns of |b|, which order like the values).
//  gemm_split_bt  B^T_hi, B^T_lo (n x kp fp16) through 64 x 128 shared-memory
//      tiles, so both tensor-core operands are K-major with 64-byte rows.
//  gemm           persistent two-CTA clusters (tcgen05 cta_group::2), one per
//      pair of SMs, walk the 256 x 256 tiles of C. CTA r of a pair holds rows
//      128r..128r+127 of the A tile and of the accumulator and only HALF of the
//      B tile (128 of its 256 columns); one tcgen05.mma.cta_group::2 (M 256,
//      N 256, K 16), issued by the leader CTA, runs both tensor cores and lets
//      each read the other's half of B. Per CTA: warp 0 feeds a 6-stage ring of
//      {A_hi, A_lo, B_hi half, B_lo half} k-blocks (32 fp16 deep, 32 KiB per
//      stage) with TMA (64-byte swizzle; out-of-range rows read as zero, which
//      is what makes ragged m and n work); warp 1 of the leader issues the MMAs
//      and releases stages with tcgen05.commit; warps 2-9 drain the 256-column
//      fp32 accumulators from tensor memory chunk by chunk and store C.
//
// Synchronisation across the pair (no multicast qualifier is used anywhere):
//  * TMA loads of both CTAs complete on the LEADER's "full" barrier (the peer
//    addresses it through the cluster window), which expects both halves.
//  * the leader's tcgen05.commit arrives on the "empty" and "accumulator full"
//    barriers of BOTH CTAs (one commit per CTA, peer address from mapa).
//  * the epilogue warps of both CTAs arrive on the leader's "accumulator empty"
//    barrier (the peer's arrivals are remote).
// Every wait is bounded; the two cluster-wide barriers at the start and the
// end are hardware barriers that every thread reaches.
//
// Tensor-bound: 2 m n k useful flops; three MMAs per k-step put the ceiling
// at one third of the fp16 tensor rate.
#include "kh_fp16_split.cuh"
#include "kh_tcgen05.cuh"

namespace {

using khd::Half8;
using khd::RowScale;
using khd::row_scale;
using khd::scale_pow2;
using khd::scale_shift;
using khd::split_fp16_pairs;
using khd::split_fp16x2;

constexpr int kBM = 128;     // rows per CTA (256 per pair)
constexpr int kBN = 256;     // columns per pair
constexpr int kBK = 32;      // fp16 elements per k-block: one 64-byte swizzle row
constexpr int kStages = 6;
constexpr int kTileBytes = kBM * kBK * 2;   // 8 KiB: A_hi, A_lo, B_hi half, B_lo half
constexpr int kStageBytes = 4 * kTileBytes; // 32 KiB per CTA
constexpr int kTmemCols = 512;              // two 256-column accumulators, used alternately
constexpr int kChunkBlocks = 8;             // k-blocks accumulated in tensor memory before a drain (K = 256)
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 64 + 32 * kEpilogueWarps; // TMA warp + MMA warp + epilogue warps
constexpr int kGroupM = 8;                  // default: pair tiles (256 rows) per rasterisation group (L2 reuse of B)

// Ordered accesses for the epilogue (see the store loop of gemm_body).
__device__ __forceinline__ int4 load_shift4(const int *p) {
  int4 v;
  asm volatile("ld.global.nc.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ int load_shift(const int *p) {
  int v;
  asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ void store_float4(float *p, float x, float y, float z, float w) {
  asm volatile("st.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}
__device__ __forceinline__ void store_float(float *p, float x) {
  asm volatile("st.global.f32 [%0], %1;" ::"l"(p), "f"(x) : "memory");
}
// The same through an NVLink multicast address: the switch delivers the store to every bound GPU.
__device__ __forceinline__ void multicast_store_float4(float *p, float x, float y, float z, float w) {
  asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(x), "f"(y), "f"(z), "f"(w)
               : "memory");
}
__device__ __forceinline__ void multicast_store_float(float *p, float x) {
  asm volatile("multimem.st.weak.global.f32 [%0], %1;" ::"l"(p), "f"(x) : "memory");
}


} // namespace

// A (m x k, any strides) -> hi, lo (m x kp fp16, contiguous, zero padded in k)
// and the scale exponent of every row. A team of kTeam threads (a warp for
// short rows, the whole block for long ones) owns a row: it reads the row once
// into registers (kHeld groups of 8 values per thread; longer rows are read
// again for the second step), reduces the largest magnitude, and writes the two splits.
template <int kTeam, int kHeld>
__device__ __forceinline__ void split_a_rows(const float *__restrict__ a, int64_t m, int64_t k, int64_t a_stride0,
                                             int64_t a_stride1, __half *__restrict__ hi, __half *__restrict__ lo,
                                             int *__restrict__ a_shift, int64_t kp, float *team_max) {
  constexpr int kTeamsPerBlock = 256 / kTeam;
  const int team = threadIdx.x / kTeam, member = threadIdx.x % kTeam;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool vec_ok = khd::is_aligned16(a) && a_stride1 == 1 && (a_stride0 & 3) == 0;
  const bool fits = kHeld > 0 && kp <= static_cast<int64_t>(kTeam) * 8 * kHeld;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * kTeamsPerBlock;
  const int64_t step = static_cast<int64_t>(gridDim.x) * kTeamsPerBlock;
  // every team of a block makes the same number of trips (block-wide barriers below)
  for (int64_t r0 = first; r0 < m; r0 += step) {
    const int64_t r = r0 + team;
    const bool live = r < m;
    const float *row = a + (live ? r : 0) * a_stride0;
    float v[kHeld > 0 ? kHeld : 1][8];
    float amax = 0.f;
    const auto load8 = [&](int64_t c, float (&out)[8]) {
      if (vec_ok && c + 8 <= k) {
        const float4 f0 = __ldcs(reinterpret_cast<const float4 *>(row + c));
        const float4 f1 = __ldcs(reinterpret_cast<const float4 *>(row + c + 4));
        out[0] = f0.x; out[1] = f0.y; out[2] = f0.z; out[3] = f0.w;
        out[4] = f1.x; out[5] = f1.y; out[6] = f1.z; out[7] = f1.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) out[j] = (c + j < k) ? row[(c + j) * a_stride1] : 0.f;
      }
    };
    if (live) {
      if (fits) {
#pragma unroll
        for (int g = 0; g < kHeld; ++g) {
          const int64_t c = (static_cast<int64_t>(g) * kTeam + member) * 8;
          if (c < kp) {
            load8(c, v[g]);
#pragma unroll
            for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[g][j]));
          }
        }
      } else {
        for (int64_t c = static_cast<int64_t>(member) * 8; c < kp; c += kTeam * 8) {
          float t[8];
          load8(c, t);
#pragma unroll
          for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(t[j]));
        }
      }
    }
    amax = khd::warp_max(amax);
    if (kTeam > 32) {
      __syncthreads();
      if (lane == 0) team_max[warp] = amax;
      __syncthreads();
      amax = team_max[0];
#pragma unroll
      for (int w = 1; w < 8; ++w) amax = fmaxf(amax, team_max[w]);
    }
    if (!live) continue;
    const int shift = scale_shift(amax);
    const RowScale scale = row_scale(shift);
    if (member == 0) a_shift[r] = shift;
    const auto store8 = [&](int64_t c, const float (&in)[8]) {
      Half8 h, l;
      const float2 x[4] = {make_float2(in[0], in[1]), make_float2(in[2], in[3]), make_float2(in[4], in[5]),
                           make_float2(in[6], in[7])};
      split_fp16_pairs<4>(x, scale, h.v, l.v);
      *reinterpret_cast<Half8 *>(hi + r * kp + c) = h;
      *reinterpret_cast<Half8 *>(lo + r * kp + c) = l;
    };
    if (fits) {
#pragma unroll
      for (int g = 0; g < kHeld; ++g) {
        const int64_t c = (static_cast<int64_t>(g) * kTeam + member) * 8;
        if (c < kp) store8(c, v[g]);
      }
    } else {
      for (int64_t c = static_cast<int64_t>(member) * 8; c < kp; c += kTeam * 8) {
        float t[8];
        load8(c, t);
        store8(c, t);
      }
    }
  }
}

// Rows of 1025..8192 values, contiguous and 16-byte aligned: the whole row is
// brought into shared memory by one bulk copy (TMA) while the block works on
// the previous row, so a row is read from HBM exactly once and the copies never
// stop. Two row buffers in dynamic shared memory.
__device__ __forceinline__ void split_a_staged(const float *__restrict__ a, int64_t m, int64_t k, int64_t a_stride0,
                                               __half *__restrict__ hi, __half *__restrict__ lo,
                                               int *__restrict__ a_shift, int64_t kp, uint32_t *status,
                                               float *team_max) {
  extern __shared__ __align__(16) uint8_t staged_rows[];
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ int s_abort;
  const uint32_t row_bytes = static_cast<uint32_t>(k) * 4u;
  const uint32_t buf0 = khd::smem_u32(staged_rows), bar0 = khd::smem_u32(&bars[0]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    s_abort = 0;
    khd::mbar_init(bar0, 1);
    khd::mbar_init(bar0 + 8, 1);
    khd::mbar_fence_init();
  }
  __syncthreads();
  const auto fetch = [&](int64_t r, int buf) {
    khd::mbar_arrive_expect_tx(bar0 + 8 * buf, row_bytes);
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     buf0 + buf * row_bytes),
                 "l"(a + r * a_stride0), "r"(row_bytes), "r"(bar0 + 8 * buf)
                 : "memory");
  };
  if (threadIdx.x == 0 && blockIdx.x < m) fetch(blockIdx.x, 0);
  int64_t trip = 0;
  for (int64_t r = blockIdx.x; r < m; r += gridDim.x, ++trip) {
    const int buf = static_cast<int>(trip & 1);
    if (threadIdx.x == 0 && r + gridDim.x < m) fetch(r + gridDim.x, buf ^ 1);
    bool ok = khd::mbar_wait(bar0 + 8 * buf, static_cast<uint32_t>(trip >> 1) & 1u, &s_abort, status,
                             khd::kStatusTmaWaitTimeout, static_cast<uint32_t>(r));
    if (!__syncthreads_and(ok)) break;
    const float *row = reinterpret_cast<const float *>(staged_rows + buf * row_bytes);
    float amax = 0.f;
    for (int64_t c = static_cast<int64_t>(threadIdx.x) * 4; c < k; c += 1024) { // k is a multiple of 4
      const float4 f = *reinterpret_cast<const float4 *>(row + c);
      amax = fmaxf(amax, fmaxf(fmaxf(fabsf(f.x), fabsf(f.y)), fmaxf(fabsf(f.z), fabsf(f.w))));
    }
    amax = khd::warp_max(amax);
    if (lane == 0) team_max[warp] = amax;
    __syncthreads();
    amax = team_max[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, team_max[w]);
    const int shift = scale_shift(amax);
    const RowScale scale = row_scale(shift);
    if (threadIdx.x == 0) a_shift[r] = shift;
    for (int64_t c = static_cast<int64_t>(threadIdx.x) * 8; c < kp; c += 2048) {
      float v[8];
      if (c + 8 <= k) {
        const float4 f0 = *reinterpret_cast<const float4 *>(row + c);
        const float4 f1 = *reinterpret_cast<const float4 *>(row + c + 4);
        v[0] = f0.x; v[1] = f0.y; v[2] = f0.z; v[3] = f0.w;
        v[4] = f1.x; v[5] = f1.y; v[6] = f1.z; v[7] = f1.w;
      } else {
#pragma unroll
        for (int q = 0; q < 8; ++q) v[q] = (c + q < k) ? row[c + q] : 0.f;
      }
      Half8 h, l;
      const float2 x[4] = {make_float2(v[0], v[1]), make_float2(v[2], v[3]), make_float2(v[4], v[5]),
                           make_float2(v[6], v[7])};
      split_fp16_pairs<4>(x, scale, h.v, l.v);
      *reinterpret_cast<Half8 *>(hi + r * kp + c) = h;
      *reinterpret_cast<Half8 *>(lo + r * kp + c) = l;
    }
    __syncthreads(); // the row buffer and team_max are free again
  }
  if (s_abort) // a wait ran out: give the copy still in flight time to land before the block leaves
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
}

__device__ __forceinline__ uint32_t dynamic_smem_bytes() {
  uint32_t v;
  asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(v));
  return v;
}

extern "C" __global__ void __launch_bounds__(256, 3)
gemm_split_a(KH_MEMREF2(const float, a), __half *__restrict__ hi, __half *__restrict__ lo,
             int *__restrict__ a_shift, uint32_t *__restrict__ b_amax, int64_t b_cols, int64_t kp,
             uint32_t *status) {
  __shared__ float team_max[8];
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < b_cols;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    b_amax[i] = 0u;
  const float *a = KH_DATA(a);
  const int64_t k = a_size1;
  const bool stageable = kp > 1024 && (k & 3) == 0 && a_stride1 == 1 && (a_stride0 & 3) == 0 &&
                         khd::is_aligned16(a) && static_cast<uint64_t>(k) * 8 <= dynamic_smem_bytes();
  if (stageable)
    split_a_staged(a, a_size0, k, a_stride0, hi, lo, a_shift, kp, status, team_max);
  else if (kp <= 1024)
    split_a_rows<32, 4>(a, a_size0, k, a_stride0, a_stride1, hi, lo, a_shift, kp, team_max);
  else
    split_a_rows<256, 0>(a, a_size0, k, a_stride0, a_stride1, hi, lo, a_shift, kp, team_max);
}

// Largest |b| of every column of B (k x n, any strides) into b_amax, which
// gemm_split_a cleared. grid.x walks 1024-column chunks, grid.y 64-row slices.
extern "C" __global__ void __launch_bounds__(256)
gemm_colmax_b(KH_MEMREF2(const float, b), uint32_t *__restrict__ b_amax) {
  const float *__restrict__ b = KH_DATA(b);
  const int64_t k = b_size0, n = b_size1;
  const bool vec_ok = khd::is_aligned16(b) && b_stride1 == 1 && (b_stride0 & 3) == 0;
  const int64_t chunks_n = (n + 1023) >> 10, slices_k = (k + 63) >> 6;
  for (int64_t t = blockIdx.x; t < chunks_n * slices_k; t += gridDim.x) {
    const int64_t slice = t / chunks_n, chunk = t - slice * chunks_n;
    const int64_t col = (chunk << 10) + threadIdx.x * 4;
    const int64_t r0 = slice << 6, r1 = (r0 + 64 < k) ? r0 + 64 : k;
    if (col >= n) continue;
    float mx[4] = {0.f, 0.f, 0.f, 0.f};
    if (vec_ok && col + 4 <= n) {
#pragma unroll 8
      for (int64_t r = r0; r < r1; ++r) {
        const float4 f = __ldg(reinterpret_cast<const float4 *>(b + r * b_stride0 + col));
        mx[0] = fmaxf(mx[0], fabsf(f.x)); mx[1] = fmaxf(mx[1], fabsf(f.y));
        mx[2] = fmaxf(mx[2], fabsf(f.z)); mx[3] = fmaxf(mx[3], fabsf(f.w));
      }
    } else {
      for (int64_t r = r0; r < r1; ++r)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (col + j < n) mx[j] = fmaxf(mx[j], fabsf(b[r * b_stride0 + (col + j) * b_stride1]));
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (col + j < n && mx[j] > 0.f) atomicMax(b_amax + col + j, __float_as_uint(mx[j]));
  }
}

// B (k x n, any strides) -> B^T hi, lo (n x kp fp16, contiguous, zero padded in
// k), every column scaled by the exponent its maximum gives; the k-tile-0
// blocks also publish the exponents. 64 (k) x 128 (n) tiles through shared
// memory: a warp reads 512 contiguous bytes of a row of B, and writes 128-byte
// runs (64 k-values) of four rows of B^T at a time, 16 bytes per lane.
extern "C" __global__ void __launch_bounds__(256)
gemm_split_bt(KH_MEMREF2(const float, b), __half *__restrict__ hi, __half *__restrict__ lo,
              const uint32_t *__restrict__ b_amax, int *__restrict__ b_shift, int64_t kp) {
  constexpr int kTK = 64, kTN = 128;
  // float4 groups of a row are stored at group ^ (row / 8 mod 8): conflict-free both ways
  __shared__ __align__(16) float tile[kTK][kTN];
  const float *__restrict__ b = KH_DATA(b);
  const int64_t k = b_size0, n = b_size1;
  const int64_t tiles_n = (n + kTN - 1) / kTN, tiles_k = (kp + kTK - 1) / kTK;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool vec_ok = khd::is_aligned16(b) && b_stride1 == 1 && (b_stride0 & 3) == 0;
  for (int64_t t = blockIdx.x; t < tiles_n * tiles_k; t += gridDim.x) {
    // k-tiles of one column strip are neighbours in time: their 128-byte writes fill whole rows of B^T
    const int64_t tn = t / tiles_k, tk = t - tn * tiles_k;
    const int64_t k0 = tk * kTK, n0 = tn * kTN;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kTK / 8; ++j) {
      const int kl = warp + 8 * j;
      const int64_t kk = k0 + kl, nn = n0 + lane * 4;
      float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
      if (kk < k) {
        if (vec_ok && nn + 4 <= n) {
          f = __ldcs(reinterpret_cast<const float4 *>(b + kk * b_stride0 + nn));
        } else {
          if (nn < n) f.x = b[kk * b_stride0 + nn * b_stride1];
          if (nn + 1 < n) f.y = b[kk * b_stride0 + (nn + 1) * b_stride1];
          if (nn + 2 < n) f.z = b[kk * b_stride0 + (nn + 2) * b_stride1];
          if (nn + 3 < n) f.w = b[kk * b_stride0 + (nn + 3) * b_stride1];
        }
      }
      *reinterpret_cast<float4 *>(&tile[kl][(lane ^ ((kl >> 3) & 7)) * 4]) = f;
    }
    __syncthreads();
    const int sub = lane >> 3, kgroup = lane & 7; // 4 rows of B^T per warp store, 8 k-values per lane
#pragma unroll
    for (int j = 0; j < kTN / 32; ++j) {
      const int nl = warp * 16 + j * 4 + sub;
      const int64_t nn = n0 + nl, kk = k0 + kgroup * 8;
      if (nn < n && kk < kp) {
        const int shift = scale_shift(__uint_as_float(__ldg(b_amax + nn)));
        const RowScale scale = row_scale(shift);
        if (tk == 0 && kgroup == 0) b_shift[nn] = shift;
        const int col = (((nl >> 2) ^ kgroup) << 2) | (nl & 3); // rows kgroup*8.. share one swizzle
        Half8 h, l;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          split_fp16x2(tile[kgroup * 8 + 2 * q][col], tile[kgroup * 8 + 2 * q + 1][col], scale, h.v[q], l.v[q]);
        }
        *reinterpret_cast<Half8 *>(hi + nn * kp + kk) = h;
        *reinterpret_cast<Half8 *>(lo + nn * kp + kk) = l;
      }
    }
  }
}

namespace {

// Destinations of the fused all-gather: every finished C tile goes to each
// replica of the full matrix, `row_offset` rows down. The tile is stored to
// base[self], this GPU's own replica, and then copied out in 512-byte warp-wide
// slices: with multimem.st through `multicast`, the replicas' NVLink multicast
// address, when there is one (the switch delivers each store to every GPU, so
// the tile crosses this GPU's links once), else with plain peer stores to the
// other listed replicas.
struct GatherTargets {
  float *base[8];
  int count;
  int self;
  int64_t row_offset;
  float *multicast; // NVLink multicast address of the replicas (one store reaches all), or null
  // Arrival flags (epoch != 0): the barrier that has to follow the all-gather, done by the kernel
  // itself. flags[d] is rank d's array of eight 64-bit words as mapped on this GPU. The last CTA of
  // this launch to finish writes `epoch` into word `self` of every other rank's array (after a
  // system-wide fence, so that every tile this GPU sent is visible before the flag) and then waits,
  // for at most two seconds, until its own array holds at least `epoch` in every other rank's word:
  // when the kernel has completed, every rank's rows are in this GPU's replica. Epochs only grow.
  unsigned long long *flags[8];
  unsigned long long epoch;
  unsigned int *finished; // this GPU's count of CTAs that are done; 0 between launches
  int wait_later;         // the kernel only signals; `await_arrivals` does the waiting
};

// The wait half of the arrival barrier: until this GPU's flag array holds at least `epoch` in every
// other rank's word, for at most two seconds (then: status code, the missing rank as detail, return).
__device__ __forceinline__ void await_peers(const GatherTargets &t, uint32_t *status) {
  unsigned long long start;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(start));
  for (int d = 0; d < t.count; ++d) {
    if (d == t.self) continue;
    for (;;) {
      unsigned long long seen, now;
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(t.flags[t.self] + d) : "memory");
      if (seen >= t.epoch) break;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (now - start > 2000000000ull) { // two seconds: give up, say who was missing, return
        khd::report_status(status, khd::kStatusPeerArrivalTimeout, static_cast<uint32_t>(d));
        return;
      }
      __nanosleep(100);
    }
  }
}

// Runs once per CTA, by one thread, after the CTA's last store. The last CTA of the launch signals
// every peer and, unless the wait was handed to a later `await_arrivals` launch (`wait_later`: the
// host runs that one beside the next step's operand preparation), waits for the peers itself.
__device__ __forceinline__ void signal_and_await_peers(const GatherTargets &t, uint32_t *status) {
  __threadfence_system(); // this CTA's stores (peer stores and multimem.st included) before the count
  if (atomicAdd(t.finished, 1u) != gridDim.x - 1) return;
  *t.finished = 0; // the next launch on this stream starts from zero again
  __threadfence_system(); // every CTA's stores before the flags
  for (int d = 0; d < t.count; ++d)
    if (d != t.self)
      asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(t.flags[d] + t.self), "l"(t.epoch) : "memory");
  if (!t.wait_later) await_peers(t, status);
}

struct TileCoord {
  int m0, n0;
};

template <int BN>
__device__ __forceinline__ TileCoord tile_coord(int64_t tile, int64_t tiles_m, int64_t tiles_n, int64_t group_m) {
  const int64_t per_group = group_m * tiles_n;
  const int64_t group = tile / per_group;
  const int64_t first_m = group * group_m;
  const int64_t rows_in_group = (tiles_m - first_m < group_m) ? (tiles_m - first_m) : group_m;
  const int64_t in_group = tile - group * per_group;
  const int64_t tile_m = first_m + in_group % rows_in_group;
  const int64_t tile_n = in_group / rows_in_group;
  return {static_cast<int>(tile_m * 2 * kBM), static_cast<int>(tile_n * BN)};
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
// Address, in the cluster's shared window, of `local_addr` inside CTA `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(local_addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load whose completion bytes are counted on a barrier given by a
// cluster-window address (the leader's), data into this CTA's shared memory.
// No L2 eviction hint on purpose. Measured at 8192^3 (DRAM bytes read per launch, one ncu pass):
// no hint 2.32 GB, evict_last on A and B 2.30, evict_last on A with evict_normal on B 2.42,
// evict_normal on both 4.47, evict_first on B 4.59: any hint below evict_last loses the sharing of
// a panel between the clusters of one wave, and nothing keeps a group's A panels across waves.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const khd::TensorMap *map, int x, int y,
                                                 uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
               "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_dst),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result),
               "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
// D[tmem of both CTAs] (+)= A[smem of each CTA] * B[halves in both CTAs' smem]; one thread of the leader issues.
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
               "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
               : "memory");
}
// Arrive on the barrier at `cluster_addr` once every MMA of the pair issued so far has finished.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}

} // namespace

// The same two steps (column maxima, then B^T hi / lo) in ONE pass over B, for the common case of
// a contiguous, 16-byte aligned B whose column strips fit the shared memory of a cluster: a
// cluster of sixteen CTAs owns a strip of 32 columns (128 bytes of every row); CTA r of the
// cluster copies rows [r * R, (r + 1) * R) of the strip into its shared memory with tensor-map
// copies (128-byte swizzle; rows and columns past the end arrive as zeros), takes the column
// maxima of its rows, the CTAs exchange them through distributed shared memory, and every CTA
// then scales and splits its rows straight out of shared memory. B is read from HBM once
// (gemm_colmax_b + gemm_split_bt read it twice), and three CTAs fit an SM at k = 8192, so the
// copies of one overlap the arithmetic of the others. Results leave as 64 (k) x 32 (n) boxes of
// B^T hi and lo, which together are exactly as large as the 64 rows of the strip they come from
// and are built IN PLACE over them (256 rows at a time: read all, barrier, write the 16-byte
// pieces in the 128-byte swizzle, barrier, one tensor-map copy per box); nothing is reused, so
// no copy is ever waited for before the end.
// Parameters: B as a rank-2 descriptor, the tensor maps of B (box 32 columns x 64 rows) and
// of B^T hi / lo (box 64 k-values x 32 rows), the exponent array, rows per CTA (a multiple of
// 256), the status word. The cluster size is the launch's.
constexpr int kPrepCols = 32;
constexpr int kPrepBoxRows = 64;                                // rows of B per tensor-map copy
constexpr int kPrepBoxBytes = kPrepBoxRows * kPrepCols * 4;     // 8 KiB = a hi box + a lo box of B^T
constexpr int kPrepGroupRows = 256;                             // rows handled between two barriers
constexpr int kPrepGroupBoxes = kPrepGroupRows / kPrepBoxRows;
constexpr int kPrepMaxGroups = 6;                               // 6 x 32 KiB of rows fit an SM

extern "C" __global__ void __launch_bounds__(256, 3)
gemm_prep_b(KH_MEMREF2(const float, b), const __grid_constant__ khd::TensorMap tm_b,
            const __grid_constant__ khd::TensorMap tm_bt_hi, const __grid_constant__ khd::TensorMap tm_bt_lo,
            int *__restrict__ b_shift, int64_t rows_per_cta, uint32_t *status) {
  extern __shared__ uint8_t prep_raw[];
  __shared__ __align__(8) uint64_t landed[kPrepMaxGroups];
  __shared__ float warp_max[8][kPrepCols];
  __shared__ float cta_max[kPrepCols];     // read by the other CTAs of the cluster
  __shared__ int col_shift[kPrepCols];
  __shared__ int s_abort;
  (void)b_alloc; (void)b_ptr; (void)b_off; (void)b_stride0; (void)b_stride1;

  const int64_t k = b_size0, n = b_size1;
  const int64_t kp = ((k + 31) / 32) * 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t rank, cluster_ctas;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(cluster_ctas));
  const int64_t strip = blockIdx.x / cluster_ctas;
  const int n0 = static_cast<int>(strip * kPrepCols);
  const int64_t row0 = static_cast<int64_t>(rank) * rows_per_cta;
  const int groups = static_cast<int>(rows_per_cta / kPrepGroupRows);
  uint8_t *rows_smem = prep_raw + ((1024u - (khd::smem_u32(prep_raw) & 1023u)) & 1023u);
  const uint32_t rows_addr = khd::smem_u32(rows_smem);

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int g = 0; g < groups; ++g) khd::mbar_init(khd::smem_u32(&landed[g]), 1);
    khd::mbar_fence_init();
    for (int g = 0; g < groups; ++g) {
      // groups that start past the last row of B hold nothing but padding: no copy is started
      // for them (and none is waited for below; every copy that is started is also awaited)
      if (row0 + static_cast<int64_t>(g) * kPrepGroupRows >= k) break;
      const uint32_t bar = khd::smem_u32(&landed[g]);
      khd::mbar_arrive_expect_tx(bar, kPrepGroupBoxes * kPrepBoxBytes);
      for (int i = 0; i < kPrepGroupBoxes; ++i) {
        const int box = g * kPrepGroupBoxes + i;
        khd::tma_load_2d(rows_addr + box * kPrepBoxBytes, &tm_b, n0, static_cast<int>(row0 + box * kPrepBoxRows), bar);
      }
    }
  }
  __syncthreads();

  // Element (row r, column `lane`) of this CTA's rows: the copies store 16-byte group c / 4 of a
  // row at position (c / 4) ^ (r & 7). A warp reads one row across its lanes: no bank conflicts.
  const uint32_t lane_bytes = static_cast<uint32_t>(lane & 3) * 4;
  const auto element = [&](int r) -> float {
    const uint32_t off = static_cast<uint32_t>(r) * 128u +
                         ((static_cast<uint32_t>(lane >> 2) ^ (static_cast<uint32_t>(r) & 7u)) << 4) + lane_bytes;
    return *reinterpret_cast<const float *>(rows_smem + off);
  };

  // ---- largest magnitude per column: this CTA's rows, then the cluster's ----
  float mx = 0.f;
  bool ok = true;
  for (int g = 0; g < groups && ok; ++g) {
    if (row0 + static_cast<int64_t>(g) * kPrepGroupRows >= k) break; // only padding from here on
    ok = khd::mbar_wait(khd::smem_u32(&landed[g]), 0u, &s_abort, status, khd::kStatusTmaWaitTimeout, 0x50u + g);
    if (!ok) break;
#pragma unroll 8
    for (int q = 0; q < kPrepGroupRows / 8; ++q) mx = fmaxf(mx, fabsf(element(g * kPrepGroupRows + q * 8 + warp)));
  }
  warp_max[warp][lane] = mx;
  __syncthreads();
  if (threadIdx.x < kPrepCols) {
    float m = warp_max[0][threadIdx.x];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, warp_max[w][threadIdx.x]);
    cta_max[threadIdx.x] = m;
  }
  cluster_sync_all(); // every CTA's maxima are written (release / acquire across the cluster)
  if (threadIdx.x < kPrepCols) {
    // all the remote reads are issued before the first is used: one round trip through the
    // cluster's shared-memory network instead of one per CTA
    float v[16];
#pragma unroll
    for (uint32_t r = 0; r < 16; ++r) {
      v[r] = 0.f;
      if (r < cluster_ctas)
        asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v[r]) : "r"(map_to_cta(khd::smem_u32(&cta_max[threadIdx.x]), r)));
    }
    float m = 0.f;
#pragma unroll
    for (uint32_t r = 0; r < 16; ++r) m = fmaxf(m, v[r]);
    const int shift = scale_shift(m);
    col_shift[threadIdx.x] = shift;
    if (rank == 0 && n0 + static_cast<int>(threadIdx.x) < n) b_shift[n0 + threadIdx.x] = shift;
  }
  // "I have read every CTA's maxima": arrive now, wait only before leaving (a CTA's shared memory
  // must outlive the other CTAs' reads of it), so the split does not stand behind a second
  // cluster-wide round trip. The block barrier publishes col_shift.
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  __syncthreads();
  if (s_abort) { // a copy never landed (block-uniform after the barriers): reported in the status word
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
    return;
  }

  // ---- scale, split, transpose, in place: 256 rows (k-values) x 32 columns at a time ----
  // Thread (column `lane`, warp w) owns the 16-byte pieces w, w + 8, w + 16, w + 24 of its column:
  // k-values piece * 8 .. + 7 of the group, one piece of a hi box and of a lo box each.
  const RowScale scale = row_scale(col_shift[lane]);
  for (int g = 0; g < groups; ++g) {
    const int64_t k_group = row0 + static_cast<int64_t>(g) * kPrepGroupRows;
    if (k_group >= kp) break; // past the padded k: nothing to write (block-uniform)
    const bool real = k_group < k; // else the rows are all padding and no copy was started
    Half8 h[4], l[4];
#pragma unroll
    for (int part = 0; part < 4; ++part) {
      const int r = g * kPrepGroupRows + (warp + 8 * part) * 8;
      float2 x[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) x[q] = real ? make_float2(element(r + 2 * q), element(r + 2 * q + 1)) : make_float2(0.f, 0.f);
      split_fp16_pairs<4>(x, scale, h[part].v, l[part].v);
    }
    __syncthreads(); // every value of the group is in registers: its bytes may be overwritten
#pragma unroll
    for (int part = 0; part < 4; ++part) {
      const int piece = warp + 8 * part; // 0..31
      const int box = g * kPrepGroupBoxes + (piece >> 3);
      // row `lane` of the box (one column of B), 16-byte piece (piece & 7), stored at piece ^ (row & 7)
      const uint32_t at = static_cast<uint32_t>(box) * kPrepBoxBytes + static_cast<uint32_t>(lane) * 128u +
                          (((static_cast<uint32_t>(piece) & 7u) ^ (static_cast<uint32_t>(lane) & 7u)) << 4);
      *reinterpret_cast<Half8 *>(rows_smem + at) = h[part];
      *reinterpret_cast<Half8 *>(rows_smem + at + kPrepBoxBytes / 2) = l[part];
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // the copy engine reads these stores
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int i = 0; i < kPrepGroupBoxes; ++i) {
        const int box = g * kPrepGroupBoxes + i;
        const int64_t kx = row0 + static_cast<int64_t>(box) * kPrepBoxRows;
        if (kx >= kp) break;
        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                         reinterpret_cast<uint64_t>(&tm_bt_hi)),
                     "r"(static_cast<int>(kx)), "r"(n0), "r"(rows_addr + box * kPrepBoxBytes)
                     : "memory");
        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                         reinterpret_cast<uint64_t>(&tm_bt_lo)),
                     "r"(static_cast<int>(kx)), "r"(n0), "r"(rows_addr + box * kPrepBoxBytes + kPrepBoxBytes / 2)
                     : "memory");
      }
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
  }
  // the copies only have to be done READING this CTA's shared memory before it goes away
  if (threadIdx.x == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); // every CTA of the cluster has read this CTA's maxima
}

namespace {

struct PendingPush {
  int m0, n0;
  int next_unit; // 0 .. units per warp; the last value = done
};

// A unit is 512 contiguous bytes (128 columns of one row) sent by one warp instruction; an epilogue
// warp owns 16 rows of its CTA's 128 x BN part of the tile: 16 * BN / 128 units.
template <int BN>
__device__ __forceinline__ void push_units(const GatherTargets &t, PendingPush &p, int how_many, int ew,
                                           int lane, int64_t m, int64_t n) {
  constexpr int kPerRow = BN / 128, kUnits = 16 * kPerRow;
  const float *local = t.base[t.self];
  for (int i = 0; i < how_many && p.next_unit < kUnits; ++i, ++p.next_unit) {
    const int64_t row = static_cast<int64_t>(p.m0) + 16 * ew + (p.next_unit / kPerRow);
    const int64_t col = static_cast<int64_t>(p.n0) + (p.next_unit % kPerRow) * 128 + lane * 4;
    if (row >= m || col >= n) continue;
    const int64_t off = (t.row_offset + row) * n + col;
    if ((n & 3) == 0) {
      const float4 v = __ldcg(reinterpret_cast<const float4 *>(local + off));
      if (t.multicast != nullptr) {
        multicast_store_float4(t.multicast + off, v.x, v.y, v.z, v.w);
      } else {
        for (int d = 0; d < t.count; ++d)
          if (d != t.self) *reinterpret_cast<float4 *>(t.base[d] + off) = v;
      }
    } else {
      for (int j = 0; j < 4 && col + j < n; ++j) {
        const float v = __ldcg(local + off + j);
        if (t.multicast != nullptr) {
          multicast_store_float(t.multicast + off + j, v);
        } else {
          for (int d = 0; d < t.count; ++d)
            if (d != t.self) t.base[d][off + j] = v;
        }
      }
    }
  }
}

// BN: columns of C per cluster tile, 256 or 128 (the host takes 128 where that fills the last
// wave of tiles better; the stage layout keeps its 8 KiB slots, a B half-tile then fills half of its two).
template <bool kGather, int BN>
__device__ __forceinline__ void gemm_body(int64_t m, int64_t n, float *__restrict__ c, int64_t c_stride0,
                                               int64_t c_stride1, const khd::TensorMap &tm_a_hi,
                                               const khd::TensorMap &tm_a_lo, const khd::TensorMap &tm_b_hi,
                                               const khd::TensorMap &tm_b_lo, int64_t k_blocks,
                                               uint32_t *status, const int *__restrict__ a_shift,
                                               const int *__restrict__ b_shift, int64_t raster, uint64_t alpha_beta,
                                               float *__restrict__ partials, unsigned int *partial_flags, int64_t split_plan,
                                               const GatherTargets *targets) {
  extern __shared__ uint8_t smem_raw[];
  // C = alpha * A.B + beta * C_old; alpha in the low and beta in the high 32 bits (1 and 0: a plain store)
  const float alpha = __uint_as_float(static_cast<uint32_t>(alpha_beta));
  const float beta = __uint_as_float(static_cast<uint32_t>(alpha_beta >> 32));
  const bool scaled_store = !(alpha == 1.f && beta == 0.f);
  const int64_t group_m = raster > 0 ? raster : kGroupM; // tile rows per rasterisation group
  // full[kStages] (leader's are used), empty[kStages], acc_full[2], acc_empty[2] (leader's), tile_stored
  __shared__ __align__(8) uint64_t bars[2 * kStages + 5];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ int s_split_role;
  // named barrier 1: the eight epilogue warps of this CTA only
  const auto epilogue_barrier = [] { asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueWarps * 32) : "memory"); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank(); // 0 = leader
  const bool leader_cta = rank == 0;

  const uint32_t ring = (khd::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t full0 = khd::smem_u32(&bars[0]);
  const uint32_t empty0 = khd::smem_u32(&bars[kStages]);
  const uint32_t acc_full0 = khd::smem_u32(&bars[2 * kStages]);
  const uint32_t acc_empty0 = khd::smem_u32(&bars[2 * kStages + 2]);
  const uint32_t tile_stored = khd::smem_u32(&bars[2 * kStages + 4]);

  const int64_t tiles_m = (m + 2 * kBM - 1) / (2 * kBM), tiles_n = (n + BN - 1) / BN;
  const int64_t num_tiles = tiles_m * tiles_n;
  const int64_t first_tile = blockIdx.x >> 1, tile_step = gridDim.x >> 1;
  // Work units. A tile is normally one unit. Where the host asks for it (`split_plan`: tiles at the
  // head of the list in its low half, at the tail in its high half), a tile is done as TWO units, one
  // per half of K, by two neighbouring clusters at the same time; the unit that finishes first leaves
  // its 128 x BN partial sums in `partials`, the second adds them to its own and stores the tile
  // (epilogue below). At the tail that is the last, partly filled wave of clusters, which then takes
  // half as long; at the head (fused all-gather of a short shard only) it makes the first tiles, and
  // with them the traffic over NVLink that bounds such a launch, start after half a tile's time.
  const int64_t head_tiles = partials != nullptr ? (split_plan & 0xffffffff) : 0;
  const int64_t tail_tiles = partials != nullptr ? (split_plan >> 32) : 0;
  const int64_t whole_tiles = num_tiles - head_tiles - tail_tiles;
  const int64_t num_units = 2 * head_tiles + whole_tiles + 2 * tail_tiles;
  struct Unit {
    int64_t tile, kb0, kb1;
    int slot; // index of the shared tile among the split ones, or -1 for a whole tile
  };
  const auto unit_of = [&](int64_t u) -> Unit {
    const int64_t half_blocks = k_blocks / 2;
    if (u < 2 * head_tiles)
      return {u >> 1, (u & 1) ? half_blocks : 0, (u & 1) ? k_blocks : half_blocks, static_cast<int>(u >> 1)};
    if (u < 2 * head_tiles + whole_tiles) return {head_tiles + (u - 2 * head_tiles), 0, k_blocks, -1};
    const int64_t v = u - 2 * head_tiles - whole_tiles;
    return {head_tiles + whole_tiles + (v >> 1), (v & 1) ? half_blocks : 0, (v & 1) ? k_blocks : half_blocks,
            static_cast<int>(head_tiles + (v >> 1))};
  };
  // The SM clock this launch really ran at: block 0 counts its SM's cycles against the global
  // nanosecond timer over its whole life and leaves both in the status buffer (bytes 32..47),
  // where the host reads them beside the management library's figure.
  long long clock_start = 0;
  unsigned long long timer_start = 0;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    clock_start = clock64();
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(timer_start));
  }

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < kStages; ++s) {
      khd::mbar_init(full0 + 8 * s, 1);
      khd::mbar_init(empty0 + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      khd::mbar_init(acc_full0 + 8 * i, 1);
      khd::mbar_init(acc_empty0 + 8 * i, 2 * kEpilogueWarps); // the epilogue warps of both CTAs
    }
    khd::mbar_init(tile_stored, kEpilogueWarps * 32);
    khd::mbar_fence_init();
    khd::tma_prefetch_descriptor(&tm_a_hi);
    khd::tma_prefetch_descriptor(&tm_a_lo);
    khd::tma_prefetch_descriptor(&tm_b_hi);
    khd::tma_prefetch_descriptor(&tm_b_lo);
  }
  if (warp == 1) {
    tmem_alloc_pair(khd::smem_u32(&s_tmem_base), kTmemCols);
    tmem_relinquish_pair();
  }
  khd::tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all(); // both CTAs' barriers exist before anything remote touches them
  khd::tc_fence_after_sync();
  const uint32_t tmem_base = s_tmem_base;

  if (warp == 0) {
    // ---- TMA producer (both CTAs): own A rows, own half of B; bytes land on the
    //      leader's full barrier ---------------------------------------------------------
    if (lane == 0) {
      uint32_t g_kb = 0;
      bool ok = true;
      for (int64_t u = first_tile; u < num_units && ok; u += tile_step) {
        const Unit unit = unit_of(u);
        const TileCoord tc = tile_coord<BN>(unit.tile, tiles_m, tiles_n, group_m);
        const int a_row = tc.m0 + static_cast<int>(rank) * kBM;
        const int b_row = tc.n0 + static_cast<int>(rank) * (BN / 2);
        for (int64_t kb = unit.kb0; kb < unit.kb1; ++kb, ++g_kb) {
          const int s = static_cast<int>(g_kb % kStages);
          const uint32_t phase = (g_kb / kStages) & 1u;
          ok = khd::mbar_wait(empty0 + 8 * s, phase ^ 1u, &s_abort, status,
                              khd::kStatusEmptyWaitTimeout, g_kb);
          if (!ok) break;
          const uint32_t stage = ring + s * kStageBytes;
          if (leader_cta) khd::mbar_arrive_expect_tx(full0 + 8 * s, 2 * (2 * kTileBytes + 2 * (BN / 2) * kBK * 2));
          const uint32_t bar = map_to_cta(full0 + 8 * s, 0);
          const int kx = static_cast<int>(kb * kBK);
          tma_load_2d_pair(stage, &tm_a_hi, kx, a_row, bar);
          tma_load_2d_pair(stage + kTileBytes, &tm_a_lo, kx, a_row, bar);
          tma_load_2d_pair(stage + 2 * kTileBytes, &tm_b_hi, kx, b_row, bar);
          tma_load_2d_pair(stage + 3 * kTileBytes, &tm_b_lo, kx, b_row, bar);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the leader CTA only. One instruction drives both tensor cores. ----
    if (leader_cta) {
      const bool elected = khd::elect_one();
      constexpr uint32_t idesc = khd::umma_idesc_f16(2 * kBM, BN);
      uint32_t g_kb = 0, g_chunk = 0;
      bool ok = true;
      for (int64_t u = first_tile; u < num_units && ok; u += tile_step) {
        const Unit unit = unit_of(u);
        for (int64_t kb = unit.kb0; kb < unit.kb1 && ok; ++kb, ++g_kb) {
          const int in_chunk = static_cast<int>((kb - unit.kb0) % kChunkBlocks);
          const int buf = static_cast<int>(g_chunk & 1u);
          if (in_chunk == 0) {
            ok = khd::mbar_wait(acc_empty0 + 8 * buf, ((g_chunk >> 1) & 1u) ^ 1u, &s_abort, status,
                                khd::kStatusEpilogueWaitTimeout, g_chunk);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
          }
          const int s = static_cast<int>(g_kb % kStages);
          const uint32_t phase = (g_kb / kStages) & 1u;
          ok = khd::mbar_wait(full0 + 8 * s, phase, &s_abort, status, khd::kStatusTmaWaitTimeout, g_kb);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          khd::tc_fence_after_sync();
          const uint32_t d = tmem_base + static_cast<uint32_t>(buf * BN);
          const uint32_t stage = ring + s * kStageBytes;
          const uint64_t a_hi = khd::umma_desc_k64(stage);
          const uint64_t a_lo = a_hi + (kTileBytes >> 4);
          const uint64_t b_hi = a_hi + (2 * kTileBytes >> 4);
          const uint64_t b_lo = a_hi + (3 * kTileBytes >> 4);
          const bool chunk_end = in_chunk == kChunkBlocks - 1 || kb == unit.kb1 - 1;
          const uint32_t empty_here = map_to_cta(empty0 + 8 * s, 0), empty_peer = map_to_cta(empty0 + 8 * s, 1);
          const uint32_t accf_here = map_to_cta(acc_full0 + 8 * buf, 0), accf_peer = map_to_cta(acc_full0 + 8 * buf, 1);
          if (elected) {
#pragma unroll
            for (int kk = 0; kk < kBK / 16; ++kk) {
              const uint64_t adv = static_cast<uint64_t>(kk * 2); // 16 fp16 = 32 bytes, >> 4
              umma_f16_pair(d, a_lo + adv, b_hi + adv, idesc, (in_chunk | kk) != 0 ? 1u : 0u);
              umma_f16_pair(d, a_hi + adv, b_lo + adv, idesc, 1u);
              umma_f16_pair(d, a_hi + adv, b_hi + adv, idesc, 1u);
            }
            umma_commit_pair(empty_here); // the stage is free in both CTAs once these MMAs retire
            umma_commit_pair(empty_peer);
            if (chunk_end) {
              umma_commit_pair(accf_here); // both epilogues may drain their half of the chunk
              umma_commit_pair(accf_peer);
            }
          }
          __syncwarp();
          if (chunk_end) ++g_chunk;
        }
      }
    }
  } else {
    // ---- epilogue (both CTAs): this CTA's 128 rows of the pair's tile ------------------
    const int ew = warp - 2;
    const int quad = warp & 3;
    const int half = ew >> 2;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    uint32_t g_chunk = 0, stored_phase = 0;
    constexpr int kPushUnits = 16 * BN / 128; // per epilogue warp and tile
    PendingPush pending{0, 0, kPushUnits};
    bool ok = true;
    for (int64_t u = first_tile; u < num_units && ok; u += tile_step) {
      const Unit unit = unit_of(u);
      const TileCoord tc = tile_coord<BN>(unit.tile, tiles_m, tiles_n, group_m);
      const int m0 = tc.m0 + static_cast<int>(rank) * kBM;
      const int64_t unit_chunks = (unit.kb1 - unit.kb0 + kChunkBlocks - 1) / kChunkBlocks;
      float acc[BN / 2];
#pragma unroll
      for (int i = 0; i < BN / 2; ++i) acc[i] = 0.f;
      for (int64_t chunk = 0; chunk < unit_chunks && ok; ++chunk, ++g_chunk) {
        const int buf = static_cast<int>(g_chunk & 1u);
        ok = khd::mbar_wait(acc_full0 + 8 * buf, (g_chunk >> 1) & 1u, &s_abort, status,
                            khd::kStatusMmaWaitTimeout, g_chunk);
        if (!ok) break;
        khd::tc_fence_after_sync();
        const uint32_t src = tmem_base + lane_base + static_cast<uint32_t>(buf * BN + half * (BN / 2));
#pragma unroll
        for (int piece = 0; piece < BN / 2 / 32; ++piece) {
          uint32_t r[32];
          khd::tmem_ld_32x32(src + piece * 32, r);
          khd::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[piece * 32 + j] += __uint_as_float(r[j]);
        }
        khd::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(acc_empty0 + 8 * buf, 0));
        if (kGather) push_units<BN>(*targets, pending, 1, ew, lane, m, n);
      }
      if (!ok) break;
      if (kGather) push_units<BN>(*targets, pending, kPushUnits, ew, lane, m, n);

      if (unit.slot >= 0) {
        // Half of K: meet the other half. Per split tile and CTA of the pair: flags[0] counts the
        // arrivals, flags[1] says the first arrival's partial sums are in `partials`.
        unsigned int *flags = partial_flags + (static_cast<size_t>(unit.slot) * 2 + rank) * 2;
        // A thread's j-th four sums sit at [warp][j][lane]: the thread at the same place of the other
        // unit reads what this one wrote, so the layout is free, and this one makes a warp's accesses contiguous.
        float4 *mine = reinterpret_cast<float4 *>(partials + (static_cast<size_t>(unit.slot) * 2 + rank) * (kBM * BN)) +
                       static_cast<size_t>(ew) * (BN / 2 / 4) * 32 + lane;
        epilogue_barrier();
        if (ew == 0 && lane == 0) s_split_role = static_cast<int>(atomicAdd(flags, 1u));
        epilogue_barrier();
        if (s_split_role == 0) {
          // first: leave the partial sums
#pragma unroll
          for (int j = 0; j < BN / 2 / 4; ++j)
            mine[j * 32] = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
          __threadfence();
          epilogue_barrier();
          if (ew == 0 && lane == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flags + 1), "r"(1u) : "memory");
          continue; // the other unit stores the tile
        }
        // second: wait (bounded) for the first one's sums, take the flags back to zero, add
        if (ew == 0 && lane == 0) {
          unsigned long long start, now;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(start));
          for (;;) {
            unsigned int ready;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(ready) : "l"(flags + 1) : "memory");
            if (ready != 0u) break;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (now - start > 2000000000ull) {
              khd::report_status(status, khd::kStatusEpilogueWaitTimeout, 9100u + static_cast<uint32_t>(unit.slot));
              s_abort = 1;
              break;
            }
            __nanosleep(64);
          }
          flags[0] = 0u;
          flags[1] = 0u;
        }
        epilogue_barrier();
        if (s_abort) {
          ok = false;
          break;
        }
#pragma unroll
        for (int j = 0; j < BN / 2 / 4; ++j) {
          const float4 other = __ldcg(mine + j * 32);
          acc[4 * j] += other.x; acc[4 * j + 1] += other.y; acc[4 * j + 2] += other.z; acc[4 * j + 3] += other.w;
        }
      }

      const int64_t row = static_cast<int64_t>(m0) + quad * 32 + lane;
      const int64_t col0 = static_cast<int64_t>(tc.n0) + half * (BN / 2);
      float *crow;
      int64_t cs1;
      bool vec_ok;
      if (kGather) {
        crow = targets->base[targets->self] + (targets->row_offset + row) * n;
        cs1 = 1;
        vec_ok = (n & 3) == 0;
      } else {
        crow = c + row * c_stride0;
        cs1 = c_stride1;
        vec_ok = c_stride1 == 1 && (c_stride0 & 3) == 0 && khd::is_aligned16(c);
      }
      if (row < m) {
        // Undo the row and column scalings (exact: the factors are powers of two)
        // and store, four columns at a time. The loads and stores are ordered
        // (volatile asm) so that only one group of exponents is live at once.
        const int row_shift = __ldg(a_shift + row);
        if (vec_ok && col0 + BN / 2 <= n) {
#pragma unroll
          for (int j = 0; j < BN / 2 / 4; ++j) {
            const int4 sh = load_shift4(b_shift + col0 + 4 * j);
            float x = scale_pow2(acc[4 * j], -(row_shift + sh.x));
            float y = scale_pow2(acc[4 * j + 1], -(row_shift + sh.y));
            float z = scale_pow2(acc[4 * j + 2], -(row_shift + sh.z));
            float w = scale_pow2(acc[4 * j + 3], -(row_shift + sh.w));
            if (scaled_store) {
              x *= alpha; y *= alpha; z *= alpha; w *= alpha;
              if (beta != 0.f) { // beta = 0 never reads C (it may hold NaN)
                const float4 old = *reinterpret_cast<const float4 *>(crow + col0 + 4 * j);
                x = fmaf(beta, old.x, x); y = fmaf(beta, old.y, y); z = fmaf(beta, old.z, z); w = fmaf(beta, old.w, w);
              }
            }
            store_float4(crow + col0 + 4 * j, x, y, z, w);
          }
        } else {
#pragma unroll
          for (int j = 0; j < BN / 2; ++j)
            if (col0 + j < n) {
              float x = scale_pow2(acc[j], -(row_shift + load_shift(b_shift + col0 + j)));
              if (scaled_store) {
                x *= alpha;
                if (beta != 0.f) x = fmaf(beta, crow[(col0 + j) * cs1], x);
              }
              store_float(crow + (col0 + j) * cs1, x);
            }
        }
      }
      if (kGather) {
        __threadfence_block();
        khd::mbar_arrive(tile_stored);
        ok = khd::mbar_wait(tile_stored, stored_phase, &s_abort, status, khd::kStatusEpilogueWaitTimeout,
                            9000u);
        stored_phase ^= 1u;
        pending = PendingPush{m0, tc.n0, 0};
      }
    }
    if (kGather && ok) push_units<BN>(*targets, pending, kPushUnits, ew, lane, m, n);
  }

  __syncthreads();
  if (s_abort) {
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
  }
  khd::tc_fence_before_sync();
  cluster_sync_all(); // nothing remote may target a CTA that has already left
  if (warp == 1) {
    khd::tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if (kGather && threadIdx.x == 0 && targets->epoch != 0) signal_and_await_peers(*targets, status);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long timer_end;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(timer_end));
    unsigned long long *record = reinterpret_cast<unsigned long long *>(status) + 4;
    record[0] = static_cast<unsigned long long>(clock64() - clock_start);
    record[1] = timer_end - timer_start;
  }
}

} // namespace

extern "C" __global__ void __launch_bounds__(kThreads, 1)
gemm(KH_MEMREF2(const float, a), KH_MEMREF2(const float, b), KH_MEMREF2(float, c),
     const __grid_constant__ khd::TensorMap tm_a_hi, const __grid_constant__ khd::TensorMap tm_a_lo,
     const __grid_constant__ khd::TensorMap tm_b_hi, const __grid_constant__ khd::TensorMap tm_b_lo,
     int64_t k_blocks, uint32_t *status, const int *a_shift, const int *b_shift, int64_t raster, uint64_t alpha_beta,
     float *partials, unsigned int *partial_flags, int64_t split_plan) {
  (void)a_alloc; (void)a_ptr; (void)a_off; (void)a_size1; (void)a_stride0; (void)a_stride1;
  (void)b_alloc; (void)b_ptr; (void)b_off; (void)b_size0; (void)b_stride0; (void)b_stride1;
  (void)c_alloc; (void)c_size0; (void)c_size1;
  gemm_body<false, kBN>(a_size0, b_size1, KH_DATA(c), c_stride0, c_stride1, tm_a_hi, tm_a_lo, tm_b_hi, tm_b_lo,
                        k_blocks, status, a_shift, b_shift, raster, alpha_beta, partials, partial_flags, split_plan, nullptr);
}

// The same with 256 x 128 tiles (the tensor maps of B then have boxes of 64 rows): taken by the
// host when twice as many, half as wide tiles leave less of the last wave of clusters idle.
extern "C" __global__ void __launch_bounds__(kThreads, 1)
gemm_n128(KH_MEMREF2(const float, a), KH_MEMREF2(const float, b), KH_MEMREF2(float, c),
          const __grid_constant__ khd::TensorMap tm_a_hi, const __grid_constant__ khd::TensorMap tm_a_lo,
          const __grid_constant__ khd::TensorMap tm_b_hi, const __grid_constant__ khd::TensorMap tm_b_lo,
          int64_t k_blocks, uint32_t *status, const int *a_shift, const int *b_shift, int64_t raster, uint64_t alpha_beta,
     float *partials, unsigned int *partial_flags, int64_t split_plan) {
  (void)a_alloc; (void)a_ptr; (void)a_off; (void)a_size1; (void)a_stride0; (void)a_stride1;
  (void)b_alloc; (void)b_ptr; (void)b_off; (void)b_size0; (void)b_stride0; (void)b_stride1;
  (void)c_alloc; (void)c_size0; (void)c_size1;
  gemm_body<false, 128>(a_size0, b_size1, KH_DATA(c), c_stride0, c_stride1, tm_a_hi, tm_a_lo, tm_b_hi, tm_b_lo,
                        k_blocks, status, a_shift, b_shift, raster, alpha_beta, partials, partial_flags, split_plan, nullptr);
}

// The M-row-sharded product with the all-gather fused into the epilogue: `a`
// is this GPU's rows of A, the tensor maps cover its split, and every finished
// tile is stored into this GPU's replica of the full C and then copied, a
// 512-byte slice at a time between chunk drains of the next tile, to the other
// replicas over NVLink (plain peer stores; the caller's barrier after the
// kernel makes them visible to the peers).
extern "C" __global__ void __launch_bounds__(kThreads, 1)
gemm_allgather(KH_MEMREF2(const float, a), KH_MEMREF2(const float, b),
               const __grid_constant__ khd::TensorMap tm_a_hi, const __grid_constant__ khd::TensorMap tm_a_lo,
               const __grid_constant__ khd::TensorMap tm_b_hi, const __grid_constant__ khd::TensorMap tm_b_lo,
               int64_t k_blocks, uint32_t *status, const int *a_shift, const int *b_shift, int64_t raster,
               uint64_t alpha_beta, float *partials, unsigned int *partial_flags, int64_t split_plan,
               const __grid_constant__ GatherTargets targets) {
  (void)a_alloc; (void)a_ptr; (void)a_off; (void)a_size1; (void)a_stride0; (void)a_stride1;
  (void)b_alloc; (void)b_ptr; (void)b_off; (void)b_size0; (void)b_stride0; (void)b_stride1;
  gemm_body<true, kBN>(a_size0, b_size1, nullptr, 0, 0, tm_a_hi, tm_a_lo, tm_b_hi, tm_b_lo, k_blocks, status,
                       a_shift, b_shift, raster, alpha_beta, partials, partial_flags, split_plan, &targets);
}

// gemm_allgather with 256 x 128 tiles (see gemm_n128).
extern "C" __global__ void __launch_bounds__(kThreads, 1)
gemm_allgather_n128(KH_MEMREF2(const float, a), KH_MEMREF2(const float, b),
                    const __grid_constant__ khd::TensorMap tm_a_hi, const __grid_constant__ khd::TensorMap tm_a_lo,
                    const __grid_constant__ khd::TensorMap tm_b_hi, const __grid_constant__ khd::TensorMap tm_b_lo,
                    int64_t k_blocks, uint32_t *status, const int *a_shift, const int *b_shift, int64_t raster,
                    uint64_t alpha_beta, float *partials, unsigned int *partial_flags, int64_t split_plan,
                    const __grid_constant__ GatherTargets targets) {
  (void)a_alloc; (void)a_ptr; (void)a_off; (void)a_size1; (void)a_stride0; (void)a_stride1;
  (void)b_alloc; (void)b_ptr; (void)b_off; (void)b_size0; (void)b_stride0; (void)b_stride1;
  gemm_body<true, 128>(a_size0, b_size1, nullptr, 0, 0, tm_a_hi, tm_a_lo, tm_b_hi, tm_b_lo, k_blocks, status,
                       a_shift, b_shift, raster, alpha_beta, partials, partial_flags, split_plan, &targets);
}

// The wait half of the arrival barrier as a launch of its own (one thread): the host puts it on a
// second stream behind a `gemm_allgather` that only signalled, so that the wait for the other GPUs'
// tiles runs beside the next step's operand preparation; the next `gemm_allgather` is ordered behind it.
// It waits for kernels of OTHER GPUs only. Bounded like every wait here.
extern "C" __global__ void __launch_bounds__(32)
await_arrivals(const __grid_constant__ GatherTargets targets, uint32_t *status) {
  if (blockIdx.x == 0 && threadIdx.x == 0) await_peers(targets, status);
}

// Sends a run of floats of this GPU's copy of a replicated buffer to the same place in every
// other copy: `targets.base[self] + first` .. `+ first + count` goes out with multimem.st through
// the copies' NVLink multicast address when there is one (the switch delivers each store to
// every GPU), else with plain peer stores. Nothing is read from a peer. Used to assemble a
// replicated operand (B of the sharded product) from slices that each rank uploads itself.
// `first` and `count` are multiples of 4 and the bases 16-byte aligned (checked on the host).
extern "C" __global__ void __launch_bounds__(256)
replicate_run(const __grid_constant__ GatherTargets targets, int64_t first, int64_t count) {
  const float4 *__restrict__ src = reinterpret_cast<const float4 *>(targets.base[targets.self] + first);
  const int64_t vecs = count >> 2;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs; i += 4 * stride) {
    float4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (i + j * stride < vecs) v[j] = __ldcs(src + i + j * stride);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t at = i + j * stride;
      if (at >= vecs) continue;
      if (targets.multicast != nullptr) {
        multicast_store_float4(targets.multicast + first + 4 * at, v[j].x, v[j].y, v[j].z, v[j].w);
      } else {
        for (int d = 0; d < targets.count; ++d)
          if (d != targets.self)
            *reinterpret_cast<float4 *>(targets.base[d] + first + 4 * at) = v[j];
      }
    }
  }
}
