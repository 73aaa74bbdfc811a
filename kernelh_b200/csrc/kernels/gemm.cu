// gemm: C = A . B, row-major fp32, A is m x k, B is k x n, C is m x n, zero
// seeded accumulator and a plain store (no alpha/beta).
//
// Replaces the kernel the reference generates from
// lib/dsl/kernels/gemm.cpp:116-296 (32x32x32 tiles of scalar fp32 FMAs, one
// k-tile staged in 8 KiB of static shared memory). Entry symbol `gemm`; the
// first 21 parameters are the reference's: (A, B, C) as rank-2 memref
// descriptors. The TMA-fed kernel then takes four tensor maps, the k-block
// count and a status pointer.
//
// Arithmetic: 3xTF32. Each operand is split once into hi = tf32(x) (round to
// nearest, low 13 mantissa bits cleared) and lo = x - hi (exact in fp32), and
// every k-step issues three tensor-core products into one fp32 accumulator in
// tensor memory: lo.hi, hi.lo, hi.hi (lo.lo, ~2^-22 relative, is dropped).
// The tensor core's fp32 accumulation truncates, which biases long sums (the
// error grew linearly with k when a whole k = 8192 product stayed in tensor
// memory), so only K = 256 is accumulated there at a time: two accumulators
// alternate, and each finished chunk is added into fp32 registers with
// round-to-nearest by the epilogue warps while the next chunk is running.
//
// Two launches:
//  gemm_split_a / gemm_split_bt  write A_hi, A_lo (m x kp) and B^T_hi, B^T_lo
//      (n x kp) into scratch, kp = k rounded up to 32 and zero padded, so both
//      tensor-core operands are K-major with 128-byte rows whatever k is.
//  gemm  persistent CTAs (one per SM) walk the 128 x 256 tiles of C. Warp 0 feeds a 4-stage ring of
//      {A_hi, A_lo, B_hi, B_lo} k-blocks (16 fp32 deep, 48 KiB per stage: three
//      loads in flight hide the L2 latency that a 2 x 96 KiB ring left exposed) with
//      TMA (64-byte swizzle, out-of-range rows read as zero, which is what
//      makes ragged m and n work); warp 1 issues tcgen05.mma (M128 N256 K8,
//      kind::tf32) and releases stages with tcgen05.commit; warps 2-9 drain the
//      256-column fp32 accumulators from tensor memory chunk by chunk and store C.
//
// Tensor-bound: 2 m n k useful flops; three MMAs per k-step put the ceiling
// at one third of the TF32 tensor rate.
#include "kh_tcgen05.cuh"

namespace {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 16; // fp32 elements per k-block: one 64-byte swizzle row
constexpr int kStages = 4;
constexpr int kATileBytes = kBM * kBK * 4;                         // 8 KiB
constexpr int kBTileBytes = kBN * kBK * 4;                         // 16 KiB
constexpr int kStageBytes = 2 * kATileBytes + 2 * kBTileBytes;     // 48 KiB
constexpr int kTmemCols = 512;      // two 256-column accumulators, used alternately
constexpr int kChunkBlocks = 16;    // k-blocks accumulated in tensor memory before a drain (K = 256)
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 64 + 32 * kEpilogueWarps; // TMA warp + MMA warp + epilogue warps
constexpr int kGroupM = 16; // m-tiles per rasterisation group (L2 reuse of B)

__device__ __forceinline__ float tf32_hi(float x) {
  // round to nearest (ties away) on the 13 dropped bits, in integer arithmetic
  uint32_t u = __float_as_uint(x);
  u = (u + 0x1000u) & 0xFFFFE000u;
  return __uint_as_float(u);
}

} // namespace

// A (m x k, any strides) -> hi, lo (m x kp, contiguous), zero padded in k.
extern "C" __global__ void __launch_bounds__(256)
gemm_split_a(KH_MEMREF2(const float, a), float *__restrict__ hi, float *__restrict__ lo, int64_t kp) {
  const float *__restrict__ a = KH_DATA(a);
  const int64_t m = a_size0, k = a_size1;
  const int64_t kp4 = kp >> 2;
  const int64_t total = m * kp4;
  const bool vec_ok = khd::is_aligned16(a) && a_stride1 == 1 && (a_stride0 & 3) == 0;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / kp4, c = (i - r * kp4) << 2;
    float v[4];
    if (vec_ok && c + 4 <= k) {
      const float4 f = __ldcs(reinterpret_cast<const float4 *>(a + r * a_stride0 + c));
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = (c + j < k) ? a[r * a_stride0 + (c + j) * a_stride1] : 0.f;
    }
    float4 h, l;
    h.x = tf32_hi(v[0]); h.y = tf32_hi(v[1]); h.z = tf32_hi(v[2]); h.w = tf32_hi(v[3]);
    l.x = v[0] - h.x; l.y = v[1] - h.y; l.z = v[2] - h.z; l.w = v[3] - h.w;
    *reinterpret_cast<float4 *>(hi + r * kp + c) = h;
    *reinterpret_cast<float4 *>(lo + r * kp + c) = l;
  }
}

// B (k x n, any strides) -> B^T hi, lo (n x kp, contiguous), zero padded in k.
// 32 x 32 tiles through shared memory so both sides stay coalesced.
extern "C" __global__ void __launch_bounds__(256)
gemm_split_bt(KH_MEMREF2(const float, b), float *__restrict__ hi, float *__restrict__ lo, int64_t kp) {
  __shared__ float tile[32][33];
  const float *__restrict__ b = KH_DATA(b);
  const int64_t k = b_size0, n = b_size1;
  const int64_t tiles_n = (n + 31) >> 5, tiles_k = kp >> 5;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5; // 32 x 8
  for (int64_t t = blockIdx.x; t < tiles_n * tiles_k; t += gridDim.x) {
    const int64_t tk = t / tiles_n, tn = t - tk * tiles_n;
    const int64_t k0 = tk << 5, n0 = tn << 5;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t kk = k0 + ty + 8 * j, nn = n0 + tx;
      tile[ty + 8 * j][tx] = (kk < k && nn < n) ? b[kk * b_stride0 + nn * b_stride1] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t nn = n0 + ty + 8 * j, kk = k0 + tx;
      if (nn < n) {
        const float v = tile[tx][ty + 8 * j];
        const float h = tf32_hi(v);
        hi[nn * kp + kk] = h;
        lo[nn * kp + kk] = v - h;
      }
    }
  }
}

namespace {

// Destinations of the fused all-gather: every finished C tile goes to each
// listed replica of the full matrix, `row_offset` rows down. base[self] is this
// GPU's own replica.
struct GatherTargets {
  float *base[8];
  int count;
  int self;
  int64_t row_offset;
};

struct TileCoord {
  int m0, n0;
};

// Tile order: groups of kGroupM m-tiles sweep n together, so the CTAs that run
// at the same time share B column panels and a few A row panels in L2.
__device__ __forceinline__ TileCoord tile_coord(int64_t tile, int64_t tiles_m, int64_t tiles_n) {
  const int64_t per_group = kGroupM * tiles_n;
  const int64_t group = tile / per_group;
  const int64_t first_m = group * kGroupM;
  const int64_t rows_in_group = (tiles_m - first_m < kGroupM) ? (tiles_m - first_m) : kGroupM;
  const int64_t in_group = tile - group * per_group;
  const int64_t tile_m = first_m + in_group % rows_in_group;
  const int64_t tile_n = in_group / rows_in_group;
  return {static_cast<int>(tile_m * kBM), static_cast<int>(tile_n * kBN)};
}

// A tile whose copy to the other replicas is still in progress. The eight
// epilogue warps push it in 32 "units" each (warp w owns rows 16w..16w+15 of
// the tile; a unit is half a row: 512 contiguous bytes, one float4 per lane).
struct PendingPush {
  int m0, n0;
  int next_unit; // 0..32; 32 = done
};

__device__ __forceinline__ void push_units(const GatherTargets &t, PendingPush &p, int how_many, int ew,
                                           int lane, int64_t m, int64_t n) {
  const float *local = t.base[t.self];
  for (int i = 0; i < how_many && p.next_unit < 32; ++i, ++p.next_unit) {
    const int64_t row = static_cast<int64_t>(p.m0) + 16 * ew + (p.next_unit >> 1);
    const int64_t col = static_cast<int64_t>(p.n0) + (p.next_unit & 1) * 128 + lane * 4;
    if (row >= m || col >= n) continue;
    const int64_t off = (t.row_offset + row) * n + col;
    if ((n & 3) == 0) {
      const float4 v = __ldcg(reinterpret_cast<const float4 *>(local + off));
      for (int d = 0; d < t.count; ++d)
        if (d != t.self) *reinterpret_cast<float4 *>(t.base[d] + off) = v;
    } else {
      for (int j = 0; j < 4 && col + j < n; ++j) {
        const float v = __ldcg(local + off + j);
        for (int d = 0; d < t.count; ++d)
          if (d != t.self) t.base[d][off + j] = v;
      }
    }
  }
}

// The kernel body: a persistent CTA (one per SM) walks tiles blockIdx.x,
// blockIdx.x + gridDim.x, ... The TMA and MMA warps run straight from one tile
// into the next; the epilogue warps drain K chunks into registers, store the
// finished tile, and (kGather) copy the previous tile to the other replicas a
// slice at a time between chunk drains, so neither the store nor the NVLink
// traffic ever stops the tensor cores.
// `m`, `n`: extents of the product this launch forms. C is written through
// (c, c_stride0, c_stride1) when kGather is false, and to the gather targets
// (contiguous rows of n floats) when it is true.
template <bool kGather>
__device__ __forceinline__ void gemm_body(int64_t m, int64_t n, float *__restrict__ c, int64_t c_stride0,
                                          int64_t c_stride1, const khd::TensorMap &tm_a_hi,
                                          const khd::TensorMap &tm_a_lo, const khd::TensorMap &tm_b_hi,
                                          const khd::TensorMap &tm_b_lo, int64_t k_blocks, uint32_t *status,
                                          const GatherTargets *targets) {
  extern __shared__ uint8_t smem_raw[];
  // full[kStages], empty[kStages], acc_full[2], acc_empty[2], tile_stored
  __shared__ __align__(8) uint64_t bars[2 * kStages + 5];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // 1024-byte aligned operand ring (the swizzle pattern is anchored there)
  const uint32_t ring = (khd::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t full0 = khd::smem_u32(&bars[0]);
  const uint32_t empty0 = khd::smem_u32(&bars[kStages]);
  const uint32_t acc_full0 = khd::smem_u32(&bars[2 * kStages]);
  const uint32_t acc_empty0 = khd::smem_u32(&bars[2 * kStages + 2]);
  const uint32_t tile_stored = khd::smem_u32(&bars[2 * kStages + 4]);

  const int64_t tiles_m = (m + kBM - 1) / kBM, tiles_n = (n + kBN - 1) / kBN;
  const int64_t num_tiles = tiles_m * tiles_n;
  const int64_t num_chunks = (k_blocks + kChunkBlocks - 1) / kChunkBlocks;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < kStages; ++s) {
      khd::mbar_init(full0 + 8 * s, 1);
      khd::mbar_init(empty0 + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      khd::mbar_init(acc_full0 + 8 * i, 1);
      khd::mbar_init(acc_empty0 + 8 * i, kEpilogueWarps); // one arrival per epilogue warp
    }
    khd::mbar_init(tile_stored, kEpilogueWarps * 32);
    khd::mbar_fence_init();
    khd::tma_prefetch_descriptor(&tm_a_hi);
    khd::tma_prefetch_descriptor(&tm_a_lo);
    khd::tma_prefetch_descriptor(&tm_b_hi);
    khd::tma_prefetch_descriptor(&tm_b_lo);
  }
  if (warp == 1) {
    khd::tmem_alloc(khd::smem_u32(&s_tmem_base), kTmemCols);
    khd::tmem_relinquish();
  }
  khd::tc_fence_before_sync();
  __syncthreads();
  khd::tc_fence_after_sync();
  const uint32_t tmem_base = s_tmem_base;

  if (warp == 0) {
    // ---- TMA producer: the stage ring runs on across tiles ----------------------
    if (lane == 0) {
      uint32_t g_kb = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const TileCoord tc = tile_coord(tile, tiles_m, tiles_n);
        for (int64_t kb = 0; kb < k_blocks; ++kb, ++g_kb) {
          const int s = static_cast<int>(g_kb % kStages);
          const uint32_t phase = (g_kb / kStages) & 1u;
          ok = khd::mbar_wait(empty0 + 8 * s, phase ^ 1u, &s_abort, status,
                              khd::kStatusEmptyWaitTimeout, g_kb);
          if (!ok) break;
          const uint32_t stage = ring + s * kStageBytes;
          const uint32_t bar = full0 + 8 * s;
          khd::mbar_arrive_expect_tx(bar, kStageBytes);
          const int kx = static_cast<int>(kb * kBK);
          khd::tma_load_2d(stage, &tm_a_hi, kx, tc.m0, bar);
          khd::tma_load_2d(stage + kATileBytes, &tm_a_lo, kx, tc.m0, bar);
          khd::tma_load_2d(stage + 2 * kATileBytes, &tm_b_hi, kx, tc.n0, bar);
          khd::tma_load_2d(stage + 2 * kATileBytes + kBTileBytes, &tm_b_lo, kx, tc.n0, bar);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: chunk buffers alternate across tiles too. The whole warp
    //      walks the loop (waits and descriptor arithmetic are warp-uniform and
    //      stay in uniform registers); only the tcgen05 instructions themselves
    //      sit under the elected lane. ---------------------------------------------------
    {
      const bool leader = khd::elect_one();
      constexpr uint32_t idesc = khd::umma_idesc_tf32(kBM, kBN);
      uint32_t g_kb = 0, g_chunk = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int64_t kb = 0; kb < k_blocks && ok; ++kb, ++g_kb) {
          const int in_chunk = static_cast<int>(kb % kChunkBlocks);
          const int buf = static_cast<int>(g_chunk & 1u);
          if (in_chunk == 0) {
            // the accumulator buffer must have been drained (two chunks ago)
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
          const uint32_t d = tmem_base + static_cast<uint32_t>(buf * kBN);
          const uint32_t stage = ring + s * kStageBytes;
          const uint64_t a_hi = khd::umma_desc_k64(stage);
          const uint64_t a_lo = a_hi + (kATileBytes >> 4);
          const uint64_t b_hi = a_hi + (2 * kATileBytes >> 4);
          const uint64_t b_lo = b_hi + (kBTileBytes >> 4);
          const bool chunk_end = in_chunk == kChunkBlocks - 1 || kb == k_blocks - 1;
          if (leader) {
#pragma unroll
            for (int kk = 0; kk < kBK / 8; ++kk) {
              const uint64_t adv = static_cast<uint64_t>(kk * 2); // 32 bytes >> 4
              khd::umma_tf32_ss(d, a_lo + adv, b_hi + adv, idesc, (in_chunk | kk) != 0 ? 1u : 0u);
              khd::umma_tf32_ss(d, a_hi + adv, b_lo + adv, idesc, 1u);
              khd::umma_tf32_ss(d, a_hi + adv, b_hi + adv, idesc, 1u);
            }
            khd::umma_commit(empty0 + 8 * s); // stage reusable once these MMAs retire
            if (chunk_end) khd::umma_commit(acc_full0 + 8 * buf); // chunk complete: hand it to the epilogue
          }
          __syncwarp();
          if (chunk_end) ++g_chunk;
        }
      }
    }
  } else {
    // ---- epilogue: drain every K chunk from tensor memory into fp32 registers
    //      (round-to-nearest adds), then store the tile. Two warps share each
    //      32-lane quarter of tensor memory and take 128 columns each. ------------------
    const int ew = warp - 2;
    const int quad = warp & 3;
    const int half = ew >> 2;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    uint32_t g_chunk = 0, stored_phase = 0;
    PendingPush pending{0, 0, 32};
    bool ok = true;
    for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const TileCoord tc = tile_coord(tile, tiles_m, tiles_n);
      float acc[kBN / 2];
#pragma unroll
      for (int i = 0; i < kBN / 2; ++i) acc[i] = 0.f;
      for (int64_t chunk = 0; chunk < num_chunks && ok; ++chunk, ++g_chunk) {
        const int buf = static_cast<int>(g_chunk & 1u);
        ok = khd::mbar_wait(acc_full0 + 8 * buf, (g_chunk >> 1) & 1u, &s_abort, status,
                            khd::kStatusMmaWaitTimeout, g_chunk);
        if (!ok) break;
        khd::tc_fence_after_sync();
        const uint32_t src = tmem_base + lane_base + static_cast<uint32_t>(buf * kBN + half * (kBN / 2));
#pragma unroll
        for (int piece = 0; piece < kBN / 2 / 32; ++piece) {
          uint32_t r[32];
          khd::tmem_ld_32x32(src + piece * 32, r);
          khd::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[piece * 32 + j] += __uint_as_float(r[j]);
        }
        khd::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) khd::mbar_arrive(acc_empty0 + 8 * buf);
        // a slice of the previous tile goes out to the other replicas meanwhile
        if (kGather) push_units(*targets, pending, 1, ew, lane, m, n);
      }
      if (!ok) break;
      if (kGather) push_units(*targets, pending, 32, ew, lane, m, n); // whatever is left of it

      const int64_t row = static_cast<int64_t>(tc.m0) + quad * 32 + lane;
      const int64_t col0 = static_cast<int64_t>(tc.n0) + half * (kBN / 2);
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
        if (vec_ok && col0 + kBN / 2 <= n) {
#pragma unroll
          for (int j = 0; j < kBN / 2 / 4; ++j)
            reinterpret_cast<float4 *>(crow + col0)[j] =
                make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < kBN / 2; ++j)
            if (col0 + j < n) crow[(col0 + j) * cs1] = acc[j];
        }
      }
      if (kGather) {
        // The tile is read back by other warps of this CTA when it is pushed: all
        // epilogue threads meet on an mbarrier (a bounded wait, unlike bar.sync).
        __threadfence_block();
        khd::mbar_arrive(tile_stored);
        ok = khd::mbar_wait(tile_stored, stored_phase, &s_abort, status, khd::kStatusEpilogueWaitTimeout,
                            9000u);
        stored_phase ^= 1u;
        pending = PendingPush{tc.m0, tc.n0, 0};
      }
    }
    if (kGather && ok) push_units(*targets, pending, 32, ew, lane, m, n);
  }

  __syncthreads();
  if (s_abort) {
    // A wait gave up: leave time for copies still in flight to land before the
    // shared memory and tensor memory are released.
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
  }
  if (warp == 1) {
    khd::tc_fence_after_sync();
    khd::tmem_dealloc(tmem_base, kTmemCols);
  }
}

} // namespace

extern "C" __global__ void __launch_bounds__(kThreads, 1)
gemm(KH_MEMREF2(const float, a), KH_MEMREF2(const float, b), KH_MEMREF2(float, c),
     const __grid_constant__ khd::TensorMap tm_a_hi, const __grid_constant__ khd::TensorMap tm_a_lo,
     const __grid_constant__ khd::TensorMap tm_b_hi, const __grid_constant__ khd::TensorMap tm_b_lo,
     int64_t k_blocks, uint32_t *status) {
  (void)a_alloc; (void)a_ptr; (void)a_off; (void)a_size1; (void)a_stride0; (void)a_stride1;
  (void)b_alloc; (void)b_ptr; (void)b_off; (void)b_size0; (void)b_stride0; (void)b_stride1;
  (void)c_alloc; (void)c_size0; (void)c_size1;
  gemm_body<false>(a_size0, b_size1, KH_DATA(c), c_stride0, c_stride1, tm_a_hi, tm_a_lo, tm_b_hi, tm_b_lo,
                   k_blocks, status, nullptr);
}

// gemm with the all-gather of the C row shards fused into its epilogue, for the
// M-row-sharded product on several GPUs of one box. A is this rank's row shard,
// B is whole; every finished C tile is stored into each rank's copy of the full
// C (`targets`, peer-mapped pointers; this rank's own copy is one of them) at
// this rank's row offset. No kernel ever loads from a peer; the stores are
// ordinary global stores, complete when the kernel completes, and the caller
// runs a barrier across ranks before anyone reads C. No counterpart in the
// reference, which is single-GPU.
extern "C" __global__ void __launch_bounds__(kThreads, 1)
gemm_allgather(KH_MEMREF2(const float, a), KH_MEMREF2(const float, b),
               const __grid_constant__ khd::TensorMap tm_a_hi,
               const __grid_constant__ khd::TensorMap tm_a_lo,
               const __grid_constant__ khd::TensorMap tm_b_hi,
               const __grid_constant__ khd::TensorMap tm_b_lo, int64_t k_blocks, uint32_t *status,
               const __grid_constant__ GatherTargets targets) {
  (void)a_alloc; (void)a_ptr; (void)a_off; (void)a_size1; (void)a_stride0; (void)a_stride1;
  (void)b_alloc; (void)b_ptr; (void)b_off; (void)b_size0; (void)b_stride0; (void)b_stride1;
  gemm_body<true>(a_size0, b_size1, nullptr, 0, 0, tm_a_hi, tm_a_lo, tm_b_hi, tm_b_lo, k_blocks, status,
                  &targets);
}
