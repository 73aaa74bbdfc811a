// gemm_pair: the 3xTF32 GEMM of gemm.cu on CTA pairs (tcgen05 cta_group::2).
//
// Same arithmetic, operands and scratch as `gemm` (see gemm.cu: hi/lo split,
// three products per k-step, K = 256 chunks drained into fp32 registers). What
// changes is who loads what. Two CTAs on neighbouring SMs form a cluster and
// own one 256 x 256 tile of C: CTA r holds rows 128r..128r+127 of the A tile
// and of the accumulator, and only HALF of the B tile (128 of its 256 columns);
// one tcgen05.mma.cta_group::2 instruction (M 256, N 256, K 8), issued by the
// leader CTA, makes both tensor cores run and lets each read the other's half
// of B. Per k-block a CTA therefore pulls 32 KiB from L2 instead of 48 KiB for
// the same tensor work, which is what the single-CTA kernel is limited by
// (it sustains ~12.5 TB/s of L2-to-SM traffic with its tensor pipe 70 % busy).
//
// Synchronisation across the pair (no multicast qualifier is used anywhere):
//  * TMA loads of both CTAs complete on the LEADER's "full" barrier (the peer
//    addresses it through the cluster window), which expects both halves.
//  * the leader's tcgen05.commit arrives on the "empty" and "accumulator full"
//    barriers of BOTH CTAs (one commit per CTA, peer address from mapa).
//  * the epilogue warps of both CTAs arrive on the leader's "accumulator empty"
//    barrier (the peer's arrivals are remote).
// Every wait is bounded like in gemm.cu; the two cluster-wide barriers at the
// start and the end are hardware barriers that every thread reaches.
#include "kh_tcgen05.cuh"

namespace {

constexpr int kBM = 128;  // rows per CTA (256 per pair)
constexpr int kBN = 256;  // columns per pair
constexpr int kBNHalf = 128;
constexpr int kBK = 16;   // fp32 per k-block: one 64-byte swizzle row
constexpr int kStages = 6;
constexpr int kTileBytes = kBM * kBK * 4;          // 8 KiB: A_hi, A_lo, B_hi half, B_lo half
constexpr int kStageBytes = 4 * kTileBytes;        // 32 KiB per CTA
constexpr int kTmemCols = 512;
constexpr int kChunkBlocks = 16;                   // K = 256 per accumulator chunk
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr int kGroupM = 8;                         // pair tiles (256 rows) per rasterisation group

struct GatherTargets {
  float *base[8];
  int count;
  int self;
  int64_t row_offset;
};

struct TileCoord {
  int m0, n0;
};

__device__ __forceinline__ TileCoord tile_coord(int64_t tile, int64_t tiles_m, int64_t tiles_n) {
  const int64_t per_group = kGroupM * tiles_n;
  const int64_t group = tile / per_group;
  const int64_t first_m = group * kGroupM;
  const int64_t rows_in_group = (tiles_m - first_m < kGroupM) ? (tiles_m - first_m) : kGroupM;
  const int64_t in_group = tile - group * per_group;
  const int64_t tile_m = first_m + in_group % rows_in_group;
  const int64_t tile_n = in_group / rows_in_group;
  return {static_cast<int>(tile_m * 2 * kBM), static_cast<int>(tile_n * kBN)};
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
__device__ __forceinline__ void umma_tf32_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
               "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
               : "memory");
}
// Arrive on the barrier at `cluster_addr` once every MMA of the pair issued so far has finished.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}

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

template <bool kGather>
__device__ __forceinline__ void gemm_pair_body(int64_t m, int64_t n, float *__restrict__ c, int64_t c_stride0,
                                               int64_t c_stride1, const khd::TensorMap &tm_a_hi,
                                               const khd::TensorMap &tm_a_lo, const khd::TensorMap &tm_b_hi,
                                               const khd::TensorMap &tm_b_lo, int64_t k_blocks,
                                               uint32_t *status, const GatherTargets *targets) {
  extern __shared__ uint8_t smem_raw[];
  // full[kStages] (leader's are used), empty[kStages], acc_full[2], acc_empty[2] (leader's), tile_stored
  __shared__ __align__(8) uint64_t bars[2 * kStages + 5];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank(); // 0 = leader
  const bool leader_cta = rank == 0;

  const uint32_t ring = (khd::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t full0 = khd::smem_u32(&bars[0]);
  const uint32_t empty0 = khd::smem_u32(&bars[kStages]);
  const uint32_t acc_full0 = khd::smem_u32(&bars[2 * kStages]);
  const uint32_t acc_empty0 = khd::smem_u32(&bars[2 * kStages + 2]);
  const uint32_t tile_stored = khd::smem_u32(&bars[2 * kStages + 4]);

  const int64_t tiles_m = (m + 2 * kBM - 1) / (2 * kBM), tiles_n = (n + kBN - 1) / kBN;
  const int64_t num_tiles = tiles_m * tiles_n;
  const int64_t num_chunks = (k_blocks + kChunkBlocks - 1) / kChunkBlocks;
  const int64_t first_tile = blockIdx.x >> 1, tile_step = gridDim.x >> 1;

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
      for (int64_t tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
        const TileCoord tc = tile_coord(tile, tiles_m, tiles_n);
        const int a_row = tc.m0 + static_cast<int>(rank) * kBM;
        const int b_row = tc.n0 + static_cast<int>(rank) * kBNHalf;
        for (int64_t kb = 0; kb < k_blocks; ++kb, ++g_kb) {
          const int s = static_cast<int>(g_kb % kStages);
          const uint32_t phase = (g_kb / kStages) & 1u;
          ok = khd::mbar_wait(empty0 + 8 * s, phase ^ 1u, &s_abort, status,
                              khd::kStatusEmptyWaitTimeout, g_kb);
          if (!ok) break;
          const uint32_t stage = ring + s * kStageBytes;
          if (leader_cta) khd::mbar_arrive_expect_tx(full0 + 8 * s, 2 * kStageBytes);
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
      constexpr uint32_t idesc = khd::umma_idesc_tf32(2 * kBM, kBN);
      uint32_t g_kb = 0, g_chunk = 0;
      bool ok = true;
      for (int64_t tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
        for (int64_t kb = 0; kb < k_blocks && ok; ++kb, ++g_kb) {
          const int in_chunk = static_cast<int>(kb % kChunkBlocks);
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
          const uint32_t d = tmem_base + static_cast<uint32_t>(buf * kBN);
          const uint32_t stage = ring + s * kStageBytes;
          const uint64_t a_hi = khd::umma_desc_k64(stage);
          const uint64_t a_lo = a_hi + (kTileBytes >> 4);
          const uint64_t b_hi = a_hi + (2 * kTileBytes >> 4);
          const uint64_t b_lo = a_hi + (3 * kTileBytes >> 4);
          const bool chunk_end = in_chunk == kChunkBlocks - 1 || kb == k_blocks - 1;
          const uint32_t empty_here = map_to_cta(empty0 + 8 * s, 0), empty_peer = map_to_cta(empty0 + 8 * s, 1);
          const uint32_t accf_here = map_to_cta(acc_full0 + 8 * buf, 0), accf_peer = map_to_cta(acc_full0 + 8 * buf, 1);
          if (elected) {
#pragma unroll
            for (int kk = 0; kk < kBK / 8; ++kk) {
              const uint64_t adv = static_cast<uint64_t>(kk * 2); // 32 bytes >> 4
              umma_tf32_pair(d, a_lo + adv, b_hi + adv, idesc, (in_chunk | kk) != 0 ? 1u : 0u);
              umma_tf32_pair(d, a_hi + adv, b_lo + adv, idesc, 1u);
              umma_tf32_pair(d, a_hi + adv, b_hi + adv, idesc, 1u);
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
    PendingPush pending{0, 0, 32};
    bool ok = true;
    for (int64_t tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
      const TileCoord tc = tile_coord(tile, tiles_m, tiles_n);
      const int m0 = tc.m0 + static_cast<int>(rank) * kBM;
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
        if (lane == 0) mbar_arrive_cluster(map_to_cta(acc_empty0 + 8 * buf, 0));
        if (kGather) push_units(*targets, pending, 1, ew, lane, m, n);
      }
      if (!ok) break;
      if (kGather) push_units(*targets, pending, 32, ew, lane, m, n);

      const int64_t row = static_cast<int64_t>(m0) + quad * 32 + lane;
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
        __threadfence_block();
        khd::mbar_arrive(tile_stored);
        ok = khd::mbar_wait(tile_stored, stored_phase, &s_abort, status, khd::kStatusEpilogueWaitTimeout,
                            9000u);
        stored_phase ^= 1u;
        pending = PendingPush{m0, tc.n0, 0};
      }
    }
    if (kGather && ok) push_units(*targets, pending, 32, ew, lane, m, n);
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
}

} // namespace

extern "C" __global__ void __launch_bounds__(kThreads, 1)
gemm_pair(KH_MEMREF2(const float, a), KH_MEMREF2(const float, b), KH_MEMREF2(float, c),
          const __grid_constant__ khd::TensorMap tm_a_hi, const __grid_constant__ khd::TensorMap tm_a_lo,
          const __grid_constant__ khd::TensorMap tm_b_hi, const __grid_constant__ khd::TensorMap tm_b_lo,
          int64_t k_blocks, uint32_t *status) {
  (void)a_alloc; (void)a_ptr; (void)a_off; (void)a_size1; (void)a_stride0; (void)a_stride1;
  (void)b_alloc; (void)b_ptr; (void)b_off; (void)b_size0; (void)b_stride0; (void)b_stride1;
  (void)c_alloc; (void)c_size0; (void)c_size1;
  gemm_pair_body<false>(a_size0, b_size1, KH_DATA(c), c_stride0, c_stride1, tm_a_hi, tm_a_lo, tm_b_hi,
                        tm_b_lo, k_blocks, status, nullptr);
}

// The M-row-sharded product with the all-gather fused into the epilogue (see
// gemm_allgather in gemm.cu), on CTA pairs.
extern "C" __global__ void __launch_bounds__(kThreads, 1)
gemm_pair_allgather(KH_MEMREF2(const float, a), KH_MEMREF2(const float, b),
                    const __grid_constant__ khd::TensorMap tm_a_hi,
                    const __grid_constant__ khd::TensorMap tm_a_lo,
                    const __grid_constant__ khd::TensorMap tm_b_hi,
                    const __grid_constant__ khd::TensorMap tm_b_lo, int64_t k_blocks, uint32_t *status,
                    const __grid_constant__ GatherTargets targets) {
  (void)a_alloc; (void)a_ptr; (void)a_off; (void)a_size1; (void)a_stride0; (void)a_stride1;
  (void)b_alloc; (void)b_ptr; (void)b_off; (void)b_size0; (void)b_stride0; (void)b_stride1;
  gemm_pair_body<true>(a_size0, b_size1, nullptr, 0, 0, tm_a_hi, tm_a_lo, tm_b_hi, tm_b_lo, k_blocks,
                       status, &targets);
}
