// attention: O = softmax(Q K^T / sqrt(d)) V, non-causal, fp32, d = 64,
// tensors [batch, heads, seq, 64] contiguous, seq a multiple of 64.
//
// Replaces the kernel the reference generates from
// lib/dsl/kernels/attention.cpp:86-289 (one 64-thread block per query row,
// every block re-staging all of K and V in tiles of 64 with a per-key online
// rescale, 268-276; head_dim pinned to 64 and seq % 64 == 0, 109-120). Entry
// symbol `attention`; the first 44 parameters are the reference's: (Q, K, V,
// O) as rank-4 memref descriptors. The TMA-fed kernel then takes six tensor
// maps and a status pointer.
//
// Flash-style: a CTA owns 128 query rows of one (batch, head) and streams K/V
// in tiles of 64 keys. Both contractions run on tcgen05 tensor cores in 3xTF32
// (operands split once into hi = tf32(x), lo = x - hi; products lo.hi, hi.lo,
// hi.hi into one fp32 accumulator):
//   S = Q K^T   A = Q tile (shared memory, K-major), B = K tile (K-major)
//   PV = P V    A = P (tensor memory), B = V^T tile (K-major over keys)
// Scores, probabilities and the per-tile PV product live in tensor memory;
// the running max, sum and the 64-wide output row live in registers of the
// thread that owns the row (one thread per tensor-memory lane).
//
// Two launches:
//  attention_split  writes Q/8 (the 1/sqrt(64) scale is exact), K and V^T as
//      hi/lo pairs into scratch.
//  attention  warp 0 feeds TMA (Q once; separate 2-deep rings of K and V^T
//      tiles, 32 KiB each, so that K of tile j+2 can load as soon as S_j has
//      run); warp 1 issues the MMAs (S of tile j+1 is issued before PV of tile
//      j so the tensor core works while softmax runs); warps 2-5 and 6-9 are
//      two softmax groups (one thread per query row each) that take the even
//      and the odd tiles with their own running max, sum and output row and
//      are merged at the end, so two tiles are in the softmax stage at once.
//      Scores, P and PV are double buffered in tensor memory, one set per group.
//
// Tensor-bound: 4 b h s^2 d useful flops; 3xTF32 puts the ceiling at one third
// of the TF32 tensor rate.
#include "kh_tcgen05.cuh"

namespace {

constexpr int kHeadDim = 64;
constexpr int kBQ = 128;  // query rows per CTA
constexpr int kBKV = 64;  // keys per tile
constexpr int kStages = 2;
constexpr int kSoftmaxThreads = 256; // two groups of one thread per query row
constexpr int kThreads = 64 + kSoftmaxThreads;
constexpr int kChunkRowsBytes = 128; // one swizzle row: 32 fp32
constexpr int kQChunkBytes = kBQ * kChunkRowsBytes;   // 16 KiB: 128 rows x 32 fp32
constexpr int kKVChunkBytes = kBKV * kChunkRowsBytes; // 8 KiB: 64 rows x 32 fp32
constexpr int kQBytes = 4 * kQChunkBytes;             // hi c0,c1 + lo c0,c1 = 64 KiB
constexpr int kHalfStageBytes = 4 * kKVChunkBytes;    // one K (or V^T) tile: hi c0,c1 + lo c0,c1 = 32 KiB
// tensor-memory columns: two score buffers, two P buffers (64 hi + 64 lo columns
// each), two PV buffers
constexpr uint32_t kColS0 = 0, kColS1 = 64, kColP0 = 128, kColP1 = 256, kColPV0 = 384, kColPV1 = 448;
constexpr uint32_t kTmemCols = 512;

__device__ __forceinline__ float tf32_hi(float x) {
  uint32_t u = __float_as_uint(x);
  u = (u + 0x1000u) & 0xFFFFE000u;
  return __uint_as_float(u);
}

// 2^x by the special-function unit (2 ulp, flushes denormals): the arguments
// here are <= 0 and the results feed a sum of at least 1.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
               "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
               : "memory");
}

// 16-column variants (smaller register footprint for temporaries)
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                 "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
                 "=r"(r[14]), "=r"(r[15])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
               "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
               "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

} // namespace

// Q, K, V [bh, seq, 64] -> q_hi, q_lo (scaled by 1/8), k_hi, k_lo [bh*seq, 64]
// and vt_hi, vt_lo [bh*64, seq] (V transposed per (batch, head)).
extern "C" __global__ void __launch_bounds__(256)
attention_split(KH_MEMREF4(const float, q), KH_MEMREF4(const float, k), KH_MEMREF4(const float, v),
                float *__restrict__ q_hi, float *__restrict__ q_lo, float *__restrict__ k_hi,
                float *__restrict__ k_lo, float *__restrict__ vt_hi, float *__restrict__ vt_lo) {
  __shared__ float tile[32][33];
  const float *__restrict__ q = KH_DATA(q);
  const float *__restrict__ k = KH_DATA(k);
  const float *__restrict__ v = KH_DATA(v);
  const int64_t bh = q_size0 * q_size1, seq = q_size2;
  const int64_t total4 = bh * seq * kHeadDim / 4;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  // Q and K keep their layout (the tensors are contiguous, so a flat sweep does).
  for (int64_t i = tid; i < total4; i += nthreads) {
    const float4 fq = __ldcs(reinterpret_cast<const float4 *>(q) + i);
    const float4 fk = __ldcs(reinterpret_cast<const float4 *>(k) + i);
    float4 h, l;
    const float sq[4] = {fq.x * 0.125f, fq.y * 0.125f, fq.z * 0.125f, fq.w * 0.125f};
    h = make_float4(tf32_hi(sq[0]), tf32_hi(sq[1]), tf32_hi(sq[2]), tf32_hi(sq[3]));
    l = make_float4(sq[0] - h.x, sq[1] - h.y, sq[2] - h.z, sq[3] - h.w);
    reinterpret_cast<float4 *>(q_hi)[i] = h;
    reinterpret_cast<float4 *>(q_lo)[i] = l;
    h = make_float4(tf32_hi(fk.x), tf32_hi(fk.y), tf32_hi(fk.z), tf32_hi(fk.w));
    l = make_float4(fk.x - h.x, fk.y - h.y, fk.z - h.z, fk.w - h.w);
    reinterpret_cast<float4 *>(k_hi)[i] = h;
    reinterpret_cast<float4 *>(k_lo)[i] = l;
  }
  // V: 32 x 32 tiles through shared memory, [seq, 64] -> [64, seq] per (batch, head).
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t tiles_s = seq >> 5, tiles_per_bh = tiles_s * 2;
  for (int64_t t = blockIdx.x; t < bh * tiles_per_bh; t += gridDim.x) {
    const int64_t b = t / tiles_per_bh, r = t - b * tiles_per_bh;
    const int64_t s0 = (r >> 1) << 5, d0 = (r & 1) << 5;
    const float *src = v + b * seq * kHeadDim;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) tile[ty + 8 * j][tx] = src[(s0 + ty + 8 * j) * kHeadDim + d0 + tx];
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float val = tile[tx][ty + 8 * j];
      const float h = tf32_hi(val);
      const int64_t o = (b * kHeadDim + d0 + ty + 8 * j) * seq + s0 + tx;
      vt_hi[o] = h;
      vt_lo[o] = val - h;
    }
  }
}

extern "C" __global__ void __launch_bounds__(kThreads, 1)
attention(KH_MEMREF4(const float, q), KH_MEMREF4(const float, k), KH_MEMREF4(const float, v),
          KH_MEMREF4(float, o), const __grid_constant__ khd::TensorMap tm_q_hi,
          const __grid_constant__ khd::TensorMap tm_q_lo, const __grid_constant__ khd::TensorMap tm_k_hi,
          const __grid_constant__ khd::TensorMap tm_k_lo, const __grid_constant__ khd::TensorMap tm_vt_hi,
          const __grid_constant__ khd::TensorMap tm_vt_lo, uint32_t *status) {
  (void)q_alloc; (void)q_ptr; (void)q_off; (void)q_size3; (void)q_stride0; (void)q_stride1;
  (void)q_stride2; (void)q_stride3;
  (void)k_alloc; (void)k_ptr; (void)k_off; (void)k_size0; (void)k_size1; (void)k_size2; (void)k_size3;
  (void)k_stride0; (void)k_stride1; (void)k_stride2; (void)k_stride3;
  (void)v_alloc; (void)v_ptr; (void)v_off; (void)v_size0; (void)v_size1; (void)v_size2; (void)v_size3;
  (void)v_stride0; (void)v_stride1; (void)v_stride2; (void)v_stride3;
  (void)o_size0; (void)o_size1; (void)o_size2; (void)o_size3; (void)o_stride0; (void)o_stride1;
  (void)o_stride2; (void)o_stride3; (void)o_alloc;
  extern __shared__ uint8_t smem_raw[];
  // q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_ready[2], pv_full[2], exchange
  __shared__ __align__(8) uint64_t bars[16];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int64_t seq = q_size2;
  const int64_t q_tiles = (seq + kBQ - 1) / kBQ;
  const int64_t bh = blockIdx.x / q_tiles;
  const int q0 = static_cast<int>((blockIdx.x - bh * q_tiles) * kBQ);
  const int num_kv = static_cast<int>(seq / kBKV);
  float *__restrict__ out = KH_DATA(o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const uint32_t smem_q = (khd::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_k = smem_q + kQBytes;                 // 2 stages of K hi c0,c1 / lo c0,c1
  const uint32_t smem_v = smem_k + kStages * kHalfStageBytes; // 2 stages of V^T hi c0,c1 / lo c0,c1
  const uint32_t bar_q = khd::smem_u32(&bars[0]);
  const uint32_t bar_k_full = khd::smem_u32(&bars[1]);
  const uint32_t bar_k_empty = khd::smem_u32(&bars[3]);
  const uint32_t bar_v_full = khd::smem_u32(&bars[5]);
  const uint32_t bar_v_empty = khd::smem_u32(&bars[7]);
  const uint32_t bar_s_full = khd::smem_u32(&bars[9]);
  const uint32_t bar_p_ready = khd::smem_u32(&bars[11]);
  const uint32_t bar_pv_full = khd::smem_u32(&bars[13]);
  const uint32_t bar_exchange = khd::smem_u32(&bars[15]);

  if (threadIdx.x == 0) {
    s_abort = 0;
    khd::mbar_init(bar_q, 1);
    for (int s = 0; s < 2; ++s) {
      khd::mbar_init(bar_k_full + 8 * s, 1);
      khd::mbar_init(bar_k_empty + 8 * s, 1);
      khd::mbar_init(bar_v_full + 8 * s, 1);
      khd::mbar_init(bar_v_empty + 8 * s, 1);
      khd::mbar_init(bar_s_full + 8 * s, 1);
      khd::mbar_init(bar_p_ready + 8 * s, kBQ); // one arrival per thread of the group that owns the buffer
      khd::mbar_init(bar_pv_full + 8 * s, 1);
    }
    khd::mbar_init(bar_exchange, kSoftmaxThreads);
    khd::mbar_fence_init();
    khd::tma_prefetch_descriptor(&tm_q_hi);
    khd::tma_prefetch_descriptor(&tm_q_lo);
    khd::tma_prefetch_descriptor(&tm_k_hi);
    khd::tma_prefetch_descriptor(&tm_k_lo);
    khd::tma_prefetch_descriptor(&tm_vt_hi);
    khd::tma_prefetch_descriptor(&tm_vt_lo);
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
    // ---- TMA producer: K and V have their own 2-deep rings. A K slot is free as
    //      soon as S of its tile has run, long before the V slot of the same tile. ------
    if (lane == 0) {
      const int q_row = static_cast<int>(bh * seq) + q0;
      khd::mbar_arrive_expect_tx(bar_q, kQBytes);
      khd::tma_load_2d(smem_q + 0 * kQChunkBytes, &tm_q_hi, 0, q_row, bar_q);
      khd::tma_load_2d(smem_q + 1 * kQChunkBytes, &tm_q_hi, 32, q_row, bar_q);
      khd::tma_load_2d(smem_q + 2 * kQChunkBytes, &tm_q_lo, 0, q_row, bar_q);
      khd::tma_load_2d(smem_q + 3 * kQChunkBytes, &tm_q_lo, 32, q_row, bar_q);
      for (int j = 0; j < num_kv; ++j) {
        const int s = j & 1;
        const uint32_t phase = static_cast<uint32_t>((j >> 1) & 1);
        if (!khd::mbar_wait(bar_k_empty + 8 * s, phase ^ 1u, &s_abort, status,
                            khd::kStatusEmptyWaitTimeout, static_cast<uint32_t>(j)))
          break;
        {
          const uint32_t st = smem_k + s * kHalfStageBytes;
          const uint32_t bar = bar_k_full + 8 * s;
          khd::mbar_arrive_expect_tx(bar, kHalfStageBytes);
          const int k_row = static_cast<int>(bh * seq) + j * kBKV;
          khd::tma_load_2d(st + 0 * kKVChunkBytes, &tm_k_hi, 0, k_row, bar);
          khd::tma_load_2d(st + 1 * kKVChunkBytes, &tm_k_hi, 32, k_row, bar);
          khd::tma_load_2d(st + 2 * kKVChunkBytes, &tm_k_lo, 0, k_row, bar);
          khd::tma_load_2d(st + 3 * kKVChunkBytes, &tm_k_lo, 32, k_row, bar);
        }
        if (!khd::mbar_wait(bar_v_empty + 8 * s, phase ^ 1u, &s_abort, status,
                            khd::kStatusEmptyWaitTimeout, 1000u + static_cast<uint32_t>(j)))
          break;
        {
          const uint32_t st = smem_v + s * kHalfStageBytes;
          const uint32_t bar = bar_v_full + 8 * s;
          khd::mbar_arrive_expect_tx(bar, kHalfStageBytes);
          const int v_row = static_cast<int>(bh * kHeadDim);
          const int v_col = j * kBKV;
          khd::tma_load_2d(st + 0 * kKVChunkBytes, &tm_vt_hi, v_col, v_row, bar);
          khd::tma_load_2d(st + 1 * kKVChunkBytes, &tm_vt_hi, v_col + 32, v_row, bar);
          khd::tma_load_2d(st + 2 * kKVChunkBytes, &tm_vt_lo, v_col, v_row, bar);
          khd::tma_load_2d(st + 3 * kKVChunkBytes, &tm_vt_lo, v_col + 32, v_row, bar);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: S_0, then per tile j: S_{j+1} (other S buffer), PV_j. The
    //      whole warp walks the loop (waits, descriptor arithmetic: warp-uniform,
    //      so it stays in uniform registers); only the tcgen05 instructions
    //      themselves sit under the elected lane. ---------------------------------------
    {
      const bool leader = khd::elect_one();
      constexpr uint32_t idesc = khd::umma_idesc_tf32(kBQ, kBKV); // M128 N64 for both products
      // descriptor of chunk c (32 of the 64 k-columns) of a tile, stepped by kk inside it
      const uint64_t dq_hi = khd::umma_desc_k128(smem_q), dq_lo = khd::umma_desc_k128(smem_q + 2 * kQChunkBytes);
      constexpr uint64_t kQChunkStep = kQChunkBytes >> 4, kKVChunkStep = kKVChunkBytes >> 4;
      auto issue_s = [&](int b) {
        const uint64_t dk_hi = khd::umma_desc_k128(smem_k + b * kHalfStageBytes);
        const uint64_t dk_lo = dk_hi + 2 * kKVChunkStep;
        const uint32_t d = tmem_base + (b ? kColS1 : kColS0);
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 8; ++kk) {
            const uint64_t qoff = (kk >> 2) * kQChunkStep + (kk & 3) * 2;
            const uint64_t koff = (kk >> 2) * kKVChunkStep + (kk & 3) * 2;
            khd::umma_tf32_ss(d, dq_lo + qoff, dk_hi + koff, idesc, kk != 0 ? 1u : 0u);
            khd::umma_tf32_ss(d, dq_hi + qoff, dk_lo + koff, idesc, 1u);
            khd::umma_tf32_ss(d, dq_hi + qoff, dk_hi + koff, idesc, 1u);
          }
          khd::umma_commit(bar_s_full + 8 * b);  // scores ready for the softmax threads
          khd::umma_commit(bar_k_empty + 8 * b); // and this K slot may be refilled
        }
        __syncwarp();
      };
      bool ok = khd::mbar_wait(bar_q, 0u, &s_abort, status, khd::kStatusTmaWaitTimeout, 1000u);
      ok = ok && khd::mbar_wait(bar_k_full, 0u, &s_abort, status, khd::kStatusTmaWaitTimeout, 0u);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        khd::tc_fence_after_sync();
        issue_s(0);
      }
      for (int j = 0; j < num_kv && ok; ++j) {
        const int b = j & 1;
        const uint32_t phase = static_cast<uint32_t>((j >> 1) & 1);
        if (j + 1 < num_kv) {
          ok = khd::mbar_wait(bar_k_full + 8 * ((j + 1) & 1), static_cast<uint32_t>(((j + 1) >> 1) & 1),
                              &s_abort, status, khd::kStatusTmaWaitTimeout, static_cast<uint32_t>(j + 1));
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          khd::tc_fence_after_sync();
          issue_s((j + 1) & 1);
        }
        ok = khd::mbar_wait(bar_p_ready + 8 * b, phase, &s_abort, status,
                            khd::kStatusEpilogueWaitTimeout, static_cast<uint32_t>(j));
        ok = ok && khd::mbar_wait(bar_v_full + 8 * b, phase, &s_abort, status,
                                  khd::kStatusTmaWaitTimeout, 2000u + static_cast<uint32_t>(j));
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        khd::tc_fence_after_sync();
        // PV_j = P_j V_j: A = P buffer b (tensor memory), B = V^T tile, D = PV buffer b
        const uint64_t dv_hi = khd::umma_desc_k128(smem_v + b * kHalfStageBytes);
        const uint64_t dv_lo = dv_hi + 2 * kKVChunkStep;
        const uint32_t d = tmem_base + (b ? kColPV1 : kColPV0);
        const uint32_t p_base = tmem_base + (b ? kColP1 : kColP0);
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < kBKV / 8; ++kk) {
            const uint64_t voff = (kk >> 2) * kKVChunkStep + (kk & 3) * 2;
            umma_tf32_ts(d, p_base + 64 + kk * 8, dv_hi + voff, idesc, kk != 0 ? 1u : 0u);
            umma_tf32_ts(d, p_base + kk * 8, dv_lo + voff, idesc, 1u);
            umma_tf32_ts(d, p_base + kk * 8, dv_hi + voff, idesc, 1u);
          }
          khd::umma_commit(bar_pv_full + 8 * b);
          khd::umma_commit(bar_v_empty + 8 * b);
        }
        __syncwarp();
      }
    }
  } else {
    // ---- softmax + output: two groups of 128 threads, one thread per query row
    //      in each. Group g (warps 2-5 / 6-9) takes the tiles of parity g with its
    //      own running max, sum and output row; the groups work on neighbouring
    //      tiles at the same time and are merged once at the end. A warp may only
    //      touch tensor-memory lanes 32*(warp%4).., which both groups cover. -----------
    const int ew = warp - 2;
    const int quad = warp & 3;
    const int g = ew >> 2;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t col_s = g ? kColS1 : kColS0, col_p = g ? kColP1 : kColP0, col_pv = g ? kColPV1 : kColPV0;
    float acc[kHeadDim]; // running output of this group's tiles, normalised to its max
#pragma unroll
    for (int i = 0; i < kHeadDim; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    constexpr float kLog2e = 1.4426950408889634f;

    for (int j = g; j < num_kv && ok; j += 2) {
      const uint32_t phase = static_cast<uint32_t>((j >> 1) & 1);
      ok = khd::mbar_wait(bar_s_full + 8 * g, phase, &s_abort, status, khd::kStatusMmaWaitTimeout,
                          static_cast<uint32_t>(j));
      if (!ok) break;
      khd::tc_fence_after_sync();
      uint32_t sv[kBKV];
      khd::tmem_ld_32x32(tmem_base + lane_base + col_s, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
      khd::tmem_ld_32x32(tmem_base + lane_base + col_s + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
      khd::tmem_ld_wait();
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < kBKV; ++i) mx = fmaxf(mx, __uint_as_float(sv[i]));
      const float m_new = fmaxf(m, mx);
      const float alpha = fast_exp2((m - m_new) * kLog2e); // m = -inf on the first tile gives 0
      const float mb = m_new * kLog2e;
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < kBKV; ++i) {
        const float p = fast_exp2(fmaf(__uint_as_float(sv[i]), kLog2e, -mb));
        sv[i] = __float_as_uint(p);
        sum += p;
      }
      l = l * alpha + sum;
      m = m_new;

      // The group's previous product PV_{j-2} read P buffer g and wrote PV buffer
      // g: fold it in (it is normalised to the previous max), which also frees
      // both buffers, then move the running output to the new max.
      if (j >= 2) {
        ok = khd::mbar_wait(bar_pv_full + 8 * g, phase ^ 1u, &s_abort, status,
                            khd::kStatusMmaWaitTimeout, 2000u + static_cast<uint32_t>(j));
        if (!ok) break;
        khd::tc_fence_after_sync();
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          uint32_t t[16];
          tmem_ld_32x16(tmem_base + lane_base + col_pv + 16 * h, t);
          khd::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[16 * h + i] = (acc[16 * h + i] + __uint_as_float(t[i])) * alpha;
        }
      }
      // P -> tensor memory as hi / lo
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        uint32_t hi[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) hi[i] = __float_as_uint(tf32_hi(__uint_as_float(sv[16 * h + i])));
        tmem_st_32x16(tmem_base + lane_base + col_p + 16 * h, hi);
#pragma unroll
        for (int i = 0; i < 16; ++i)
          hi[i] = __float_as_uint(__uint_as_float(sv[16 * h + i]) - __uint_as_float(hi[i]));
        tmem_st_32x16(tmem_base + lane_base + col_p + 64 + 16 * h, hi);
      }
      tmem_st_wait();
      khd::tc_fence_before_sync();
      khd::mbar_arrive(bar_p_ready + 8 * g);
    }
    // this group's last product
    const int my_tiles = (num_kv - g + 1) / 2;
    if (ok && my_tiles > 0) {
      const int jl = g + 2 * (my_tiles - 1);
      ok = khd::mbar_wait(bar_pv_full + 8 * g, static_cast<uint32_t>((jl >> 1) & 1), &s_abort, status,
                          khd::kStatusMmaWaitTimeout, 3000u);
      if (ok) {
        khd::tc_fence_after_sync();
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          uint32_t t[16];
          tmem_ld_32x16(tmem_base + lane_base + col_pv + 16 * h, t);
          khd::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[16 * h + i] += __uint_as_float(t[i]);
        }
      }
    }
    // Merge: group 1 hands (max, sum, output row) to group 0 through the Q
    // buffer, which is free once the very last product of the CTA has run.
    if (ok && num_kv > 0) {
      const int jt = num_kv - 1;
      ok = khd::mbar_wait(bar_pv_full + 8 * (jt & 1), static_cast<uint32_t>((jt >> 1) & 1), &s_abort,
                          status, khd::kStatusMmaWaitTimeout, 3001u);
    }
    float *merge = reinterpret_cast<float *>(smem_raw + (smem_q - khd::smem_u32(smem_raw))) +
                   row_in_tile * (kHeadDim + 3);
    if (ok && g == 1) {
      merge[0] = m;
      merge[1] = l;
#pragma unroll
      for (int i = 0; i < kHeadDim; ++i) merge[2 + i] = acc[i];
    }
    khd::mbar_arrive(bar_exchange);
    ok = ok && khd::mbar_wait(bar_exchange, 0u, &s_abort, status, khd::kStatusEpilogueWaitTimeout, 5000u);
    if (ok && g == 0 && num_kv > 0) {
      const float m1 = merge[0], l1 = merge[1];
      const float mt = fmaxf(m, m1);
      const float w0 = fast_exp2((m - mt) * kLog2e), w1 = fast_exp2((m1 - mt) * kLog2e);
      const float inv = 1.0f / (l * w0 + l1 * w1);
      const int64_t row = static_cast<int64_t>(q0) + row_in_tile;
      float *orow = out + (bh * seq + row) * kHeadDim;
      if (row < seq) {
#pragma unroll
        for (int i = 0; i < kHeadDim / 4; ++i)
          __stcs(reinterpret_cast<float4 *>(orow) + i,
                 make_float4((acc[4 * i + 0] * w0 + merge[2 + 4 * i + 0] * w1) * inv,
                             (acc[4 * i + 1] * w0 + merge[2 + 4 * i + 1] * w1) * inv,
                             (acc[4 * i + 2] * w0 + merge[2 + 4 * i + 2] * w1) * inv,
                             (acc[4 * i + 3] * w0 + merge[2 + 4 * i + 3] * w1) * inv));
      }
    }
    khd::tc_fence_before_sync();
  }

  __syncthreads();
  if (s_abort) {
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
  }
  if (warp == 1) {
    khd::tc_fence_after_sync();
    khd::tmem_dealloc(tmem_base, kTmemCols);
  }
}
