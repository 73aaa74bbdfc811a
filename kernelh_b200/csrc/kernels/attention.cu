// attention: O = softmax(Q K^T / sqrt(d)) V, non-causal, fp32, d = 64,
// tensors [batch, heads, seq, 64] contiguous (seq a multiple of 64 in the plain entries; any seq
// and the causal mask in `attention_masked`).
//
// Replaces the kernel the reference generates from
// lib/dsl/kernels/attention.cpp:86-289 (one 64-thread block per query row,
// every block re-staging all of K and V in tiles of 64 with a per-key online
// rescale, 268-276; head_dim pinned to 64 and seq % 64 == 0, 109-120). Entry
// symbol `attention`; the first 44 parameters are the reference's: (Q, K, V,
// O) as rank-4 memref descriptors. The TMA-fed kernel then takes six tensor
// maps, the scale exponents and a status pointer.
//
// Flash-style: a CTA owns 128 query rows of one (batch, head) and streams K/V
// in tiles of 64 keys. Both contractions run on tcgen05 tensor cores as three
// fp16 products of scaled hi/lo splits (see kh_fp16_split.cuh; products lo.hi,
// hi.lo, hi.hi into one fp32 accumulator):
//   S = Q K^T   A = Q tile (shared memory, K-major), B = K tile (K-major)
//   PV = P V    A = P (tensor memory, two fp16 per column), B = V^T tile
//               (K-major over keys)
// Q, K and V are scaled by one power of two per tile of 64 rows (the tile's
// largest magnitude goes to [2^14, 2^15)). A score tile therefore carries one
// factor per (query tile, key tile), which the softmax folds, with 1/sqrt(64),
// into the constant it multiplies that tile's scores by; a PV tile carries the
// factor of its V tile, applied when the tile is added to the running output
// row. P lies in [0, 1] and is multiplied by 2^14 before its split so that its
// lo part stays a normal fp16.
// Scores, probabilities and the per-tile PV product live in tensor memory;
// the running max, sum and the 64-wide output row live in registers of the
// thread that owns the row (one thread per tensor-memory lane).
//
// Two launches:
//  attention_split  writes Q, K and V^T as scaled fp16 hi/lo pairs into scratch
//      and the exponent of every 64-row tile.
//  attention  a persistent grid, one CTA of four warpgroups per SM; a CTA takes
//      work items (128 query rows of one (batch, head) each) b, b + gridDim.x,
//      ... and keeps its pipelines running across them. Warpgroup 0: warp 0
//      feeds TMA (the Q tile of an item into one of two buffers; separate
//      4-deep rings of K and V^T tiles), warps 1 and 2 issue the MMAs, one warp
//      per softmax group (S of the group's next tile goes into its score
//      buffer as soon as the group has read the current scores out, ahead of PV
//      of the current tile, so a group never waits for scores and the tensor
//      core works while softmax runs). Warpgroups 1 and 2 are the two softmax
//      groups (one thread per query row each) that take the even and the odd
//      tiles with their own running max, sum and output row, so two tiles are
//      in the softmax stage at once; at the end of an item a group parks its
//      row in tensor memory and moves on. Warpgroup 3 combines the two parked
//      rows and writes the finished rows out. The warpgroups trade registers
//      at the start (setmaxnreg): most go to the softmax threads.
//      Scores, P, PV and the parked rows sit in tensor memory, one set per group.
//
// Tensor-bound: 4 b h s^2 d useful flops; three products put the ceiling at one
// third of the fp16 tensor rate.
#include "kh_fp16_split.cuh"
#include "kh_tcgen05.cuh"

namespace {

using khd::Half8;
using khd::RowScale;
using khd::row_scale;
using khd::scale_shift;
using khd::split_fp16_pairs;
using khd::split_fp16x2;

constexpr int kHeadDim = 64;
constexpr int kBQ = 128;  // query rows per CTA
constexpr int kBKV = 64;  // keys per tile
constexpr int kStages = 4; // K and V^T tiles in flight (rings of their own)
// Four warpgroups: [producer, issuer of group 0, issuer of group 1, spare], softmax
// group 0, softmax group 1, output. A warp of the last three touches the
// tensor-memory lanes 32 * (warp % 4) .. of its rows.
constexpr int kThreads = 512;
// registers per thread after the warpgroups have traded them (sum x 128 = the register file)
constexpr int kRegsControl = 56, kRegsSoftmax = 184, kRegsOutput = 88;
constexpr int kRegisterBoundThreads = kThreads; // 128 registers per thread at launch
constexpr int kRowBytes = 128;                       // 64 fp16: one 128-byte swizzle row
constexpr int kQTileBytes = kBQ * kRowBytes;         // 16 KiB: 128 rows, hi or lo
constexpr int kKVTileBytes = kBKV * kRowBytes;       // 8 KiB: 64 rows (keys, or rows of V^T), hi or lo
constexpr int kQBytes = 2 * kQTileBytes;             // hi + lo = 32 KiB
constexpr int kHalfStageBytes = 2 * kKVTileBytes;    // one K (or V^T) tile: hi + lo = 16 KiB
constexpr int kPShift = 14;                          // P is split as P * 2^14
// tensor-memory columns: two score buffers, two P buffers (32 columns of packed
// fp16 pairs for hi, 32 for lo), two PV buffers
constexpr uint32_t kColS0 = 0, kColS1 = 64, kColP0 = 128, kColP1 = 192, kColPV0 = 256, kColPV1 = 320,
                   kColOut0 = 384, kColOut1 = 448; // a group's finished row of an item, parked for the output warps
constexpr uint32_t kTmemCols = 512;

// 2^x by the special-function unit (2 ulp, flushes denormals): the arguments
// here are <= 0 and the results feed a sum of at least 1.
// Registers move between warpgroups (each executes one of these once, as a whole).
template <int kRegs>
__device__ __forceinline__ void registers_release() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs>
__device__ __forceinline__ void registers_take() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// D[tmem] (+)= A[tmem] * B[smem]; A holds two fp16 per 32-bit column (k even in the low half)
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
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

__device__ __forceinline__ uint32_t half2_bits(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }

} // namespace

// Q, K, V [bh, seq, 64] -> q_hi, q_lo, k_hi, k_lo [bh*seq, 64] and vt_hi, vt_lo
// [bh*64, seq] (V transposed per (batch, head)) as fp16 (seq rounded up to whole 64-row tiles in all six). The unit of scaling is
// a tile of 64 rows (queries or keys) of one slice: a block takes one tile of one
// tensor at a time, finds its largest magnitude, and writes the two splits scaled
// by the exponent that gives; shifts[(t * bh + slice) * tiles + tile] receives
// the exponent (t = 0, 1, 2 for Q, K, V).
extern "C" __global__ void __launch_bounds__(256, 5)
attention_split(KH_MEMREF4(const float, q), KH_MEMREF4(const float, k), KH_MEMREF4(const float, v),
                __half *__restrict__ q_hi, __half *__restrict__ q_lo, __half *__restrict__ k_hi,
                __half *__restrict__ k_lo, __half *__restrict__ vt_hi, __half *__restrict__ vt_lo,
                int *__restrict__ shifts) {
  // float4 groups of a row are stored at group ^ (row / 8 mod 8): conflict-free both ways
  __shared__ __align__(16) float tile[64][64];
  __shared__ float warp_max[2][8]; // alternating per job, so one barrier per job orders it
  const int64_t bh = q_size0 * q_size1, seq = q_size2;
  // Job arithmetic is 32-bit and free of 64-bit divisions (a software routine of about a hundred
  // instructions each, several per tile and thread, which once made this kernel issue-bound):
  // a tensor has bh * seq / 64 tiles (< 2^31 for anything that fits the GPU), a tile's source is
  // 4096 contiguous floats, and only V needs (slice, tile) separately.
  // seq need not be a multiple of 64: the last tile of a slice is then short, its missing rows count
  // as zeros, and the splits are laid out with every slice padded to whole tiles (seq_p rows).
  const uint32_t tiles = static_cast<uint32_t>((seq + 63) >> 6);
  const bool ragged = (seq & 63) != 0;
  const int64_t seq_p = static_cast<int64_t>(tiles) << 6;
  const uint32_t per_tensor = static_cast<uint32_t>(bh) * tiles;
  const uint32_t jobs = 3u * per_tensor;
  const float *const src_q = KH_DATA(q), *const src_k = KH_DATA(k), *const src_v = KH_DATA(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the tile of a job is 64 x 64 contiguous values = 1024 float4; a thread takes float4 tid, tid + 256, ...
  const auto tensor_of = [&](uint32_t job) { return (job >= per_tensor ? 1u : 0u) + (job >= 2u * per_tensor ? 1u : 0u); };
  // loads a job's tile: float4 tid + 256 j of the tile is group tid % 16 of row tid / 16 + 16 j
  const auto load_tile = [&](uint32_t job, float4 &a0, float4 &a1, float4 &a2, float4 &a3) {
    const uint32_t t = tensor_of(job), rest = job - t * per_tensor; // rest = slice * tiles + tile
    const float *base = t == 0 ? src_q : (t == 1 ? src_k : src_v); // selects, not an indexed local array
    if (!ragged) {
      const float4 *p = reinterpret_cast<const float4 *>(base + static_cast<size_t>(rest) * (64 * kHeadDim)) + threadIdx.x;
      a0 = __ldcs(p); a1 = __ldcs(p + 256); a2 = __ldcs(p + 512); a3 = __ldcs(p + 768);
      return;
    }
    const uint32_t slice = rest / tiles, tile_in_slice = rest - slice * tiles;
    const int valid = min(64, static_cast<int>(seq - static_cast<int64_t>(tile_in_slice) * 64)); // rows the tile really has
    const float4 *p = reinterpret_cast<const float4 *>(base + (static_cast<size_t>(slice) * seq + tile_in_slice * 64) * kHeadDim) +
                      threadIdx.x;
    const int row = static_cast<int>(threadIdx.x >> 4);
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    a0 = row < valid ? __ldcs(p) : zero;
    a1 = row + 16 < valid ? __ldcs(p + 256) : zero;
    a2 = row + 32 < valid ? __ldcs(p + 512) : zero;
    a3 = row + 48 < valid ? __ldcs(p + 768) : zero;
  };
  // The attention kernel that follows may be scheduled as soon as SMs drain: its CTAs set up
  // their barriers and tensor memory and then wait for this whole grid before reading anything.
  khd::grid_dependents_may_launch();
  float4 n0 = make_float4(0.f, 0.f, 0.f, 0.f), n1 = n0, n2 = n0, n3 = n0;
  if (blockIdx.x < jobs) load_tile(blockIdx.x, n0, n1, n2, n3);
  int parity = 0;
  for (uint32_t job = blockIdx.x; job < jobs; job += gridDim.x, parity ^= 1) {
    const uint32_t t = tensor_of(job), rest = job - t * per_tensor;
    const float4 f0 = n0, f1 = n1, f2 = n2, f3 = n3;
    // the next tile's loads fly while this one is worked on (jobs < 2^31 - grid)
    if (job + gridDim.x < jobs) load_tile(job + gridDim.x, n0, n1, n2, n3);
    float m = fmaxf(fmaxf(fmaxf(fabsf(f0.x), fabsf(f0.y)), fmaxf(fabsf(f0.z), fabsf(f0.w))),
                    fmaxf(fmaxf(fabsf(f1.x), fabsf(f1.y)), fmaxf(fabsf(f1.z), fabsf(f1.w))));
    m = fmaxf(m, fmaxf(fmaxf(fmaxf(fabsf(f2.x), fabsf(f2.y)), fmaxf(fabsf(f2.z), fabsf(f2.w))),
                       fmaxf(fmaxf(fabsf(f3.x), fabsf(f3.y)), fmaxf(fabsf(f3.z), fabsf(f3.w)))));
    m = khd::warp_max_redux_numbers(m);
    if (lane == 0) warp_max[parity][warp] = m; // the job before last used this half: a barrier lies between
    if (t == 2) {
      __syncthreads(); // the previous job (a V tile too, or the last K tile) is done with the tile
      // V goes through shared memory: row = key, 16 float4 groups per row; float4 tid + 256 j
      // is group tid % 16 of row tid / 16 + 16 j
      const int sl = threadIdx.x >> 4, g = threadIdx.x & 15;
      *reinterpret_cast<float4 *>(&tile[sl][(g ^ ((sl >> 3) & 7)) * 4]) = f0;
      *reinterpret_cast<float4 *>(&tile[sl + 16][(g ^ (((sl + 16) >> 3) & 7)) * 4]) = f1;
      *reinterpret_cast<float4 *>(&tile[sl + 32][(g ^ (((sl + 32) >> 3) & 7)) * 4]) = f2;
      *reinterpret_cast<float4 *>(&tile[sl + 48][(g ^ (((sl + 48) >> 3) & 7)) * 4]) = f3;
    }
    __syncthreads();
    m = warp_max[parity][0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, warp_max[parity][w]);
    const int shift = scale_shift(m);
    const RowScale sc = row_scale(shift);
    if (threadIdx.x == 0) shifts[job] = shift;
    if (t < 2) {
      // four values -> 8 bytes of hi and of lo; a warp store covers 256 contiguous bytes
      const float2 x[8] = {make_float2(f0.x, f0.y), make_float2(f0.z, f0.w), make_float2(f1.x, f1.y),
                           make_float2(f1.z, f1.w), make_float2(f2.x, f2.y), make_float2(f2.z, f2.w),
                           make_float2(f3.x, f3.y), make_float2(f3.z, f3.w)};
      __half2 h[8], l[8];
      split_fp16_pairs<8>(x, sc, h, l);
      // (slice * seq + s0) * 64 = rest * 4096: the splits of Q and K are laid out like their sources
      uint2 *out_hi = reinterpret_cast<uint2 *>((t == 0 ? q_hi : k_hi) + static_cast<size_t>(rest) * (64 * kHeadDim)) + threadIdx.x;
      uint2 *out_lo = reinterpret_cast<uint2 *>((t == 0 ? q_lo : k_lo) + static_cast<size_t>(rest) * (64 * kHeadDim)) + threadIdx.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        out_hi[256 * j] = make_uint2(half2_bits(h[2 * j]), half2_bits(h[2 * j + 1]));
        out_lo[256 * j] = make_uint2(half2_bits(l[2 * j]), half2_bits(l[2 * j + 1]));
      }
    } else {
      const uint32_t slice = rest / tiles, s0 = (rest - slice * tiles) << 6;
      const int sub = lane >> 3, sgroup = lane & 7; // 4 rows of V^T per warp store, 8 keys per lane
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int dl = warp * 8 + j * 4 + sub;
        const int col = (((dl >> 2) ^ sgroup) << 2) | (dl & 3); // rows sgroup*8.. share one swizzle
        Half8 h, l;
        float2 x[4];
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) x[qd] = make_float2(tile[sgroup * 8 + 2 * qd][col], tile[sgroup * 8 + 2 * qd + 1][col]);
        split_fp16_pairs<4>(x, sc, h.v, l.v);
        const int64_t o = (static_cast<int64_t>(slice) * kHeadDim + dl) * seq_p + s0 + sgroup * 8;
        *reinterpret_cast<Half8 *>(vt_hi + o) = h;
        *reinterpret_cast<Half8 *>(vt_lo + o) = l;
      }
    }
  }
}

namespace {

// Where a finished output tile also goes when the (batch, head) slices are
// sharded over several GPUs and every GPU keeps the whole output: either the
// NVLink multicast address of the replicas (one multimem.st reaches all of
// them), or the other GPUs' replicas one by one (plain peer stores). All
// pointers address this rank's first slice inside the respective replica.
struct GatherOut {
  float *peer[8];
  int count;
  int self;
  float *multicast;
};

__device__ __forceinline__ void multicast_store_float4(float *p, float4 v) {
  asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w)
               : "memory");
}

// The kernel body. `slices`: (batch, head) problems of this launch; `seq`: keys
// (= queries) per slice; `out`: this launch's [slices, seq, 64] output. The
// grid is persistent: CTA b takes the work items (one tile of 128 query rows of
// one slice each) b, b + gridDim.x, ... and every role walks the same list, so
// that the loads and the first score products of the next item run while the
// softmax groups finish the current one. kGather: after the 128 x 64 output tile
// of an item (32 KiB, contiguous) is stored, the group that stored it reads it
// back from L2 and sends it to the other replicas in 512-byte warp-wide pieces.
// kMask: the instantiation that can mask scores - `causal` (query i sees keys 0..i) and / or a seq
// that is not a multiple of 64 (the last key tile's missing keys). Separate from the plain one: the
// mask costs the softmax threads registers, 5 us of 105 at batch 8 x 16 heads x 1024 as a run-time flag.
template <bool kGather, bool kMask>
__device__ __forceinline__ void attention_body(int64_t slices, int64_t seq, float *__restrict__ out,
                                               const khd::TensorMap &tm_q_hi, const khd::TensorMap &tm_q_lo,
                                               const khd::TensorMap &tm_k_hi, const khd::TensorMap &tm_k_lo,
                                               const khd::TensorMap &tm_vt_hi, const khd::TensorMap &tm_vt_lo,
                                               const int *__restrict__ shifts, uint32_t *status, int causal_flag,
                                               const GatherOut *targets) {
  extern __shared__ uint8_t smem_raw[];
  // q_full[2], q_empty[2], k_full, k_empty, v_full, v_empty [kStages each], s_full[2], s_free[2],
  // p_ready[2], pv_full[2], parked[2], out_free
  __shared__ __align__(8) uint64_t bars[4 + 4 * kStages + 8 + 3];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ float s_row_m[2][kBQ], s_row_l[2][kBQ]; // max and sum that go with a group's parked row

  const bool causal = kMask && causal_flag != 0;
  const int64_t seq_p = (seq + kBKV - 1) / kBKV * kBKV; // rows a slice has in the splits (whole 64-row tiles)
  const int64_t q_tiles = (seq + kBQ - 1) / kBQ;
  const int64_t items = slices * q_tiles;
  const int num_kv = static_cast<int>(seq_p / kBKV);
  // Key tiles an item (128 query rows starting at row q0 of its slice) goes through. With the causal
  // mask (query i sees keys <= i) that is up to and including the two 64-key tiles on the item's
  // diagonal: always an even number, so both softmax groups keep a tile parity each; the rows of the
  // two diagonal tiles are masked in the softmax. Every role computes the same count.
  const auto kv_tiles_of = [&](int q0) { return causal ? min(num_kv, 2 * (q0 / kBQ) + 2) : num_kv; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const uint32_t smem_q = (khd::smem_u32(smem_raw) + 1023u) & ~1023u; // two Q tiles (hi, lo each)
  const uint32_t smem_k = smem_q + 2 * kQBytes;                       // kStages stages of K hi, lo
  const uint32_t smem_v = smem_k + kStages * kHalfStageBytes;         // kStages stages of V^T hi, lo
  const uint32_t smem_scratch = smem_v + kStages * kHalfStageBytes;   // 16 KiB: half an output row per query row
  const uint32_t bar_q_full = khd::smem_u32(&bars[0]);
  const uint32_t bar_q_empty = khd::smem_u32(&bars[2]);
  const uint32_t bar_k_full = khd::smem_u32(&bars[4]);
  const uint32_t bar_k_empty = khd::smem_u32(&bars[4 + kStages]);
  const uint32_t bar_v_full = khd::smem_u32(&bars[4 + 2 * kStages]);
  const uint32_t bar_v_empty = khd::smem_u32(&bars[4 + 3 * kStages]);
  const uint32_t bar_s_full = khd::smem_u32(&bars[4 + 4 * kStages]);
  const uint32_t bar_s_free = khd::smem_u32(&bars[6 + 4 * kStages]);
  const uint32_t bar_p_ready = khd::smem_u32(&bars[8 + 4 * kStages]);
  const uint32_t bar_pv_full = khd::smem_u32(&bars[10 + 4 * kStages]);
  const uint32_t bar_parked = khd::smem_u32(&bars[12 + 4 * kStages]);   // [group]: its row of the item is parked
  const uint32_t bar_out_free = khd::smem_u32(&bars[14 + 4 * kStages]); // the output warps have read both rows

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < 2; ++s) {
      khd::mbar_init(bar_q_full + 8 * s, 1);
      khd::mbar_init(bar_q_empty + 8 * s, 2); // both issuers are done with the Q tile
      khd::mbar_init(bar_s_full + 8 * s, 1);
      khd::mbar_init(bar_s_free + 8 * s, kBQ);  // one arrival per thread of the group once it holds the scores
      khd::mbar_init(bar_p_ready + 8 * s, kBQ); // one arrival per thread of the group that owns the buffer
      khd::mbar_init(bar_pv_full + 8 * s, 1);
    }
    for (int s = 0; s < kStages; ++s) {
      khd::mbar_init(bar_k_full + 8 * s, 1);
      khd::mbar_init(bar_k_empty + 8 * s, 1);
      khd::mbar_init(bar_v_full + 8 * s, 1);
      khd::mbar_init(bar_v_empty + 8 * s, 1);
    }
    khd::mbar_init(bar_parked, kBQ);
    khd::mbar_init(bar_parked + 8, kBQ);
    khd::mbar_init(bar_out_free, kBQ);
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
  // The launch may have been scheduled under the tail of attention_split: everything above touched
  // only this CTA's own shared and tensor memory; the splits and exponents are read from here on.
  khd::grid_dependency_wait();

  const int wg = warp >> 2;
  if (wg == 0) {
  registers_release<kRegsControl>();
  if (warp == 0) {
    // ---- TMA producer: per item the Q tile (two buffers, so the next item's
    //      tile loads while this one is in use), then the item's K and V^T
    //      tiles through rings of kStages tiles that run on across items. A K
    //      slot is free as soon as S of its tile has run, long before the V
    //      slot of that tile. -----------------------------------------------------------
    if (lane == 0) {
      uint32_t tile = 0; // tiles loaded so far
      bool ok = true;
      int n = 0;
      for (int64_t w = blockIdx.x; w < items && ok; w += gridDim.x, ++n) {
        const int64_t bh = w / q_tiles;
        const int q0 = static_cast<int>((w - bh * q_tiles) * kBQ);
        const int qb = n & 1;
        ok = khd::mbar_wait(bar_q_empty + 8 * qb, static_cast<uint32_t>((n >> 1) & 1) ^ 1u, &s_abort, status,
                            khd::kStatusEmptyWaitTimeout, 4000u);
        if (!ok) break;
        {
          const uint32_t bar = bar_q_full + 8 * qb;
          const int q_row = static_cast<int>(bh * seq_p) + q0;
          khd::mbar_arrive_expect_tx(bar, kQBytes);
          khd::tma_load_2d(smem_q + qb * kQBytes, &tm_q_hi, 0, q_row, bar);
          khd::tma_load_2d(smem_q + qb * kQBytes + kQTileBytes, &tm_q_lo, 0, q_row, bar);
        }
        const int kv_end = kv_tiles_of(q0);
        for (int j = 0; j < kv_end; ++j, ++tile) {
          const int s = static_cast<int>(tile % kStages);
          const uint32_t phase = (tile / kStages) & 1u;
          ok = khd::mbar_wait(bar_k_empty + 8 * s, phase ^ 1u, &s_abort, status, khd::kStatusEmptyWaitTimeout,
                              static_cast<uint32_t>(j));
          if (!ok) break;
          {
            const uint32_t st = smem_k + s * kHalfStageBytes;
            const uint32_t bar = bar_k_full + 8 * s;
            khd::mbar_arrive_expect_tx(bar, kHalfStageBytes);
            const int k_row = static_cast<int>(bh * seq_p) + j * kBKV;
            khd::tma_load_2d(st, &tm_k_hi, 0, k_row, bar);
            khd::tma_load_2d(st + kKVTileBytes, &tm_k_lo, 0, k_row, bar);
          }
          ok = khd::mbar_wait(bar_v_empty + 8 * s, phase ^ 1u, &s_abort, status, khd::kStatusEmptyWaitTimeout,
                              1000u + static_cast<uint32_t>(j));
          if (!ok) break;
          {
            const uint32_t st = smem_v + s * kHalfStageBytes;
            const uint32_t bar = bar_v_full + 8 * s;
            khd::mbar_arrive_expect_tx(bar, kHalfStageBytes);
            const int v_row = static_cast<int>(bh * kHeadDim);
            const int v_col = j * kBKV;
            khd::tma_load_2d(st, &tm_vt_hi, v_col, v_row, bar);
            khd::tma_load_2d(st + kKVTileBytes, &tm_vt_lo, v_col, v_row, bar);
          }
        }
      }
    }
  } else if (warp == 1 || warp == 2) {
    // ---- MMA issuers, one warp per softmax group: warp 1 takes the even tiles
    //      of every item, the last warp the odd ones (a single thread cannot
    //      issue tcgen05.mma fast enough for both). Per tile j of its parity:
    //      S_{j+2} into the group's score buffer as soon as the group has read
    //      S_j out (s_free), then PV_j once P_j is written; the scores of a
    //      group's next tile, the first tile of the next item included, are
    //      computed while it still works on the current one. The whole warp walks
    //      the loop (waits, descriptor arithmetic: warp-uniform, so it stays in
    //      uniform registers); only the tcgen05 instructions themselves sit
    //      under the elected lane. ------------------------------------------------------
    {
      const int g = warp - 1;
      const bool leader = khd::elect_one();
      constexpr uint32_t idesc = khd::umma_idesc_f16(kBQ, kBKV); // M128 N64 K16 for both products
      constexpr uint64_t kKVTileStep = kKVTileBytes >> 4;
      const uint32_t col_s = tmem_base + (g ? kColS1 : kColS0), col_p = tmem_base + (g ? kColP1 : kColP0),
                     col_pv = tmem_base + (g ? kColPV1 : kColPV0);
      uint32_t tile_base = 0;  // tiles of the items before this one
      uint32_t s_count = 0;    // score products this warp has issued
      uint32_t pv_count = 0;   // PV products this warp has issued
      bool ok = true;
      int n = 0;
      int kv_end = 0;
      for (int64_t w = blockIdx.x; w < items && ok; w += gridDim.x, ++n, tile_base += static_cast<uint32_t>(kv_end)) {
        kv_end = kv_tiles_of(static_cast<int>((w % q_tiles) * kBQ));
        const int qb = n & 1;
        ok = khd::mbar_wait(bar_q_full + 8 * qb, static_cast<uint32_t>((n >> 1) & 1), &s_abort, status,
                            khd::kStatusTmaWaitTimeout, 1000u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        khd::tc_fence_after_sync();
        // a tile row is one 128-byte swizzle row (64 fp16); a k-step of 16 fp16 moves 32 bytes (2 encoded)
        const uint64_t dq_hi = khd::umma_desc_k128(smem_q + qb * kQBytes);
        const uint64_t dq_lo = khd::umma_desc_k128(smem_q + qb * kQBytes + kQTileBytes);
        // S_t = Q K_t^T into this group's score buffer; tile t of the item sits in ring slot (tile_base + t) % kStages
        auto issue_s = [&](int t) -> bool {
          const uint32_t tile = tile_base + static_cast<uint32_t>(t);
          const int slot = static_cast<int>(tile % kStages);
          bool ready = khd::mbar_wait(bar_k_full + 8 * slot, (tile / kStages) & 1u, &s_abort, status,
                                      khd::kStatusTmaWaitTimeout, static_cast<uint32_t>(t));
          if (s_count >= 1) // the group holds the scores of its previous tile in registers
            ready = ready && khd::mbar_wait(bar_s_free + 8 * g, (s_count - 1) & 1u, &s_abort, status,
                                            khd::kStatusEpilogueWaitTimeout, 3000u + static_cast<uint32_t>(t));
          ready = __all_sync(0xffffffffu, ready);
          if (!ready) return false;
          khd::tc_fence_after_sync();
          const uint64_t dk_hi = khd::umma_desc_k128(smem_k + slot * kHalfStageBytes);
          const uint64_t dk_lo = dk_hi + kKVTileStep;
          if (leader) {
#pragma unroll
            for (int kk = 0; kk < kHeadDim / 16; ++kk) {
              const uint64_t off = static_cast<uint64_t>(kk * 2);
              khd::umma_f16_ss(col_s, dq_lo + off, dk_hi + off, idesc, kk != 0 ? 1u : 0u);
              khd::umma_f16_ss(col_s, dq_hi + off, dk_lo + off, idesc, 1u);
              khd::umma_f16_ss(col_s, dq_hi + off, dk_hi + off, idesc, 1u);
            }
            khd::umma_commit(bar_s_full + 8 * g);     // scores ready for the softmax threads
            khd::umma_commit(bar_k_empty + 8 * slot); // and this K slot may be refilled
            if (t + 2 >= kv_end) khd::umma_commit(bar_q_empty + 8 * qb); // this warp's last use of the Q tile
          }
          __syncwarp();
          ++s_count;
          return true;
        };
        if (g < kv_end) {
          ok = issue_s(g);
        } else if (leader) {
          khd::mbar_arrive(bar_q_empty + 8 * qb); // no tile of this parity: nothing of Q is used here
        }
        for (int j = g; j < kv_end && ok; j += 2) {
          const uint32_t tile = tile_base + static_cast<uint32_t>(j);
          const int slot = static_cast<int>(tile % kStages);
          if (j + 2 < kv_end && !issue_s(j + 2)) {
            ok = false;
            break;
          }
          ok = khd::mbar_wait(bar_p_ready + 8 * g, pv_count & 1u, &s_abort, status,
                              khd::kStatusEpilogueWaitTimeout, static_cast<uint32_t>(j));
          ok = ok && khd::mbar_wait(bar_v_full + 8 * slot, (tile / kStages) & 1u, &s_abort, status,
                                    khd::kStatusTmaWaitTimeout, 2000u + static_cast<uint32_t>(j));
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          khd::tc_fence_after_sync();
          // PV_j = P_j V_j: A = the group's P buffer (tensor memory), B = V^T tile, D = its PV buffer
          const uint64_t dv_hi = khd::umma_desc_k128(smem_v + slot * kHalfStageBytes);
          const uint64_t dv_lo = dv_hi + kKVTileStep;
          if (leader) {
#pragma unroll
            for (int kk = 0; kk < kBKV / 16; ++kk) { // 16 keys = 8 packed columns of P
              const uint64_t voff = static_cast<uint64_t>(kk * 2);
              umma_f16_ts(col_pv, col_p + 32 + kk * 8, dv_hi + voff, idesc, kk != 0 ? 1u : 0u);
              umma_f16_ts(col_pv, col_p + kk * 8, dv_lo + voff, idesc, 1u);
              umma_f16_ts(col_pv, col_p + kk * 8, dv_hi + voff, idesc, 1u);
            }
            khd::umma_commit(bar_pv_full + 8 * g);
            khd::umma_commit(bar_v_empty + 8 * slot);
          }
          __syncwarp();
          ++pv_count;
        }
      }
    }
  }
  } else if (wg == 1 || wg == 2) {
    registers_take<kRegsSoftmax>();
    // ---- softmax: two groups of 128 threads (warpgroups 1 and 2), one thread per
    //      query row in each. Group g takes the tiles of parity g of every item
    //      with its own running max, sum and output row; the groups work on
    //      neighbouring tiles at the same time and never wait for each other. At
    //      the end of an item a group parks (max, sum, row) - the row in tensor
    //      memory - for the output warps and goes on to the next item. A warp may
    //      only touch tensor-memory lanes 32*(warp%4).., which both groups cover. ------
    const int ew = warp - 4;
    const int quad = warp & 3;
    const int g = ew >> 2;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t col_s = g ? kColS1 : kColS0, col_p = g ? kColP1 : kColP0, col_pv = g ? kColPV1 : kColPV0;
    const uint32_t col_out = g ? kColOut1 : kColOut0;
    constexpr float kLog2eOverSqrtD = 1.4426950408889634f * 0.125f;
    uint32_t tiles_done = 0; // tiles this group has been through, over all items
    bool ok = true;
    int n = 0;
    // Exponents of the 64-row tiles: shifts[(t * slices + slice) * tiles + tile], t = 0, 1, 2 for Q, K, V.
    // Those an item starts with (its row's Q tile, the group's first K and V tile)
    // are fetched while the item before it finishes.
    int item_shift_q = 0, item_shift_k = 0, item_shift_v = 0;
    const auto fetch_item_shifts = [&](int64_t w) {
      const int64_t bh = w / q_tiles;
      const int row_q = static_cast<int>((w - bh * q_tiles) * kBQ) + row_in_tile;
      item_shift_q = __ldg(shifts + bh * num_kv + (row_q < seq ? row_q >> 6 : 0));
      item_shift_k = g < num_kv ? __ldg(shifts + (slices + bh) * num_kv + g) : 0;
      item_shift_v = g < num_kv ? __ldg(shifts + (2 * slices + bh) * num_kv + g) : 0;
    };
    if (blockIdx.x < items) fetch_item_shifts(blockIdx.x);
    for (int64_t w = blockIdx.x; w < items && ok; w += gridDim.x, ++n) {
      const int64_t bh = w / q_tiles;
      float acc[kHeadDim]; // running output of this group's tiles, normalised to its max
#pragma unroll
      for (int i = 0; i < kHeadDim; ++i) acc[i] = 0.f;
      float m = -INFINITY, l = 0.f;
      // The running max `m` is kept in exp2 units, i.e. true score * log2(e) / sqrt(64).
      const int *k_shifts = shifts + (slices + bh) * num_kv, *v_shifts = shifts + (2 * slices + bh) * num_kv;
      const int shift_q = item_shift_q;
      float v_factor_prev = 0.f; // 2^-(exponent of the V tile) of this group's previous product
      // the exponents of this group's next tile are fetched one tile ahead
      int shift_k_next = item_shift_k, shift_v_next = item_shift_v;
      bool first = true; // no product of this item to fold in yet

      const int q0_item = static_cast<int>((w - bh * q_tiles) * kBQ);
      const int kv_end = kv_tiles_of(q0_item);
      const int diagonal = causal ? q0_item / kBKV : num_kv; // first key tile that needs the causal mask
      const int keys_in_last = static_cast<int>(seq - static_cast<int64_t>(num_kv - 1) * kBKV); // 64 unless seq is ragged
      for (int j = g; j < kv_end && ok; j += 2) {
        const uint32_t phase = tiles_done & 1u;
        const int shift_k = shift_k_next, shift_v = shift_v_next;
        if (j + 2 < kv_end) {
          shift_k_next = __ldg(k_shifts + j + 2);
          shift_v_next = __ldg(v_shifts + j + 2);
        }
        ok = khd::mbar_wait(bar_s_full + 8 * g, phase, &s_abort, status, khd::kStatusMmaWaitTimeout,
                            static_cast<uint32_t>(j));
        if (!ok) break;
        khd::tc_fence_after_sync();
        uint32_t sv[kBKV];
        khd::tmem_ld_32x32(tmem_base + lane_base + col_s, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
        khd::tmem_ld_32x32(tmem_base + lane_base + col_s + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
        khd::tmem_ld_wait();
        khd::tc_fence_before_sync();
        khd::mbar_arrive(bar_s_free + 8 * g); // the score buffer may take S_{j+2}
        // this tile's scores carry 2^(shift_q + shift_k): one positive factor brings them to exp2 units
        const float f = khd::scale_pow2(kLog2eOverSqrtD, -(shift_q + shift_k));
        if (kMask && (j >= diagonal || j == num_kv - 1)) {
          // Keys of this tile the thread's query sees: all 64; on a diagonal tile of the causal mask
          // only 0 .. (its row - the tile's first key) (none at all on the second diagonal tile for the
          // upper 64 queries); in the last tile of a ragged seq only the keys that exist. The rest
          // count as -inf.
          int last_seen = kBKV - 1;
          if (j >= diagonal) last_seen = row_in_tile - (j - diagonal) * kBKV;
          if (j == num_kv - 1) last_seen = min(last_seen, keys_in_last - 1);
#pragma unroll
          for (int i = 0; i < kBKV; ++i)
            if (i > last_seen) sv[i] = 0xff800000u; // -inf
        }
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < kBKV; ++i) mx = fmaxf(mx, __uint_as_float(sv[i]));
        const float m_new = fmaxf(m, mx * f);
        // a row that has seen nothing but masked keys so far keeps max = -inf; its exponentials are
        // taken against 0 instead (they are all exp2(-inf) = 0), so that no inf - inf arises
        const float m_ref = (kMask && m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = fast_exp2(m - m_ref); // m = -inf on the first tile gives 0
        // P is produced as P * 2^14 straight from the exponent (its split wants that
        // range); the row sum `l` and the output row are kept in the same units.
        const float offset = static_cast<float>(kPShift) - m_ref;
        // (two fp32 per instruction where the arithmetic allows)
        const float2 f2 = make_float2(f, f), offset2 = make_float2(offset, offset);
        float2 sum2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < kBKV; i += 2) {
          const float2 x = __ffma2_rn(make_float2(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])), f2, offset2);
          const float2 p = make_float2(fast_exp2(x.x), fast_exp2(x.y));
          sv[i] = __float_as_uint(p.x);
          sv[i + 1] = __float_as_uint(p.y);
          sum2 = __fadd2_rn(sum2, p);
        }
        l = l * alpha + (sum2.x + sum2.y);
        m = m_new;

        // The group's previous product PV_{j-2} read P buffer g and wrote PV buffer
        // g: fold it in (it is normalised to the previous max), which also frees
        // both buffers, then move the running output to the new max.
        if (!first) {
          ok = khd::mbar_wait(bar_pv_full + 8 * g, phase ^ 1u, &s_abort, status,
                              khd::kStatusMmaWaitTimeout, 2000u + static_cast<uint32_t>(j));
          if (!ok) break;
          khd::tc_fence_after_sync();
          const float2 vf2 = make_float2(v_factor_prev, v_factor_prev), alpha2 = make_float2(alpha, alpha);
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            uint32_t t[16];
            tmem_ld_32x16(tmem_base + lane_base + col_pv + 16 * h, t);
            khd::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              const float2 r = __fmul2_rn(__ffma2_rn(make_float2(__uint_as_float(t[i]), __uint_as_float(t[i + 1])), vf2,
                                                     make_float2(acc[16 * h + i], acc[16 * h + i + 1])),
                                          alpha2);
              acc[16 * h + i] = r.x;
              acc[16 * h + i + 1] = r.y;
            }
          }
        }
        v_factor_prev = khd::scale_pow2(1.0f, -shift_v); // V was split as V * 2^shift
        // P (times 2^14) -> tensor memory as fp16 hi / lo, two keys per 32-bit column
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t hi[16], lo[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            // hi = the top 11 significant bits (exact in fp16), lo = fp16 of the rest
            const float p0 = __uint_as_float(sv[32 * h + 2 * i]);
            const float p1 = __uint_as_float(sv[32 * h + 2 * i + 1]);
            const float h0 = __uint_as_float(sv[32 * h + 2 * i] & 0xFFFFE000u);
            const float h1 = __uint_as_float(sv[32 * h + 2 * i + 1] & 0xFFFFE000u);
            hi[i] = half2_bits(__floats2half2_rn(h0, h1));
            lo[i] = half2_bits(__floats2half2_rn(p0 - h0, p1 - h1));
          }
          tmem_st_32x16(tmem_base + lane_base + col_p + 16 * h, hi);
          tmem_st_32x16(tmem_base + lane_base + col_p + 32 + 16 * h, lo);
        }
        tmem_st_wait();
        khd::tc_fence_before_sync();
        khd::mbar_arrive(bar_p_ready + 8 * g);
        ++tiles_done;
        first = false;
      }
      if (w + gridDim.x < items) fetch_item_shifts(w + gridDim.x);
      // this group's last product of the item
      if (ok && !first) {
        ok = khd::mbar_wait(bar_pv_full + 8 * g, (tiles_done - 1) & 1u, &s_abort, status,
                            khd::kStatusMmaWaitTimeout, 3000u);
        if (ok) {
          khd::tc_fence_after_sync();
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            uint32_t t[16];
            tmem_ld_32x16(tmem_base + lane_base + col_pv + 16 * h, t);
            khd::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[16 * h + i] = fmaf(__uint_as_float(t[i]), v_factor_prev, acc[16 * h + i]);
          }
        }
      }
      if (!ok) break;
      // park (max, sum, row) for the output warps, once they have read the previous item's
      if (n > 0)
        ok = khd::mbar_wait(bar_out_free, static_cast<uint32_t>((n - 1) & 1), &s_abort, status,
                            khd::kStatusEpilogueWaitTimeout, 5000u);
      if (!ok) break;
      s_row_m[g][row_in_tile] = m;
      s_row_l[g][row_in_tile] = l;
#pragma unroll
      for (int h = 0; h < 4; ++h)
        tmem_st_32x16(tmem_base + lane_base + col_out + 16 * h, *reinterpret_cast<const uint32_t(*)[16]>(&acc[16 * h]));
      tmem_st_wait();
      khd::tc_fence_before_sync();
      khd::mbar_arrive(bar_parked + 8 * g);
    }
    khd::tc_fence_before_sync();
  } else {
    registers_release<kRegsOutput>();
    // ---- output (warpgroup 3), one thread per query row: combine the two groups'
    //      parked rows of an item, 32 columns at a time: stage the finished half
    //      rows in shared memory (each warp its own 32 rows of 128 bytes: 16-byte
    //      chunk c of row r at chunk c ^ (r % 8), conflict-free both for a thread
    //      per row and for the row-major copy) and copy them out, four 128-byte
    //      half rows per warp instruction - to the other replicas too when there
    //      are any. ----------------------------------------------------------------------
    const int quad = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const int row_in_tile = quad * 32 + lane;
    constexpr int kHalfChunks = kHeadDim / 8; // 16-byte chunks in half a row
    float4 *staged = reinterpret_cast<float4 *>(smem_raw + (smem_scratch - khd::smem_u32(smem_raw))) +
                     quad * 32 * kHalfChunks; // this warp's 32 half rows
    bool ok = true;
    int n = 0;
    for (int64_t w = blockIdx.x; w < items && ok; w += gridDim.x, ++n) {
      const int64_t bh = w / q_tiles;
      const int q0 = static_cast<int>((w - bh * q_tiles) * kBQ);
      ok = khd::mbar_wait(bar_parked, static_cast<uint32_t>(n & 1), &s_abort, status,
                          khd::kStatusEpilogueWaitTimeout, 5001u) &&
           khd::mbar_wait(bar_parked + 8, static_cast<uint32_t>(n & 1), &s_abort, status,
                          khd::kStatusEpilogueWaitTimeout, 5002u);
      if (!ok) break;
      khd::tc_fence_after_sync();
      const float m0 = s_row_m[0][row_in_tile], l0 = s_row_l[0][row_in_tile];
      const float m1 = s_row_m[1][row_in_tile], l1 = s_row_l[1][row_in_tile];
      const float mt = fmaxf(m0, m1);
      float w0 = fast_exp2(m0 - mt), w1 = fast_exp2(m1 - mt); // a group without tiles parks max = -inf: weight 0
      const float inv = 1.0f / (l0 * w0 + l1 * w1);
      w0 *= inv;
      w1 *= inv;
      const int64_t first_row = bh * seq + q0;
      const int rows_here = (seq - q0 < kBQ) ? static_cast<int>(seq - q0) : kBQ;
      float4 *dst = reinterpret_cast<float4 *>(out + first_row * kHeadDim);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t a[16], b[16];
          tmem_ld_32x16(tmem_base + lane_base + kColOut0 + 32 * half + 16 * h, a);
          tmem_ld_32x16(tmem_base + lane_base + kColOut1 + 32 * half + 16 * h, b);
          khd::tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 4; ++c)
            staged[lane * kHalfChunks + ((4 * h + c) ^ (lane & 7))] =
                make_float4(__uint_as_float(a[4 * c + 0]) * w0 + __uint_as_float(b[4 * c + 0]) * w1,
                            __uint_as_float(a[4 * c + 1]) * w0 + __uint_as_float(b[4 * c + 1]) * w1,
                            __uint_as_float(a[4 * c + 2]) * w0 + __uint_as_float(b[4 * c + 2]) * w1,
                            __uint_as_float(a[4 * c + 3]) * w0 + __uint_as_float(b[4 * c + 3]) * w1);
        }
        if (half == 1) {
          khd::tc_fence_before_sync();
          khd::mbar_arrive(bar_out_free); // both parked rows and their (max, sum) are read
        }
        __syncwarp();
#pragma unroll 4
        for (int k = 0; k < kHalfChunks; ++k) {
          const int q = k * 32 + lane; // this warp's half rows, row-major
          const int r = q >> 3, c = q & 7;
          if (quad * 32 + r >= rows_here) break;
          const float4 v = staged[r * kHalfChunks + (c ^ (r & 7))];
          const int64_t at = static_cast<int64_t>(quad * 32 + r) * (kHeadDim / 4) + half * kHalfChunks + c;
          __stcs(dst + at, v);
          if (kGather) {
            const int64_t off = first_row * kHeadDim + at * 4;
            if (targets->multicast != nullptr) {
              multicast_store_float4(targets->multicast + off, v);
            } else {
              for (int d = 0; d < targets->count; ++d)
                if (d != targets->self) *reinterpret_cast<float4 *>(targets->peer[d] + off) = v;
            }
          }
        }
        __syncwarp(); // the staged half rows are free again
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

} // namespace

extern "C" __global__ void __launch_bounds__(kRegisterBoundThreads, 1)
attention(KH_MEMREF4(const float, q), KH_MEMREF4(const float, k), KH_MEMREF4(const float, v),
          KH_MEMREF4(float, o), const __grid_constant__ khd::TensorMap tm_q_hi,
          const __grid_constant__ khd::TensorMap tm_q_lo, const __grid_constant__ khd::TensorMap tm_k_hi,
          const __grid_constant__ khd::TensorMap tm_k_lo, const __grid_constant__ khd::TensorMap tm_vt_hi,
          const __grid_constant__ khd::TensorMap tm_vt_lo, const int *__restrict__ shifts, uint32_t *status) {
  (void)q_alloc; (void)q_ptr; (void)q_off; (void)q_size3; (void)q_stride0;
  (void)q_stride1; (void)q_stride2; (void)q_stride3;
  (void)k_alloc; (void)k_ptr; (void)k_off; (void)k_size0; (void)k_size1; (void)k_size2; (void)k_size3;
  (void)k_stride0; (void)k_stride1; (void)k_stride2; (void)k_stride3;
  (void)v_alloc; (void)v_ptr; (void)v_off; (void)v_size0; (void)v_size1; (void)v_size2; (void)v_size3;
  (void)v_stride0; (void)v_stride1; (void)v_stride2; (void)v_stride3;
  (void)o_size0; (void)o_size1; (void)o_size2; (void)o_size3; (void)o_stride0; (void)o_stride1;
  (void)o_stride2; (void)o_stride3; (void)o_alloc;
  attention_body<false, false>(q_size0 * q_size1, q_size2, KH_DATA(o), tm_q_hi, tm_q_lo, tm_k_hi, tm_k_lo, tm_vt_hi, tm_vt_lo, shifts,
                               status, 0, nullptr);
}

// The same for (batch, head) slices sharded over several GPUs, with the
// all-gather of the output fused in: `o` is this rank's slices inside its own
// replica of the whole output, and every finished tile is also sent to the
// other replicas (see GatherOut). The caller's barrier across ranks after the
// kernel makes the peers' stores visible.
extern "C" __global__ void __launch_bounds__(kRegisterBoundThreads, 1)
attention_allgather(KH_MEMREF4(const float, q), KH_MEMREF4(const float, k), KH_MEMREF4(const float, v),
                    KH_MEMREF4(float, o), const __grid_constant__ khd::TensorMap tm_q_hi,
                    const __grid_constant__ khd::TensorMap tm_q_lo, const __grid_constant__ khd::TensorMap tm_k_hi,
                    const __grid_constant__ khd::TensorMap tm_k_lo, const __grid_constant__ khd::TensorMap tm_vt_hi,
                    const __grid_constant__ khd::TensorMap tm_vt_lo, const int *__restrict__ shifts,
                    uint32_t *status, const __grid_constant__ GatherOut targets) {
  (void)q_alloc; (void)q_ptr; (void)q_off; (void)q_size3; (void)q_stride0;
  (void)q_stride1; (void)q_stride2; (void)q_stride3;
  (void)k_alloc; (void)k_ptr; (void)k_off; (void)k_size0; (void)k_size1; (void)k_size2; (void)k_size3;
  (void)k_stride0; (void)k_stride1; (void)k_stride2; (void)k_stride3;
  (void)v_alloc; (void)v_ptr; (void)v_off; (void)v_size0; (void)v_size1; (void)v_size2; (void)v_size3;
  (void)v_stride0; (void)v_stride1; (void)v_stride2; (void)v_stride3;
  (void)o_size0; (void)o_size1; (void)o_size2; (void)o_size3; (void)o_stride0; (void)o_stride1;
  (void)o_stride2; (void)o_stride3; (void)o_alloc;
  attention_body<true, false>(q_size0 * q_size1, q_size2, KH_DATA(o), tm_q_hi, tm_q_lo, tm_k_hi, tm_k_lo, tm_vt_hi, tm_vt_lo, shifts,
                              status, 0, &targets);
}

// `attention` for the shapes that need scores masked: the causal mask (shape key causal=1: query i
// attends to keys 0..i) and / or a seq that is not a multiple of 64. One more parameter: `causal`.
extern "C" __global__ void __launch_bounds__(kRegisterBoundThreads, 1)
attention_masked(KH_MEMREF4(const float, q), KH_MEMREF4(const float, k), KH_MEMREF4(const float, v),
                 KH_MEMREF4(float, o), const __grid_constant__ khd::TensorMap tm_q_hi,
                 const __grid_constant__ khd::TensorMap tm_q_lo, const __grid_constant__ khd::TensorMap tm_k_hi,
                 const __grid_constant__ khd::TensorMap tm_k_lo, const __grid_constant__ khd::TensorMap tm_vt_hi,
                 const __grid_constant__ khd::TensorMap tm_vt_lo, const int *__restrict__ shifts, uint32_t *status,
                 int causal) {
  (void)q_alloc; (void)q_ptr; (void)q_off; (void)q_size3; (void)q_stride0;
  (void)q_stride1; (void)q_stride2; (void)q_stride3;
  (void)k_alloc; (void)k_ptr; (void)k_off; (void)k_size0; (void)k_size1; (void)k_size2; (void)k_size3;
  (void)k_stride0; (void)k_stride1; (void)k_stride2; (void)k_stride3;
  (void)v_alloc; (void)v_ptr; (void)v_off; (void)v_size0; (void)v_size1; (void)v_size2; (void)v_size3;
  (void)v_stride0; (void)v_stride1; (void)v_stride2; (void)v_stride3;
  (void)o_size0; (void)o_size1; (void)o_size2; (void)o_size3; (void)o_stride0; (void)o_stride1;
  (void)o_stride2; (void)o_stride3; (void)o_alloc;
  attention_body<false, true>(q_size0 * q_size1, q_size2, KH_DATA(o), tm_q_hi, tm_q_lo, tm_k_hi, tm_k_lo, tm_vt_hi, tm_vt_lo, shifts,
                              status, causal, nullptr);
}
