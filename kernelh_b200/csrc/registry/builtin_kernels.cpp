// The seven kernel templates as registry records: shape validation (same keys
// and the same "which key is wrong" behaviour as the reference's templates,
// e.g. lib/dsl/kernels/gemm.cpp:119-132), launch geometry for B200, and the
// launch sequence. Work counts follow the reference's metric conventions
// (bench/harness/metrics.cpp:14-52).
#include "executor.hpp"
#include "registry.hpp"

#include <algorithm>
#include <cstring>
#include <stdexcept>

namespace kh {
namespace {

int64_t require_positive(const ShapeMap &shape, const char *kernel, const char *key) {
  auto it = shape.find(key);
  if (it == shape.end())
    throw std::runtime_error(std::string(kernel) + " template: shape attribute '" + key +
                             "' is required (pass --shape " + key + "=<size>)");
  if (it->second <= 0)
    throw std::runtime_error(std::string(kernel) + " template: shape attribute '" + key +
                             "' must be positive (got " + std::to_string(it->second) + ")");
  return it->second;
}

long sm_count(const DeviceLimits &l) {
  const long n = query_cu_count(l);
  return n > 0 ? n : (l.cu_count > 0 ? l.cu_count : 148);
}

// Persistent grid: `needed` blocks of work spread over whole waves of
// sms * per_sm resident blocks, so every block does the same number of trips.
unsigned balanced_grid(int64_t needed, long sms, int per_sm) {
  const int64_t resident = static_cast<int64_t>(sms) * per_sm;
  if (needed <= resident) return static_cast<unsigned>(std::max<int64_t>(needed, 1));
  const int64_t waves = (needed + resident - 1) / resident;
  return static_cast<unsigned>((needed + waves - 1) / waves);
}

// ---------------------------------------------------------------- elementwise
KernelPlan plan_vecadd(const ShapeMap &shape, const DeviceLimits &l) {
  const int64_t n = require_positive(shape, "vecadd", "n");
  KernelPlan p;
  p.kernel = "vecadd";
  p.shape = shape;
  p.tensors = {{"a", {n}, false}, {"b", {n}, false}, {"c", {n}, true}};
  LaunchStep s;
  s.entry = "vecadd";
  s.overlap_tail = true;
  s.block = {256, 1, 1};
  s.grid = {balanced_grid((n / 4 + 1023) / 1024, sm_count(l), 6), 1, 1}; // 4 float4 per thread per trip
  s.param_count = 15;
  p.steps = {s};
  p.work = 3.0 * static_cast<double>(n) * 4.0;
  return p;
}

Result<void> run_elementwise3(Executor &ex, const KernelPlan &p, const std::vector<void *> &b,
                              StreamHandle stream, const char *code_object) {
  auto fn = ex.function(code_object, p.steps[0].entry);
  if (!fn) return std::unexpected(fn.error());
  LaunchArgs args;
  for (size_t i = 0; i < 3; ++i) args.add_memref(b[i], p.tensors[i].shape);
  return ex.launch(*fn, p.steps[0], args, stream);
}

KernelPlan plan_fused_gelu(const ShapeMap &shape, const DeviceLimits &l) {
  int64_t n = 0;
  if (shape.count("n")) {
    n = shape.at("n");
  } else if (shape.count("rows") && shape.count("cols")) {
    n = shape.at("rows") * shape.at("cols");
    if (shape.at("rows") <= 0 || shape.at("cols") <= 0) n = 0;
  } else {
    throw std::runtime_error("fused_gelu template: shape requires 'n', or 'rows' AND 'cols' "
                             "(pass --shape n=<size> or --shape rows=R,cols=C)");
  }
  if (n <= 0) throw std::runtime_error("fused_gelu template: shape element count must be positive");
  const bool bias = shape.count("bias") && shape.at("bias") != 0;
  KernelPlan p;
  p.kernel = "fused_gelu";
  p.shape = shape;
  if (bias)
    p.tensors = {{"x", {n}, false}, {"bias", {n}, false}, {"out", {n}, true}};
  else
    p.tensors = {{"x", {n}, false}, {"tmp", {n}, false}, {"out", {n}, true}};
  LaunchStep s;
  s.entry = bias ? "fused_gelu_bias" : "fused_gelu";
  s.overlap_tail = true;
  s.block = {256, 1, 1};
  // Four float4 per thread and trip, the last trip predicated. Up to two trips' worth of work
  // runs as four blocks on every SM (measured best at the 2^22-element benchmark size: more
  // blocks than that only add idle trips, fewer leave the memory system short of requests);
  // beyond that, whole waves of five blocks per SM with equal trip counts.
  {
    const long sms = sm_count(l);
    const int64_t needed = (n / 4 + 1023) / 1024;
    s.grid = {needed <= 8 * sms ? static_cast<unsigned>(std::clamp<int64_t>(needed, 1, 4 * sms))
                                : balanced_grid(needed, sms, 5),
              1, 1};
  }
  s.param_count = 15;
  p.steps = {s};
  // The reference counts 3*n*4 bytes for this kernel although its fused form never
  // touches `tmp`; kept for comparability. The bias form really moves 3*n*4.
  p.work = 3.0 * static_cast<double>(n) * 4.0;
  return p;
}

// ---------------------------------------------------------------- row kernels
LaunchStep row_kernel_step(const char *entry, int64_t rows, int64_t cols, const DeviceLimits &l,
                           int params) {
  LaunchStep s;
  s.entry = entry;
  s.overlap_tail = true;
  s.param_count = params;
  const long sms = sm_count(l);
  if (cols % 4 == 0 && cols <= 1024) {
    // a warp per row; aim for one pass with the same number of rows on every SM
    const int64_t per_sm = (rows + sms - 1) / sms;
    if (per_sm <= 64) {
      const int64_t blocks_per_sm = (per_sm + 7) / 8;
      const int64_t warps = (per_sm + blocks_per_sm - 1) / blocks_per_sm;
      s.block = {static_cast<unsigned>(32 * warps), 1, 1};
      const int64_t needed = (rows + warps - 1) / warps;
      s.grid = {static_cast<unsigned>(std::min<int64_t>(needed, sms * blocks_per_sm)), 1, 1};
    } else {
      s.block = {256, 1, 1};
      s.grid = {static_cast<unsigned>(sms * 8), 1, 1};
    }
  } else {
    // the block per row (registers up to 8192 columns, generic beyond)
    s.block = {256, 1, 1};
    s.grid = {static_cast<unsigned>(std::min<int64_t>(rows, sms * 8)), 1, 1};
  }
  return s;
}

KernelPlan plan_rows(const char *kernel, const ShapeMap &shape, const DeviceLimits &l, bool affine) {
  if (!shape.count("rows") || !shape.count("cols"))
    throw std::runtime_error(std::string(kernel) + " template: shape attributes 'rows' and 'cols' "
                             "are required (pass --shape rows=R,cols=C)");
  const int64_t rows = shape.at("rows"), cols = shape.at("cols");
  if (rows <= 0 || cols <= 0)
    throw std::runtime_error(std::string(kernel) +
                             " template: shape attributes 'rows' and 'cols' must be positive");
  KernelPlan p;
  p.kernel = kernel;
  p.shape = shape;
  if (affine)
    p.tensors = {{"x", {rows, cols}, false}, {"gamma", {cols}, false}, {"beta", {cols}, false},
                 {"y", {rows, cols}, true}};
  else
    p.tensors = {{"x", {rows, cols}, false}, {"y", {rows, cols}, true}};
  p.steps = {row_kernel_step(kernel, rows, cols, l, affine ? 24 : 14)};
  p.work = 2.0 * static_cast<double>(rows) * static_cast<double>(cols) * 4.0 +
           (affine ? 2.0 * static_cast<double>(cols) * 4.0 : 0.0);
  return p;
}

Result<void> run_rows(Executor &ex, const KernelPlan &p, const std::vector<void *> &b,
                      StreamHandle stream) {
  auto fn = ex.function(p.kernel, p.steps[0].entry);
  if (!fn) return std::unexpected(fn.error());
  LaunchArgs args;
  for (size_t i = 0; i < p.tensors.size(); ++i) args.add_memref(b[i], p.tensors[i].shape);
  return ex.launch(*fn, p.steps[0], args, stream);
}

// ---------------------------------------------------------------- scan
// One block per SM: twelve compute warps and a look-back warp over tiles of
// 12 x 1024 elements held in four shared-memory tile buffers.
constexpr int64_t kScanTile = 12 * 1024;
constexpr int64_t kScanRow = 32; // floats per row of the tensor-map view
constexpr size_t kScanSmem = 4 * static_cast<size_t>(kScanTile) * 4 + 1024;

KernelPlan plan_scan(const ShapeMap &shape, const DeviceLimits &l) {
  const int64_t n = require_positive(shape, "scan", "n");
  KernelPlan p;
  p.kernel = "scan";
  p.shape = shape;
  p.tensors = {{"x", {n}, false}, {"y", {n}, true}};
  const int64_t tiles = (n + kScanTile - 1) / kScanTile;
  LaunchStep s;
  s.entry = "scan";
  s.block = {13 * 32, 1, 1};
  s.grid = {static_cast<unsigned>(std::min<int64_t>(tiles, sm_count(l))), 1, 1};
  s.dynamic_smem = kScanSmem;
  s.param_count = 15 + 2 + 2 + 1; // three descriptors, two scalars, two tensor maps, flags
  p.steps = {s};
  p.workspace_bytes = static_cast<size_t>(4 + 2 * tiles) * 8;
  p.work = 2.0 * static_cast<double>(n) * 4.0;
  return p;
}

// x or y seen as [n / 32 rows][32 floats] for the kernel's tensor-map copies; nullopt-like
// `false` when the buffer cannot be copied that way (the kernel then uses plain accesses).
bool scan_tensor_map(Executor &ex, const void *ptr, int64_t n, TensorMapBytes *out) {
  std::memset(out, 0, sizeof *out);
  if (ptr == nullptr || (reinterpret_cast<uintptr_t>(ptr) & 15u) != 0 || n < kScanRow) return false;
  TensorMapSpec t;
  t.global_address = ptr;
  t.rank = 2;
  t.elem_bytes = 4;
  t.dims[0] = static_cast<uint64_t>(kScanRow);
  t.dims[1] = static_cast<uint64_t>(n / kScanRow);
  t.strides_bytes[0] = static_cast<uint64_t>(kScanRow) * 4;
  t.box[0] = static_cast<uint32_t>(kScanRow);
  t.box[1] = 32;
  t.swizzle_bytes = 128;
  auto m = ex.backend().encode_tensor_map(t);
  if (!m) return false;
  *out = *m;
  return true;
}

// `spin_limit` 0 = the kernel's default; `tile_bias` 0 in production (see the kernel).
Result<void> launch_scan(Executor &ex, const KernelPlan &p, const std::vector<void *> &b, StreamHandle stream,
                         uint32_t spin_limit, uint32_t tile_bias) {
  auto fn = ex.function("scan", "scan");
  if (!fn) return std::unexpected(fn.error());
  const int64_t n = p.tensors[0].shape[0];
  const int64_t tiles = (n + kScanTile - 1) / kScanTile;
  auto state = ex.scan_state(tiles);
  if (!state) return std::unexpected(state.error());
  TensorMapBytes x_map, y_map;
  uint32_t flags = 0;
  if (scan_tensor_map(ex, b[0], n, &x_map)) flags |= 1u;
  if (scan_tensor_map(ex, b[1], n, &y_map)) flags |= 2u;
  LaunchArgs args;
  args.add_memref(b[0], {n});
  args.add_memref(b[1], {n});
  args.add_memref(*state, {static_cast<int64_t>(4 + 2 * tiles)});
  args.add_scalar<uint32_t>(spin_limit);
  args.add_scalar<uint32_t>(tile_bias);
  args.add_tensor_map(x_map);
  args.add_tensor_map(y_map);
  args.add_scalar<uint32_t>(flags);
  return ex.launch(*fn, p.steps[0], args, stream);
}

Result<void> run_scan(Executor &ex, const KernelPlan &p, const std::vector<void *> &b,
                      StreamHandle stream) {
  return launch_scan(ex, p, b, stream, 0u, 0u);
}

// ---------------------------------------------------------------- gemm
// Two-CTA clusters own 256 x 256 tiles of C; a CTA stages 128 rows of A and 128
// of the tile's B columns per 32-deep k-block (fp16 hi and lo of each).
constexpr int kGemmBM = 128, kGemmBN = 256, kGemmBK = 32, kGemmStages = 6;
constexpr size_t kGemmStageBytes = 4 * (kGemmBM * kGemmBK * 2);

// Scratch of one product, every part 256-byte aligned: the fp16 hi / lo splits
// of A (m x kp) and B^T (n x kp), the scale exponents of A's rows and B's
// columns, and the column maxima of B.
struct GemmScratch {
  size_t a_hi, a_lo, b_hi, b_lo, a_shift, b_amax, b_shift, total;
};
GemmScratch gemm_scratch(int64_t m, int64_t n, int64_t kp) {
  const auto pad = [](size_t v) { return (v + 255) / 256 * 256; };
  GemmScratch g{};
  size_t at = 0;
  const auto take = [&](size_t bytes) {
    const size_t here = at;
    at += pad(bytes);
    return here;
  };
  g.a_hi = take(static_cast<size_t>(m * kp) * 2);
  g.a_lo = take(static_cast<size_t>(m * kp) * 2);
  g.b_hi = take(static_cast<size_t>(n * kp) * 2);
  g.b_lo = take(static_cast<size_t>(n * kp) * 2);
  g.a_shift = take(static_cast<size_t>(m) * 4);
  g.b_amax = take(static_cast<size_t>(n) * 4);
  g.b_shift = take(static_cast<size_t>(n) * 4);
  g.total = at;
  return g;
}

// The cluster size gemm_prep_b is launched with (8 or 16 CTAs) and the rows of B one CTA then
// holds (a multiple of 256); {0, 0} when the one-pass preparation does not apply: rows of B must
// be 16-byte multiples for the tensor map, and a strip must fit the shared memory of a cluster.
constexpr int kPrepCols = 32, kPrepBoxRows = 64, kPrepGroupRows = 256, kPrepMaxGroups = 6;
struct PrepShape {
  int cluster;
  int64_t rows;
};
PrepShape prep_b_shape(int64_t n, int64_t k) {
  if (n % 4 != 0) return {0, 0};
  const int64_t kp = (k + kGemmBK - 1) / kGemmBK * kGemmBK;
  for (int cluster : {8, 16}) { // the larger (not portable, opt-in) size only for strips eight CTAs cannot hold three to an SM
    const int64_t rows = ((kp + cluster - 1) / cluster + kPrepGroupRows - 1) / kPrepGroupRows * kPrepGroupRows;
    if (rows / kPrepGroupRows <= (cluster == 8 ? 2 : kPrepMaxGroups)) return {cluster, rows};
  }
  return {0, 0};
}
int64_t prep_b_rows_per_cta(int64_t n, int64_t k) { return prep_b_shape(n, k).rows; }
LaunchStep gemm_prep_b_step(int64_t n, int64_t k) {
  const PrepShape shape = prep_b_shape(n, k);
  LaunchStep s;
  s.entry = "gemm_prep_b";
  s.block = {256, 1, 1};
  s.cluster = static_cast<unsigned>(shape.cluster);
  s.grid = {static_cast<unsigned>(((n + kPrepCols - 1) / kPrepCols) * shape.cluster), 1, 1};
  // the CTA's rows of the strip (the boxes of B^T are built in place over them) and alignment slack
  s.dynamic_smem = static_cast<size_t>(shape.rows) * kPrepCols * 4 + 1024;
  s.param_count = 7 + 3 + 3;
  return s;
}

// The launches of one m x n x k product: split A, prepare B (one pass: gemm_prep_b; or,
// where that does not apply, column maxima of B and then the split of B^T), multiply.
// The list always has the two-pass steps at [1] and [2]; `fused` tells which are used.
std::vector<LaunchStep> gemm_steps(int64_t m, int64_t n, int64_t k, const DeviceLimits &l) {
  const int64_t kp = (k + kGemmBK - 1) / kGemmBK * kGemmBK;
  const long sms = sm_count(l);
  LaunchStep sa;
  sa.entry = "gemm_split_a";
  sa.block = {256, 1, 1};
  // a warp per row for short rows (8 rows per block); the whole block for long ones, which
  // are staged in two shared-memory row buffers when a row is at most 32 KiB
  const bool staged = kp > 1024 && k % 4 == 0 && k * 4 <= 32768;
  sa.grid = {balanced_grid(kp <= 1024 ? (m + 7) / 8 : m, sms, 3), 1, 1};
  sa.dynamic_smem = staged ? static_cast<size_t>(k) * 8 : 0;
  sa.param_count = 7 + 7;
  LaunchStep cm;
  cm.entry = "gemm_colmax_b";
  cm.block = {256, 1, 1};
  cm.grid = {balanced_grid(((n + 1023) / 1024) * ((k + 63) / 64), sms, 8), 1, 1};
  cm.param_count = 7 + 1;
  LaunchStep sb;
  sb.entry = "gemm_split_bt";
  sb.block = {256, 1, 1};
  sb.grid = {balanced_grid(((n + 127) / 128) * ((kp + 63) / 64), sms, 6), 1, 1}; // 64 x 128 tiles
  sb.param_count = 7 + 5;
  LaunchStep g;
  g.block = {320, 1, 1};
  g.cluster = 2;
  // persistent: one cluster per pair of SMs walks the 256 x BN tiles of C. BN = 256 unless the
  // product is so small that wide tiles leave at least half of the clusters without any tile
  // (1000^3: 16 wide tiles on 74 clusters, 32 narrow ones). A narrow tile takes 0.74 of a wide
  // tile's time, not half (measured at 8192^3: 2.74 ms against 1.86 on constant data: the issue
  // rate of one MMA thread and the A traffic per flop), so it never pays for filling the last wave
  // of a large product. KERNELH_GEMM_TILE_N = 128 / 256 forces one (for measurements).
  const int64_t clusters = std::max<long>(sms / 2, 1);
  const int64_t tiles_m = (m + 2 * kGemmBM - 1) / (2 * kGemmBM);
  const int64_t tiles256 = tiles_m * ((n + 255) / 256), tiles128 = tiles_m * ((n + 127) / 128);
  const int64_t cost256 = 4 * ((tiles256 + clusters - 1) / clusters), cost128 = 3 * ((tiles128 + clusters - 1) / clusters);
  bool narrow = cost128 < cost256;
  if (const char *forced = std::getenv("KERNELH_GEMM_TILE_N")) {
    if (std::strcmp(forced, "128") == 0) narrow = true;
    if (std::strcmp(forced, "256") == 0) narrow = false;
  }
  g.entry = narrow ? "gemm_n128" : "gemm";
  const int64_t tiles = narrow ? tiles128 : tiles256;
  g.grid = {static_cast<unsigned>(2 * std::min<int64_t>(tiles, clusters)), 1, 1};
  g.dynamic_smem = kGemmStages * kGemmStageBytes + 1024;
  g.param_count = 21 + 4 + 2 + 2 + 1 + 1 + 3;
  g.tmem_columns = 512;
  return {sa, cm, sb, g};
}

KernelPlan plan_gemm(const ShapeMap &shape, const DeviceLimits &l) {
  const int64_t m = require_positive(shape, "gemm", "m");
  const int64_t n = require_positive(shape, "gemm", "n");
  const int64_t k = require_positive(shape, "gemm", "k");
  KernelPlan p;
  p.kernel = "gemm";
  p.shape = shape;
  p.tensors = {{"A", {m, k}, false}, {"B", {k, n}, false}, {"C", {m, n}, true}};
  const int64_t kp = (k + kGemmBK - 1) / kGemmBK * kGemmBK;
  p.workspace_bytes = gemm_scratch(m, n, kp).total;
  p.steps = gemm_steps(m, n, k, l);
  if (prep_b_rows_per_cta(n, k) > 0) // one pass over B instead of two (taken when B is 16-byte aligned)
    p.steps = {p.steps[0], gemm_prep_b_step(n, k), p.steps[3]};
  p.work = 2.0 * static_cast<double>(m) * static_cast<double>(n) * static_cast<double>(k);
  p.work_is_flops = true;
  return p;
}

// Destinations of gemm_allgather's fused all-gather; layout shared with the kernel.
struct GatherTargets {
  float *base[8];
  int count;
  int self;
  int64_t row_offset;
  float *multicast;
  unsigned long long *flags[8]; // arrival flags of every rank as mapped here; used when epoch != 0
  unsigned long long epoch;
  unsigned int *finished;       // this GPU's finished-CTA counter (in the executor's status buffer)
  int wait_later;               // signal only; await_arrivals waits (on the executor's second stream)
};
static_assert(sizeof(GatherTargets) == 176 && sizeof(GatherTargets) <= LaunchArgs::kMaxStructBytes,
              "GatherTargets is passed by value: its layout is shared with kernels/gemm.cu");

// One product being enqueued: sizes, scratch and the entry points.
struct GemmJob {
  Executor &ex;
  int64_t m, n, k, kp;
  GemmScratch lay;
  char *base = nullptr; // scratch
  KernelFunction split_a, colmax_b, split_bt, prep_b, multiply, multiply_gather, multiply_n128, multiply_gather_n128;
  float alpha = 1.f, beta = 0.f; // C = alpha * A.B + beta * C (1 and 0: a plain store that never reads C)
  uint64_t at(size_t off) const { return reinterpret_cast<uint64_t>(base + off); }
};

Result<GemmJob> gemm_job(Executor &ex, int64_t m, int64_t n, int64_t k) {
  GemmJob j{ex, m, n, k, (k + kGemmBK - 1) / kGemmBK * kGemmBK, {}, nullptr, {}, {}, {}, {}, {}, {}, {}, {}};
  j.lay = gemm_scratch(m, n, j.kp);
  auto ws = ex.workspace(j.lay.total);
  if (!ws) return std::unexpected(ws.error());
  j.base = static_cast<char *>(*ws);
  const std::pair<const char *, KernelFunction *> entries[] = {{"gemm_split_a", &j.split_a},
                                                               {"gemm_colmax_b", &j.colmax_b},
                                                               {"gemm_split_bt", &j.split_bt},
                                                               {"gemm_prep_b", &j.prep_b},
                                                               {"gemm", &j.multiply},
                                                               {"gemm_allgather", &j.multiply_gather},
                                                               {"gemm_n128", &j.multiply_n128},
                                                               {"gemm_allgather_n128", &j.multiply_gather_n128}};
  for (const auto &[name, slot] : entries) {
    auto f = ex.function("gemm", name);
    if (!f) return std::unexpected(f.error());
    *slot = *f;
  }
  return j;
}

// Exponents and the fp16 splits of B^T: in one pass over B (gemm_prep_b) when B is 16-byte
// aligned and its strips fit, else column maxima first and the split after. `clear_maxima`:
// zero the maxima of the two-pass form here (otherwise the gemm_split_a launched before did).
Result<void> gemm_enqueue_b(const GemmJob &j, const void *b_dev, StreamHandle stream, bool clear_maxima) {
  const int64_t rows_per_cta = prep_b_rows_per_cta(j.n, j.k);
  if (rows_per_cta > 0 && first_misaligned16({{"B", b_dev}}) == nullptr) {
    TensorMapSpec in;
    in.global_address = b_dev;
    in.rank = 2;
    in.elem_bytes = 4;
    in.dims[0] = static_cast<uint64_t>(j.n);
    in.dims[1] = static_cast<uint64_t>(j.k);
    in.strides_bytes[0] = static_cast<uint64_t>(j.n) * 4;
    in.box[0] = kPrepCols;
    in.box[1] = kPrepBoxRows;
    in.swizzle_bytes = 128;
    auto t_b = j.ex.backend().encode_tensor_map(in);
    if (!t_b) return std::unexpected(t_b.error());
    const auto out_map = [&](size_t offset) {
      TensorMapSpec o;
      o.global_address = j.base + offset;
      o.rank = 2;
      o.elem_bytes = 2;
      o.dims[0] = static_cast<uint64_t>(j.kp);
      o.dims[1] = static_cast<uint64_t>(j.n);
      o.strides_bytes[0] = static_cast<uint64_t>(j.kp) * 2;
      o.box[0] = kPrepBoxRows; // 64 k-values: one 128-byte swizzle row
      o.box[1] = kPrepCols;
      o.swizzle_bytes = 128;
      return j.ex.backend().encode_tensor_map(o);
    };
    auto t_hi = out_map(j.lay.b_hi);
    if (!t_hi) return std::unexpected(t_hi.error());
    auto t_lo = out_map(j.lay.b_lo);
    if (!t_lo) return std::unexpected(t_lo.error());
    LaunchArgs args;
    args.add_memref(const_cast<void *>(b_dev), {j.k, j.n});
    args.add_tensor_map(*t_b);
    args.add_tensor_map(*t_hi);
    args.add_tensor_map(*t_lo);
    args.add_scalar<uint64_t>(j.at(j.lay.b_shift));
    args.add_scalar<int64_t>(rows_per_cta);
    args.add_scalar<uint64_t>(reinterpret_cast<uint64_t>(j.ex.status_word()));
    return j.ex.launch(j.prep_b, gemm_prep_b_step(j.n, j.k), args, stream);
  }
  const std::vector<LaunchStep> steps = gemm_steps(j.m, j.n, j.k, j.ex.limits());
  if (clear_maxima)
    if (auto r = j.ex.backend().memset32_async(j.base + j.lay.b_amax, 0, static_cast<size_t>(j.n), stream); !r)
      return r;
  {
    LaunchArgs args;
    args.add_memref(const_cast<void *>(b_dev), {j.k, j.n});
    args.add_scalar<uint64_t>(j.at(j.lay.b_amax));
    if (auto r = j.ex.launch(j.colmax_b, steps[1], args, stream); !r) return r;
  }
  LaunchArgs args;
  args.add_memref(const_cast<void *>(b_dev), {j.k, j.n});
  args.add_scalar<uint64_t>(j.at(j.lay.b_hi));
  args.add_scalar<uint64_t>(j.at(j.lay.b_lo));
  args.add_scalar<uint64_t>(j.at(j.lay.b_amax));
  args.add_scalar<uint64_t>(j.at(j.lay.b_shift));
  args.add_scalar<int64_t>(j.kp);
  return j.ex.launch(j.split_bt, steps[2], args, stream);
}

// Exponents and fp16 splits of rows [row0, row0 + rows) of A, read from `a_rows`.
// `clear_cols` > 0 also zeroes that many column maxima of B for a later gemm_enqueue_b.
Result<void> gemm_enqueue_a(const GemmJob &j, const void *a_rows, int64_t row0, int64_t rows,
                            const LaunchStep &step, StreamHandle stream, int64_t clear_cols) {
  LaunchArgs args;
  args.add_memref(const_cast<void *>(a_rows), {rows, j.k});
  args.add_scalar<uint64_t>(j.at(j.lay.a_hi + static_cast<size_t>(row0 * j.kp) * 2));
  args.add_scalar<uint64_t>(j.at(j.lay.a_lo + static_cast<size_t>(row0 * j.kp) * 2));
  args.add_scalar<uint64_t>(j.at(j.lay.a_shift + static_cast<size_t>(row0) * 4));
  args.add_scalar<uint64_t>(j.at(j.lay.b_amax));
  args.add_scalar<int64_t>(clear_cols);
  args.add_scalar<int64_t>(j.kp);
  args.add_scalar<uint64_t>(reinterpret_cast<uint64_t>(j.ex.status_word()));
  return j.ex.launch(j.split_a, step, args, stream);
}

// C rows [row0, row0 + rows) = (split rows of A) . (split B): `c_rows` is where
// row `row0` of C goes (ignored when gathering).
Result<void> gemm_enqueue_multiply(const GemmJob &j, const void *a_rows, const void *b_dev, void *c_rows,
                                   int64_t row0, int64_t rows, LaunchStep step, StreamHandle stream,
                                   const GatherTargets *gather) {
  const bool narrow = step.entry == "gemm_n128"; // 256 x 128 tiles: a CTA stages 64 columns of B per k-block
  auto make_map = [&](size_t offset, int64_t map_rows, uint32_t box_rows = kGemmBM) {
    TensorMapSpec s;
    s.global_address = j.base + offset;
    s.rank = 2;
    s.elem_bytes = 2;
    s.dims[0] = static_cast<uint64_t>(j.kp);
    s.dims[1] = static_cast<uint64_t>(map_rows);
    s.strides_bytes[0] = static_cast<uint64_t>(j.kp) * 2;
    s.box[0] = kGemmBK;
    s.box[1] = box_rows; // 128 rows of A, or this CTA's half of the tile's columns of B
    s.swizzle_bytes = 64;
    return j.ex.backend().encode_tensor_map(s);
  };
  const size_t a_off = static_cast<size_t>(row0 * j.kp) * 2;
  auto t_ah = make_map(j.lay.a_hi + a_off, rows);
  if (!t_ah) return std::unexpected(t_ah.error());
  auto t_al = make_map(j.lay.a_lo + a_off, rows);
  if (!t_al) return std::unexpected(t_al.error());
  auto t_bh = make_map(j.lay.b_hi, j.n, narrow ? 64u : 128u);
  if (!t_bh) return std::unexpected(t_bh.error());
  auto t_bl = make_map(j.lay.b_lo, j.n, narrow ? 64u : 128u);
  if (!t_bl) return std::unexpected(t_bl.error());

  LaunchArgs args;
  args.add_memref(const_cast<void *>(a_rows), {rows, j.k});
  args.add_memref(const_cast<void *>(b_dev), {j.k, j.n});
  if (!gather) args.add_memref(c_rows, {rows, j.n});
  args.add_tensor_map(*t_ah);
  args.add_tensor_map(*t_al);
  args.add_tensor_map(*t_bh);
  args.add_tensor_map(*t_bl);
  args.add_scalar<int64_t>(j.kp / kGemmBK);
  args.add_scalar<uint64_t>(reinterpret_cast<uint64_t>(j.ex.status_word()));
  args.add_scalar<uint64_t>(j.at(j.lay.a_shift + static_cast<size_t>(row0) * 4));
  args.add_scalar<uint64_t>(j.at(j.lay.b_shift));
  // tile rows per rasterisation group; 0 = the kernel's default. KERNELH_GEMM_RASTER overrides (measurements).
  int64_t raster = 0;
  if (const char *forced = std::getenv("KERNELH_GEMM_RASTER")) raster = std::atoll(forced);
  args.add_scalar<int64_t>(raster);
  uint32_t alpha_bits, beta_bits;
  std::memcpy(&alpha_bits, &j.alpha, 4);
  std::memcpy(&beta_bits, &j.beta, 4);
  args.add_scalar<uint64_t>(static_cast<uint64_t>(alpha_bits) | (static_cast<uint64_t>(beta_bits) << 32));
  // Tiles done as two units, half of K each, by two clusters at once (partial sums meet in scratch):
  //  - at the TAIL: the last, partly filled wave of clusters, when it holds at most half a wave of tiles
  //    and there is a full wave before it; it then takes half as long (2048 x 8192 x 8192, the 4-GPU
  //    shard: 3.46 waves are paid as 3.5 instead of 4);
  //  - at the HEAD, only with the fused all-gather of a short shard (fewer than 2.5 waves of tiles) whose
  //    traffic into every GPU, started after the first wave, would outlast the tensor work: half a wave of
  //    tiles, so that the first tiles are finished, and NVLink starts, after half a tile's time; taken
  //    only when it costs no wave (1024 x 8192 x 8192, the 8-GPU shard: 0.5 + 1 + 0.5 waves instead of
  //    1 + 1, with the first push at 0.5 instead of 1).
  // The meeting flags are zeroed before every such launch. KERNELH_GEMM_SPLIT_TAIL=0 switches both off.
  void *partials = nullptr, *partial_flags = nullptr;
  int64_t split_plan = 0;
  {
    const int64_t clusters = step.grid.x / 2;
    const int64_t tile_cols = narrow ? 128 : 256;
    const int64_t tiles = ((rows + 2 * kGemmBM - 1) / (2 * kGemmBM)) * ((j.n + tile_cols - 1) / tile_cols);
    const int64_t k_blocks = j.kp / kGemmBK;
    const char *off = std::getenv("KERNELH_GEMM_SPLIT_TAIL");
    const bool allowed = k_blocks % 16 == 0 && !(off && off[0] == '0');
    const auto tail_of = [&](int64_t t) { // tiles of the last wave worth splitting, else 0
      const int64_t left = t % clusters;
      return (t > clusters && left > 0 && 2 * left <= clusters) ? left : int64_t{0};
    };
    const auto half_waves = [&](int64_t t) { // cost of t tiles in half waves, with the tail rule
      const int64_t left = t % clusters;
      return 2 * (t / clusters) + (left == 0 ? 0 : (tail_of(t) > 0 ? 1 : 2));
    };
    int64_t head = 0;
    if (allowed && gather != nullptr && tiles > clusters) {
      const int64_t candidate = clusters / 2;
      const char *force = std::getenv("KERNELH_GEMM_SPLIT_HEAD"); // "0" / "1": measurements
      // Is the launch bound by what flows INTO this GPU? Every other rank sends a shard like this one;
      // nothing can leave before the first tiles are done. Measured on this hardware: 770 GB/s into a
      // GPU over NVLink, 0.153 ms for a wave of 256 x 256 x 8192 tiles (where the all-gather hides
      // under the tensor work, splitting the head only costs: 0.491 against 0.475 ms on 4 GPUs).
      const double wave_ms = 0.153 * static_cast<double>(k_blocks) / 256.0 * (narrow ? 0.74 : 1.0);
      const double ingress_ms = static_cast<double>(gather->count - 1) * static_cast<double>(rows) *
                                static_cast<double>(j.n) * 4.0 / 770e6;
      const bool ingress_bound = wave_ms + ingress_ms > 0.5 * static_cast<double>(half_waves(tiles)) * wave_ms;
      const bool pays = 2 * tiles < 5 * clusters && ingress_bound && 1 + half_waves(tiles - candidate) <= half_waves(tiles);
      if ((pays && !(force && force[0] == '0')) || (force && force[0] == '1')) head = candidate;
    }
    const int64_t tail = allowed ? tail_of(tiles - head) : 0;
    if (head + tail > 0) {
      auto scratch = j.ex.gemm_partials(static_cast<size_t>(head + tail) * 2 * kGemmBM * static_cast<size_t>(tile_cols) * 4,
                                        static_cast<size_t>(head + tail) * 2 * 2 * 4);
      if (!scratch) return std::unexpected(scratch.error());
      partials = scratch->first;
      partial_flags = scratch->second;
      split_plan = head | (tail << 32);
      if (auto r = j.ex.backend().memset32_async(partial_flags, 0, static_cast<size_t>(head + tail) * 4, stream); !r) return r;
    }
  }
  args.add_scalar<uint64_t>(reinterpret_cast<uint64_t>(partials));
  args.add_scalar<uint64_t>(reinterpret_cast<uint64_t>(partial_flags));
  args.add_scalar<int64_t>(split_plan);
  if (gather) {
    args.add_struct_bytes(gather, sizeof *gather);
    step.entry = narrow ? "gemm_allgather_n128" : "gemm_allgather";
    // a wait for the previous launch's peers that is still running beside this step's preparation:
    // the tiles of this launch go out only after it (the peers have then taken the previous ones in)
    if (auto r = j.ex.join_arrival_wait(stream); !r) return r;
  }
  const KernelFunction &fn = gather ? (narrow ? j.multiply_gather_n128 : j.multiply_gather)
                                    : (narrow ? j.multiply_n128 : j.multiply);
  return j.ex.launch(fn, step, args, stream);
}

Result<void> launch_gemm(Executor &ex, const KernelPlan &p, const std::vector<void *> &b,
                         StreamHandle stream, const GatherTargets *gather) {
  const int64_t m = p.tensors[0].shape[0], k = p.tensors[0].shape[1], n = p.tensors[1].shape[1];
  auto job = gemm_job(ex, m, n, k);
  if (!job) return std::unexpected(job.error());
  if (auto r = gemm_enqueue_a(*job, b[0], 0, m, p.steps[0], stream, n); !r) return r;
  if (auto r = gemm_enqueue_b(*job, b[1], stream, false); !r) return r;
  return gemm_enqueue_multiply(*job, b[0], b[1], gather ? nullptr : b[2], 0, m, p.steps.back(), stream, gather);
}

Result<void> run_gemm(Executor &ex, const KernelPlan &p, const std::vector<void *> &b,
                      StreamHandle stream) {
  return launch_gemm(ex, p, b, stream, nullptr);
}

} // namespace

// C = alpha * A.B + beta * C: the scaled store of the gemm epilogue (beta = 0 never reads C).
Result<void> run_gemm_scaled(Executor &ex, const void *a, const void *b, void *c, int64_t m, int64_t n, int64_t k,
                             float alpha, float beta, StreamHandle stream) {
  KernelPlan p;
  try {
    p = plan_gemm({{"m", m}, {"n", n}, {"k", k}}, ex.limits());
  } catch (const std::exception &e) {
    return fail(2, e.what());
  }
  auto job = gemm_job(ex, m, n, k);
  if (!job) return std::unexpected(job.error());
  job->alpha = alpha;
  job->beta = beta;
  if (auto r = gemm_enqueue_a(*job, a, 0, m, p.steps[0], stream, n); !r) return r;
  if (auto r = gemm_enqueue_b(*job, b, stream, false); !r) return r;
  return gemm_enqueue_multiply(*job, a, b, c, 0, m, p.steps.back(), stream, nullptr);
}

namespace {

// Host-buffer form of the product, pipelined over PCIe: B goes up first and is
// split; A then goes up in row blocks, and while block i+1 is on the wire,
// block i is split and multiplied and the finished rows of C of block i-1 go
// back down (the two directions of the link run at once). `dev` are device
// staging buffers for A, B and C.
// Row blocks of the host-buffer product: about eight blocks of whole 256-row cluster tiles
// (sixteen equal ones measured slower: more launches and tensor maps per step than the shorter tail
// saves), except at the two ends. The LAST block is cut again into a half and two quarters: what
// follows the last upload - that block's split, product and the trip of its rows of C back - is the
// part of the step nothing overlaps, and it shrinks with the block. The FIRST block is cut the same
// way, smallest first: the downloads of C take as long as the uploads of A, and they cannot start
// before the first block's rows are up and multiplied.
std::vector<std::pair<int64_t, int64_t>> host_row_blocks(int64_t m) {
  const int64_t block_rows = std::max<int64_t>(256, ((m + 7) / 8 + 255) / 256 * 256);
  std::vector<std::pair<int64_t, int64_t>> blocks;
  for (int64_t row0 = 0; row0 < m; row0 += block_rows) blocks.push_back({row0, std::min(block_rows, m - row0)});
  const auto [last0, last_rows] = blocks.back();
  if (blocks.size() > 1 && last_rows >= 1024 && last_rows % 1024 == 0) {
    blocks.pop_back();
    blocks.push_back({last0, last_rows / 2});
    blocks.push_back({last0 + last_rows / 2, last_rows / 4});
    blocks.push_back({last0 + 3 * last_rows / 4, last_rows / 4});
  }
  const char *head = std::getenv("KERNELH_HOST_BLOCKS_HEAD"); // "0": the first block stays whole (measurements)
  if (blocks.size() > 4 && block_rows >= 1024 && block_rows % 1024 == 0 && !(head && head[0] == '0')) {
    blocks.erase(blocks.begin());
    blocks.insert(blocks.begin(), {{0, block_rows / 4}, {block_rows / 4, block_rows / 4}, {block_rows / 2, block_rows / 2}});
  }
  return blocks;
}

Result<void> run_gemm_host(Executor &ex, const KernelPlan &p, const std::vector<void *> &host,
                           const std::vector<void *> &dev, const HostStreams &hs) {
  const int64_t m = p.tensors[0].shape[0], k = p.tensors[0].shape[1], n = p.tensors[1].shape[1];
  Backend &be = ex.backend();
  auto job = gemm_job(ex, m, n, k);
  if (!job) return std::unexpected(job.error());
  const std::vector<std::pair<int64_t, int64_t>> blocks = host_row_blocks(m);
  std::vector<EventHandle> events;
  const auto fresh_event = [&]() -> Result<EventHandle> {
    auto e = be.event_create();
    if (e) events.push_back(*e);
    return e;
  };
  const auto body = [&]() -> Result<void> {
    if (host[1] != nullptr)
      if (auto r = be.memcpy_h2d_async(dev[1], host[1], static_cast<size_t>(k * n) * 4, hs.in); !r) return r;
    auto b_up = fresh_event();
    if (!b_up) return std::unexpected(b_up.error());
    if (auto r = be.event_record(*b_up, hs.in); !r) return r;
    if (auto r = be.stream_wait_event(hs.compute, *b_up); !r) return r;
    if (auto r = gemm_enqueue_b(*job, dev[1], hs.compute, true); !r) return r;
    for (const auto &[row0, rows] : blocks) {
      char *a_rows = static_cast<char *>(dev[0]) + static_cast<size_t>(row0 * k) * 4;
      char *c_rows = static_cast<char *>(dev[2]) + static_cast<size_t>(row0 * n) * 4;
      if (host[0] != nullptr)
        if (auto r = be.memcpy_h2d_async(a_rows, static_cast<const char *>(host[0]) + static_cast<size_t>(row0 * k) * 4,
                                         static_cast<size_t>(rows * k) * 4, hs.in);
            !r)
          return r;
      auto a_up = fresh_event();
      if (!a_up) return std::unexpected(a_up.error());
      if (auto r = be.event_record(*a_up, hs.in); !r) return r;
      if (auto r = be.stream_wait_event(hs.compute, *a_up); !r) return r;
      const std::vector<LaunchStep> steps = gemm_steps(rows, n, k, ex.limits());
      if (auto r = gemm_enqueue_a(*job, a_rows, row0, rows, steps[0], hs.compute, 0); !r) return r;
      if (auto r = gemm_enqueue_multiply(*job, a_rows, dev[1], c_rows, row0, rows, steps[3], hs.compute, nullptr); !r)
        return r;
      auto c_done = fresh_event();
      if (!c_done) return std::unexpected(c_done.error());
      if (auto r = be.event_record(*c_done, hs.compute); !r) return r;
      if (auto r = be.stream_wait_event(hs.out, *c_done); !r) return r;
      if (host[2] != nullptr)
        if (auto r = be.memcpy_d2h_async(static_cast<char *>(host[2]) + static_cast<size_t>(row0 * n) * 4, c_rows,
                                         static_cast<size_t>(rows * n) * 4, hs.out);
            !r)
          return r;
    }
    return {};
  };
  Result<void> enqueued = body();
  // drain all three streams whatever happened, then report the first failure
  Result<void> s_in = be.stream_synchronize(hs.in);
  Result<void> s_compute = ex.synchronize(hs.compute);
  Result<void> s_out = be.stream_synchronize(hs.out);
  for (EventHandle e : events) (void)be.event_destroy(e);
  if (!enqueued) return enqueued;
  if (!s_compute) return s_compute;
  if (!s_in) return s_in;
  return s_out;
}

} // namespace

// The M-row-sharded product with the all-gather fused into the epilogue:
// `a_shard` is this rank's (m_shard x k) rows of A, `b` the whole B, and
// `replicas[i]` the address, valid on this device, of rank i's full C.
Result<void> run_gemm_allgather(Executor &ex, const void *a_shard, const void *b,
                                const std::vector<void *> &replicas, void *multicast, int rank,
                                int world, int64_t m_shard, int64_t n, int64_t k, StreamHandle stream) {
  if (world < 1 || world > 8)
    return fail(2, "gemm_allgather: between 1 and 8 ranks are supported, got " + std::to_string(world));
  if (static_cast<int>(replicas.size()) != world)
    return fail(2, "gemm_allgather: " + std::to_string(world) + " C replicas expected, got " +
                       std::to_string(replicas.size()));
  if (rank < 0 || rank >= world)
    return fail(2, "gemm_allgather: rank " + std::to_string(rank) + " is outside the replica list");
  KernelPlan plan;
  try {
    plan = plan_gemm({{"m", m_shard}, {"n", n}, {"k", k}}, ex.limits());
  } catch (const std::exception &e) {
    return fail(2, e.what());
  }
  GatherTargets t{};
  t.count = world;
  t.multicast = static_cast<float *>(multicast);
  // the epilogue's pushes are multimem.st.v4 / float4 peer stores: no scalar path for the bases
  if (first_misaligned16({{"C multicast address", multicast}}))
    return fail(2, "gemm_allgather: the C multicast address is not 16-byte aligned");
  for (int i = 0; i < world; ++i) {
    // with a multicast address only this rank's own replica is stored to directly
    if (replicas[i] == nullptr && (multicast == nullptr || i == rank))
      return fail(2, "gemm_allgather: null C replica pointer");
    if (first_misaligned16({{"C replica", replicas[i]}}))
      return fail(2, "gemm_allgather: C replica " + std::to_string(i) + " is not 16-byte aligned");
    t.base[i] = static_cast<float *>(replicas[i]);
  }
  t.self = rank;
  t.row_offset = static_cast<int64_t>(rank) * m_shard;
  // armed by Executor::arm_arrival_flags for this one launch: the kernel then ends with the barrier itself
  if (ArrivalFlags armed = ex.take_arrival_flags(); armed.epoch != 0) {
    if (static_cast<int>(armed.flags.size()) != world)
      return fail(2, "gemm_allgather: " + std::to_string(world) + " arrival-flag arrays expected, got " +
                         std::to_string(armed.flags.size()));
    for (int i = 0; i < world; ++i) {
      if (armed.flags[i] == nullptr || (reinterpret_cast<uintptr_t>(armed.flags[i]) & 7u) != 0)
        return fail(2, "gemm_allgather: arrival-flag array " + std::to_string(i) + " is null or not 8-byte aligned");
      t.flags[i] = static_cast<unsigned long long *>(armed.flags[i]);
    }
    t.epoch = armed.epoch;
    t.finished = reinterpret_cast<unsigned int *>(ex.status_word()) + 16;
    t.wait_later = armed.overlap ? 1 : 0;
  }
  if (auto r = launch_gemm(ex, plan, {const_cast<void *>(a_shard), const_cast<void *>(b), nullptr}, stream, &t); !r)
    return r;
  if (t.wait_later) {
    // the wait for the peers, on the executor's second stream, ordered behind this launch; the NEXT
    // fused launch (or kh_join_arrivals / kh_synchronize) is ordered behind it
    auto fn = ex.function("gemm", "await_arrivals");
    if (!fn) return std::unexpected(fn.error());
    return ex.enqueue_arrival_wait(*fn, &t, sizeof t, stream);
  }
  return {};
}

// The scan launched so that its first look-back can never succeed: every ticket is shifted
// by one tile, tile 0 is therefore never produced, and the look-back of tile 1 gives up
// after `spin_limit` polls. Exists to show, on a healthy GPU and without any fault, that a
// bounded wait that runs out is reported through the status word and leaves the context usable.
Result<void> run_scan_lookback_probe(Executor &ex, const void *x, void *y, int64_t n, uint32_t spin_limit,
                                     StreamHandle stream) {
  if (n < 2 * kScanTile)
    return fail(2, "scan look-back probe: n must cover at least two tiles (" + std::to_string(2 * kScanTile) +
                       " elements)");
  if (spin_limit == 0 || spin_limit > (1u << 20))
    return fail(2, "scan look-back probe: the poll limit must be between 1 and 1048576");
  KernelPlan plan;
  try {
    plan = plan_scan({{"n", n}}, ex.limits());
  } catch (const std::exception &e) {
    return fail(2, e.what());
  }
  return launch_scan(ex, plan, {const_cast<void *>(x), y}, stream, spin_limit, 1u);
}

Result<void> run_gemm_host_sharded_begin(Executor &ex, const void *a_shard_host, const void *b_slice_host,
                                         const std::vector<void *> &b_replicas, void *b_multicast, int rank,
                                         int world, int64_t m_shard, int64_t n, int64_t k) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world || static_cast<int>(b_replicas.size()) != world)
    return fail(2, "gemm_host_sharded: rank / replica list do not match a world of 1 to 8 ranks");
  if (a_shard_host == nullptr || b_slice_host == nullptr || b_replicas[static_cast<size_t>(rank)] == nullptr)
    return fail(2, "gemm_host_sharded: null buffer");
  if (k % world != 0 || ((k / world) * n) % 4 != 0)
    return fail(2, "gemm_host_sharded: the rows of B (k = " + std::to_string(k) + ") must split evenly over " +
                       std::to_string(world) + " ranks into slices of a multiple of four floats");
  if (first_misaligned16({{"B multicast address", b_multicast}}))
    return fail(2, "gemm_host_sharded: the B multicast address is not 16-byte aligned");
  for (int i = 0; i < world; ++i) {
    if (b_replicas[static_cast<size_t>(i)] == nullptr && (b_multicast == nullptr || i == rank))
      return fail(2, "gemm_host_sharded: null B replica pointer");
    if (first_misaligned16({{"B replica", b_replicas[static_cast<size_t>(i)]}}))
      return fail(2, "gemm_host_sharded: B replica " + std::to_string(i) + " is not 16-byte aligned");
  }
  KernelPlan plan;
  try {
    plan = plan_gemm({{"m", m_shard}, {"n", n}, {"k", k}}, ex.limits());
  } catch (const std::exception &e) {
    return fail(2, e.what());
  }
  Backend &be = ex.backend();
  auto hs = ex.host_streams();
  if (!hs) return std::unexpected(hs.error());
  auto dev_a = ex.host_staging(0, static_cast<size_t>(m_shard * k) * 4);
  if (!dev_a) return std::unexpected(dev_a.error());
  auto dev_c = ex.host_staging(2, static_cast<size_t>(m_shard * n) * 4);
  if (!dev_c) return std::unexpected(dev_c.error());
  auto job = gemm_job(ex, m_shard, n, k);
  if (!job) return std::unexpected(job.error());
  auto push = ex.function("gemm", "replicate_run");
  if (!push) return std::unexpected(push.error());

  // this rank's rows of B: up into its own replica, then on to the others
  const int64_t slice_rows = k / world, first = static_cast<int64_t>(rank) * slice_rows * n, count = slice_rows * n;
  char *b_local = static_cast<char *>(b_replicas[static_cast<size_t>(rank)]);
  if (auto r = be.memcpy_h2d_async(b_local + static_cast<size_t>(first) * 4, b_slice_host,
                                   static_cast<size_t>(count) * 4, hs->in);
      !r)
    return r;
  auto b_up = be.event_create();
  if (!b_up) return std::unexpected(b_up.error());
  if (auto r = be.event_record(*b_up, hs->in); !r) return r;
  if (auto r = be.stream_wait_event(hs->compute, *b_up); !r) return r;
  if (world > 1) {
    GatherTargets t{};
    t.count = world;
    t.self = rank;
    t.multicast = static_cast<float *>(b_multicast);
    for (int i = 0; i < world; ++i) t.base[i] = static_cast<float *>(b_replicas[static_cast<size_t>(i)]);
    LaunchStep step;
    step.entry = "replicate_run";
    step.block = {256, 1, 1};
    step.grid = {static_cast<unsigned>(std::min<int64_t>((count / 4 + 1023) / 1024, sm_count(ex.limits()) * 4)), 1, 1};
    step.param_count = 3;
    LaunchArgs args;
    args.add_struct_bytes(&t, sizeof t);
    args.add_scalar<int64_t>(first);
    args.add_scalar<int64_t>(count);
    if (auto r = ex.launch(*push, step, args, hs->compute); !r) return r;
  }
  // the A shard: in row blocks, each with its own event (the uploads go on while the ranks meet)
  const std::vector<std::pair<int64_t, int64_t>> blocks = host_row_blocks(m_shard);
  std::vector<EventHandle> a_events;
  for (const auto &[row0, rows] : blocks) {
    if (auto r = be.memcpy_h2d_async(static_cast<char *>(*dev_a) + static_cast<size_t>(row0 * k) * 4,
                                     static_cast<const char *>(a_shard_host) + static_cast<size_t>(row0 * k) * 4,
                                     static_cast<size_t>(rows * k) * 4, hs->in);
        !r)
      return r;
    auto e = be.event_create();
    if (!e) return std::unexpected(e.error());
    if (auto r = be.event_record(*e, hs->in); !r) return r;
    a_events.push_back(*e);
  }
  // the slice has left this GPU when the compute stream is idle
  Result<void> pushed = be.stream_synchronize(hs->compute);
  (void)be.event_destroy(*b_up);
  if (!pushed) {
    for (EventHandle e : a_events) (void)be.event_destroy(e);
    return pushed;
  }

  const HostStreams streams = *hs;
  void *a_dev = *dev_a, *c_dev = *dev_c;
  const GemmJob j = *job;
  ex.pending_host_finish = [&ex, j, streams, a_dev, c_dev, b_local, a_events, n, k, blocks](void *c_host) -> Result<void> {
    Backend &be2 = ex.backend();
    std::vector<EventHandle> events = a_events;
    const auto body = [&]() -> Result<void> {
      if (auto r = gemm_enqueue_b(j, b_local, streams.compute, true); !r) return r;
      for (size_t i = 0; i < blocks.size(); ++i) {
        const auto [row0, rows] = blocks[i];
        char *a_rows = static_cast<char *>(a_dev) + static_cast<size_t>(row0 * k) * 4;
        char *c_rows = static_cast<char *>(c_dev) + static_cast<size_t>(row0 * n) * 4;
        if (auto r = be2.stream_wait_event(streams.compute, a_events[i]); !r) return r;
        const std::vector<LaunchStep> steps = gemm_steps(rows, n, k, ex.limits());
        if (auto r = gemm_enqueue_a(j, a_rows, row0, rows, steps[0], streams.compute, 0); !r) return r;
        if (auto r = gemm_enqueue_multiply(j, a_rows, b_local, c_rows, row0, rows, steps[3], streams.compute, nullptr);
            !r)
          return r;
        auto c_done = be2.event_create();
        if (!c_done) return std::unexpected(c_done.error());
        events.push_back(*c_done);
        if (auto r = be2.event_record(*c_done, streams.compute); !r) return r;
        if (auto r = be2.stream_wait_event(streams.out, *c_done); !r) return r;
        if (c_host != nullptr)
          if (auto r = be2.memcpy_d2h_async(static_cast<char *>(c_host) + static_cast<size_t>(row0 * n) * 4, c_rows,
                                            static_cast<size_t>(rows * n) * 4, streams.out);
              !r)
            return r;
      }
      return {};
    };
    Result<void> enqueued = body();
    Result<void> s_in = be2.stream_synchronize(streams.in);
    Result<void> s_compute = ex.synchronize(streams.compute);
    Result<void> s_out = be2.stream_synchronize(streams.out);
    for (EventHandle e : events) (void)be2.event_destroy(e);
    if (!enqueued) return enqueued;
    if (!s_compute) return s_compute;
    if (!s_in) return s_in;
    return s_out;
  };
  return {};
}

Result<void> run_gemm_host_sharded_finish(Executor &ex, void *c_shard_host) {
  if (!ex.pending_host_finish)
    return fail(2, "gemm_host_sharded: finish without a begin (phase 0 must come first on this context)");
  auto finish = std::move(ex.pending_host_finish);
  ex.pending_host_finish = nullptr;
  return finish(c_shard_host);
}

void register_attention_kernel(); // attention_kernel.cpp

void register_builtin_kernels() {
  register_kernel({"vecadd", "vecadd", plan_vecadd,
                   [](Executor &ex, const KernelPlan &p, const std::vector<void *> &b, StreamHandle s) {
                     return run_elementwise3(ex, p, b, s, "vecadd");
                   }});
  register_kernel({"fused_gelu", "fused_gelu", plan_fused_gelu,
                   [](Executor &ex, const KernelPlan &p, const std::vector<void *> &b, StreamHandle s) {
                     return run_elementwise3(ex, p, b, s, "fused_gelu");
                   }});
  register_kernel({"softmax", "softmax",
                   [](const ShapeMap &s, const DeviceLimits &l) { return plan_rows("softmax", s, l, false); },
                   run_rows});
  register_kernel({"layernorm", "layernorm",
                   [](const ShapeMap &s, const DeviceLimits &l) { return plan_rows("layernorm", s, l, true); },
                   run_rows});
  register_kernel({"scan", "scan", plan_scan, run_scan});
  // The reference's registry also holds `scan_totals`, the second kernel of its two-launch
  // scan (lib/dsl/kernels/scan.cpp:350-453: seven buffers, 'n' required and positive). The
  // single-pass `scan` here leaves nothing for it to do: the name resolves, the shape rules
  // and the buffer list are the reference's, and running it launches nothing.
  register_kernel({"scan_totals", "scan",
                   [](const ShapeMap &shape, const DeviceLimits &) {
                     auto it = shape.find("n");
                     if (it == shape.end())
                       throw std::runtime_error("scan_totals template: shape attribute 'n' is required (pass "
                                                "--shape n=<size>)");
                     if (it->second <= 0)
                       throw std::runtime_error("scan_totals template: shape attribute 'n' must be positive");
                     const int64_t n = it->second, t = (n + 255) / 256;
                     KernelPlan p;
                     p.kernel = "scan_totals";
                     p.shape = shape;
                     p.tensors = {{"totals_hi", {t}, false}, {"totals_lo", {t}, false}, {"off_hi", {t}, true},
                                  {"off_lo", {t}, true},     {"off_lo2", {t}, true},    {"y", {n}, true},
                                  {"y_lo", {n}, true}};
                     return p; // no launch steps
                   },
                   [](Executor &, const KernelPlan &, const std::vector<void *> &, StreamHandle) -> Result<void> {
                     return {};
                   }});
  register_kernel({"gemm", "gemm", plan_gemm, run_gemm, run_gemm_host});
  register_attention_kernel();
}

} // namespace kh
