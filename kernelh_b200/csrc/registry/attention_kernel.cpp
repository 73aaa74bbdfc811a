// Registry record of the attention template: shape rules of the reference's
// lib/dsl/kernels/attention.cpp:94-120 (all four keys required and positive,
// head_dim pinned to 64, seq a multiple of the 64-key tile), the scratch
// layout of the scaled fp16 hi/lo split, the six tensor maps and the two launches.
#include "executor.hpp"
#include "registry.hpp"

#include <stdexcept>

namespace kh {
namespace {

constexpr int64_t kHeadDim = 64, kBQ = 128, kBKV = 64;
// two Q tiles hi/lo (32 KiB each) + four stages each of K and V^T hi/lo (16 KiB per stage) +
// 16 KiB in which the output warps stage half rows + alignment slack
constexpr size_t kAttnSmem = 2 * 32 * 1024 + 2 * 4 * 16 * 1024 + 16 * 1024 + 1024;

KernelPlan plan_attention(const ShapeMap &shape, const DeviceLimits &l) {
  for (const char *key : {"batch", "heads", "seq", "head_dim"})
    if (!shape.count(key))
      throw std::runtime_error("attention template: shape attributes 'batch', 'heads', 'seq' and "
                               "'head_dim' are required (missing '" + std::string(key) + "')");
  const int64_t b = shape.at("batch"), h = shape.at("heads"), s = shape.at("seq"),
                d = shape.at("head_dim");
  if (b <= 0 || h <= 0 || s <= 0 || d <= 0)
    throw std::runtime_error("attention template: shape attributes 'batch', 'heads', 'seq' and "
                             "'head_dim' must be positive");
  if (d != kHeadDim)
    throw std::runtime_error("attention template: the kernel is pinned to head_dim = 64 (got "
                             "head_dim = " + std::to_string(d) + ")");
  // `causal` (optional, 0 or 1): query i attends to keys 0..i only. Not a key of the reference's
  // template (lib/dsl/kernels/attention.cpp:109-120 has no mask): the first of its generalisations.
  const int64_t causal = shape.count("causal") ? shape.at("causal") : 0;
  if (causal != 0 && causal != 1)
    throw std::runtime_error("attention template: shape attribute 'causal' must be 0 or 1 (got causal = " +
                             std::to_string(causal) + ")");
  KernelPlan p;
  p.kernel = "attention";
  p.shape = shape;
  for (const char *name : {"Q", "K", "V"}) p.tensors.push_back({name, {b, h, s, d}, false});
  p.tensors.push_back({"O", {b, h, s, d}, true});
  // The reference pins seq to a multiple of its 64-key tile (lib/dsl/kernels/attention.cpp:109-120);
  // here any seq runs: the splits pad every slice to whole tiles and the last tile's missing keys are masked.
  const int64_t tiles = (s + kBKV - 1) / kBKV, s_padded = tiles * kBKV;
  const int64_t elems = b * h * s_padded * d;
  // six fp16 arrays, then one exponent per 64-row tile of Q, K and V
  p.workspace_bytes = static_cast<size_t>(elems) * 2 * 6 + static_cast<size_t>(b * h * tiles) * 3 * 4;
  long sms = query_cu_count(l);
  if (sms <= 0) sms = 148;
  LaunchStep split;
  split.entry = "attention_split";
  split.block = {256, 1, 1};
  split.grid = {static_cast<unsigned>(std::min<int64_t>(3 * b * h * tiles, sms * 5)), 1, 1}; // a block per 64-row tile at a time, five blocks resident per SM
  split.param_count = 33 + 7;
  LaunchStep main;
  const bool masked = causal != 0 || s % kBKV != 0;
  main.entry = masked ? "attention_masked" : "attention";
  main.overlap_tail = true; // its set-up runs under the tail of attention_split
  main.block = {512, 1, 1}; // warpgroups: producer + two MMA issuers, two softmax groups, output
  // persistent: a CTA per SM walks the (slice, 128-query tile) work items
  main.grid = {static_cast<unsigned>(std::min<int64_t>(b * h * ((s + kBQ - 1) / kBQ), sms)), 1, 1};
  main.dynamic_smem = kAttnSmem;
  main.param_count = 44 + 6 + 2 + (masked ? 1 : 0);
  main.tmem_columns = 512;
  p.steps = {split, main};
  p.work = 4.0 * static_cast<double>(b) * static_cast<double>(h) * static_cast<double>(s) *
           static_cast<double>(s) * static_cast<double>(d);
  if (causal) // the unmasked (query, key) pairs: s (s + 1) / 2 of the s^2
    p.work = 4.0 * static_cast<double>(b) * static_cast<double>(h) * (static_cast<double>(s) * (static_cast<double>(s) + 1.0) / 2.0) *
             static_cast<double>(d);
  p.work_is_flops = true;
  return p;
}

// Destinations of attention_allgather's fused all-gather; layout shared with the kernel.
struct GatherOut {
  float *peer[8];
  int count;
  int self;
  float *multicast;
};

Result<void> launch_attention(Executor &ex, const KernelPlan &p, const std::vector<void *> &buf,
                              StreamHandle stream, const GatherOut *gather) {
  if (const char *bad = first_misaligned16({{"Q", buf[0]}, {"K", buf[1]}, {"V", buf[2]}, {"O", buf[3]}}))
    return fail(2, std::string("attention: buffer '") + bad +
                       "' is not 16-byte aligned; the kernel reads and writes 128-bit vectors and has no scalar path");
  const std::vector<int64_t> &shape = p.tensors[0].shape;
  const int64_t bh = shape[0] * shape[1], seq = shape[2];
  const int64_t s = (seq + kBKV - 1) / kBKV * kBKV; // rows of a slice in the splits: whole 64-row tiles
  const int64_t elems = bh * s * kHeadDim;
  auto ws = ex.workspace(p.workspace_bytes);
  if (!ws) return std::unexpected(ws.error());
  char *base = static_cast<char *>(*ws);
  const size_t part = static_cast<size_t>(elems) * 2; // one fp16 array; elems is a multiple of 4096
  char *q_hi = base, *q_lo = base + part, *k_hi = base + 2 * part, *k_lo = base + 3 * part,
       *vt_hi = base + 4 * part, *vt_lo = base + 5 * part;
  char *shifts = base + 6 * part;

  auto f_split = ex.function("attention", "attention_split");
  if (!f_split) return std::unexpected(f_split.error());
  const bool causal = p.shape.count("causal") && p.shape.at("causal") != 0;
  const bool masked = causal || seq % kBKV != 0;
  if (gather && masked)
    return fail(2, "attention: the fused all-gather takes whole 64-key tiles and no causal mask (seq = " +
                       std::to_string(seq) + (causal ? ", causal" : "") + ")");
  auto f_main = ex.function("attention", gather ? "attention_allgather" : p.steps[1].entry);
  if (!f_main) return std::unexpected(f_main.error());
  {
    LaunchArgs args;
    for (int i = 0; i < 3; ++i) args.add_memref(buf[i], shape);
    for (char *ptr : {q_hi, q_lo, k_hi, k_lo, vt_hi, vt_lo, shifts})
      args.add_scalar<uint64_t>(reinterpret_cast<uint64_t>(ptr));
    if (auto r = ex.launch(*f_split, p.steps[0], args, stream); !r) return r;
  }
  // Q, K: [bh*s rows, 64 fp16]; V^T: [bh*64 rows, s fp16] (s = seq padded to whole tiles). 64-column boxes = one 128-byte swizzle row.
  auto make_map = [&](const char *ptr, int64_t cols, int64_t rows, uint32_t box_rows) {
    TensorMapSpec t;
    t.global_address = ptr;
    t.rank = 2;
    t.elem_bytes = 2;
    t.dims[0] = static_cast<uint64_t>(cols);
    t.dims[1] = static_cast<uint64_t>(rows);
    t.strides_bytes[0] = static_cast<uint64_t>(cols) * 2;
    t.box[0] = 64;
    t.box[1] = box_rows;
    t.swizzle_bytes = 128;
    return ex.backend().encode_tensor_map(t);
  };
  LaunchArgs args;
  for (int i = 0; i < 4; ++i) args.add_memref(buf[i], shape);
  struct M { const char *p; int64_t cols, rows; uint32_t box; };
  const M maps[6] = {{q_hi, kHeadDim, bh * s, static_cast<uint32_t>(kBQ)},
                     {q_lo, kHeadDim, bh * s, static_cast<uint32_t>(kBQ)},
                     {k_hi, kHeadDim, bh * s, static_cast<uint32_t>(kBKV)},
                     {k_lo, kHeadDim, bh * s, static_cast<uint32_t>(kBKV)},
                     {vt_hi, s, bh * kHeadDim, static_cast<uint32_t>(kHeadDim)},
                     {vt_lo, s, bh * kHeadDim, static_cast<uint32_t>(kHeadDim)}};
  for (const M &mm : maps) {
    auto t = make_map(mm.p, mm.cols, mm.rows, mm.box);
    if (!t) return std::unexpected(t.error());
    args.add_tensor_map(*t);
  }
  args.add_scalar<uint64_t>(reinterpret_cast<uint64_t>(shifts));
  args.add_scalar<uint64_t>(reinterpret_cast<uint64_t>(ex.status_word()));
  if (masked) args.add_scalar<int64_t>(causal ? 1 : 0);
  LaunchStep step = p.steps[1];
  if (gather) {
    args.add_struct_bytes(gather, sizeof *gather);
    step.entry = "attention_allgather";
  }
  return ex.launch(*f_main, step, args, stream);
}

Result<void> run_attention(Executor &ex, const KernelPlan &p, const std::vector<void *> &buf,
                           StreamHandle stream) {
  return launch_attention(ex, p, buf, stream, nullptr);
}

} // namespace

// Attention over `slices` (batch, head) problems of this rank with the all-gather
// of the output fused into the kernel: `replicas[i]` is rank i's whole
// [world * slices, seq, 64] output as mapped on this device (only replicas[rank]
// is needed when `multicast`, the replicas' NVLink multicast address, is given).
Result<void> run_attention_allgather(Executor &ex, const void *q, const void *k, const void *v,
                                     const std::vector<void *> &replicas, void *multicast, int rank,
                                     int world, int64_t slices, int64_t seq, StreamHandle stream) {
  if (world < 1 || world > 8)
    return fail(2, "attention_allgather: between 1 and 8 ranks are supported, got " + std::to_string(world));
  if (rank < 0 || rank >= world || static_cast<int>(replicas.size()) != world)
    return fail(2, "attention_allgather: rank / replica list do not match the world size");
  KernelPlan plan;
  try {
    plan = plan_attention({{"batch", slices}, {"heads", 1}, {"seq", seq}, {"head_dim", kHeadDim}}, ex.limits());
  } catch (const std::exception &e) {
    return fail(2, e.what());
  }
  const int64_t shard_elems = slices * seq * kHeadDim; // this rank's slices start this far into a replica
  GatherOut t{};
  t.count = world;
  t.self = rank;
  t.multicast = multicast ? static_cast<float *>(multicast) + rank * shard_elems : nullptr;
  if (first_misaligned16({{"O multicast address", multicast}}))
    return fail(2, "attention_allgather: the output multicast address is not 16-byte aligned");
  for (int i = 0; i < world; ++i) {
    if (replicas[i] == nullptr && (multicast == nullptr || i == rank))
      return fail(2, "attention_allgather: null output replica pointer");
    if (first_misaligned16({{"O replica", replicas[i]}}))
      return fail(2, "attention_allgather: output replica " + std::to_string(i) + " is not 16-byte aligned");
    t.peer[i] = replicas[i] ? static_cast<float *>(replicas[i]) + rank * shard_elems : nullptr;
  }
  return launch_attention(ex, plan,
                          {const_cast<void *>(q), const_cast<void *>(k), const_cast<void *>(v), t.peer[rank]},
                          stream, &t);
}

void register_attention_kernel() {
  register_kernel({"attention", "attention", plan_attention, run_attention});
}

} // namespace kh
