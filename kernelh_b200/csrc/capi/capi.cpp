// Implementation of the C ABI declared in include/kernelh_b200.h: a thin shell
// over the C++ runtime, registry and harness. No exception leaves this file.
#include "kernelh_b200.h"

#include "../harness/csv.hpp"
#include "../harness/metrics.hpp"
#include "../harness/timer.hpp"
#include "../registry/executor.hpp"
#include "../registry/registry.hpp"
#include "../runtime/launch_verifier.hpp"
#include "../runtime/occupancy.hpp"
#include "../runtime/resources.hpp"

#include <atomic>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

struct kh_context {
  std::unique_ptr<kh::Executor> exec;
};

namespace {

thread_local std::string g_last_error;

int set_error(int code, const std::string &message) {
  g_last_error = message;
  return code == 0 ? 1 : code;
}
int set_error(const kh::Error &e) { return set_error(e.code, e.message); }

int copy_out(const std::string &s, char *buf, int cap) {
  if (buf != nullptr && cap > 0) {
    const size_t n = std::min(s.size(), static_cast<size_t>(cap - 1));
    std::memcpy(buf, s.data(), n);
    buf[n] = '\0';
  }
  return static_cast<int>(s.size());
}

template <typename F> int guarded(F &&f) {
  try {
    return f();
  } catch (const std::exception &e) {
    return set_error(2, e.what());
  } catch (...) {
    return set_error(1, "unknown C++ exception");
  }
}

// The tensor-core kernels and the fused all-gathers move 128-bit vectors (and
// multimem.st.v4 / float4 peer stores) without a scalar path: an address that is
// not 16-byte aligned is refused here, on the host, before anything is launched.
// Returns 0 when every non-null address is aligned.
int refuse_misaligned(const char *entry, std::initializer_list<std::pair<const char *, const void *>> buffers) {
  if (const char *bad = kh::first_misaligned16(buffers))
    return set_error(2, std::string(entry) + ": buffer '" + bad +
                            "' is not 16-byte aligned; this kernel has no scalar path "
                            "(pass an aligned allocation or copy the view)");
  return 0;
}

// Every entry point that takes a context passes through here: besides the null check, the
// context's device becomes the calling thread's current one, so a process that holds several
// contexts (one per GPU) never allocates or launches on the device of the context it used last.
int need_ctx(kh_context *ctx) {
  if (ctx == nullptr || !ctx->exec) return set_error(2, "null kernelh_b200 context");
  if (auto r = ctx->exec->backend().make_current(); !r) return set_error(r.error());
  return 0;
}

int launch_named(kh_context *ctx, const char *kernel, const kh::ShapeMap &shape,
                 std::vector<void *> buffers, void *stream) {
  if (int rc = need_ctx(ctx)) return rc;
  return guarded([&] {
    auto r = ctx->exec->run(kernel, shape, buffers, stream);
    return r ? 0 : set_error(r.error());
  });
}

} // namespace

extern "C" {

const char *kh_last_error(void) { return g_last_error.c_str(); }
// For entry points implemented outside this file: records the calling thread's
// error message and returns the code to hand back.
int kh_detail_set_error(int code, const char *message) { return set_error(code, message ? message : ""); }
const char *kh_version(void) { return "kernelh_b200 0.1 (sm_100a)"; }

int kh_context_create(int device_ordinal, kh_context **out) {
  if (out == nullptr) return set_error(2, "kh_context_create: null out pointer");
  *out = nullptr;
  return guarded([&] {
    auto backend = kh::make_cuda_backend();
    if (!backend) return set_error(backend.error());
    auto exec = kh::Executor::create(*backend, device_ordinal);
    if (!exec) return set_error(exec.error());
    *out = new kh_context{std::move(*exec)};
    return 0;
  });
}

void kh_context_destroy(kh_context *ctx) { delete ctx; }

int kh_device_count(int *count) {
  return guarded([&] {
    auto backend = kh::make_cuda_backend();
    if (!backend) return set_error(backend.error());
    auto n = (*backend)->device_count();
    if (!n) return set_error(n.error());
    if (count) *count = *n;
    return 0;
  });
}

int kh_device_info_get(kh_context *ctx, kh_device_info *out) {
  if (int rc = need_ctx(ctx)) return rc;
  if (out == nullptr) return set_error(2, "kh_device_info_get: null out pointer");
  const kh::DeviceInfo &i = ctx->exec->info();
  std::memset(out, 0, sizeof *out);
  copy_out(i.name, out->name, sizeof out->name);
  out->vram_bytes = i.vram_bytes;
  out->static_smem_per_block = i.lds_bytes_per_workgroup;
  out->optin_smem_per_block = i.smem_optin_per_block;
  out->smem_per_sm = i.smem_per_sm;
  out->l2_bytes = i.l2_bytes;
  out->sm_count = static_cast<int32_t>(i.cu_count);
  out->warp_size = i.wavefront_size;
  out->max_threads_per_block = i.max_threads_per_workgroup;
  out->regs_per_sm = i.regs_per_sm;
  out->max_blocks_per_sm = i.max_blocks_per_sm;
  out->cc_major = i.cc_major;
  out->cc_minor = i.cc_minor;
  out->ordinal = i.ordinal;
  return 0;
}

int kh_launch(kh_context *ctx, const char *kernel, const char *shape, void *const *device_buffers,
              int n_buffers, void *stream) {
  if (kernel == nullptr || shape == nullptr) return set_error(2, "kh_launch: null kernel or shape");
  const kh::ShapeMap map = kh::parse_shape_text(shape);
  if (map.empty()) return set_error(2, std::string("malformed --shape text '") + shape + "' (expected k=v,k=v with integer values)");
  std::vector<void *> bufs(device_buffers, device_buffers + (n_buffers > 0 ? n_buffers : 0));
  return launch_named(ctx, kernel, map, std::move(bufs), stream);
}

int kh_run_host(kh_context *ctx, const char *kernel, const char *shape, void *const *host_buffers,
                int n_buffers) {
  if (int rc = need_ctx(ctx)) return rc;
  if (kernel == nullptr || shape == nullptr) return set_error(2, "kh_run_host: null kernel or shape");
  const kh::ShapeMap map = kh::parse_shape_text(shape);
  if (map.empty()) return set_error(2, std::string("malformed --shape text '") + shape + "' (expected k=v,k=v with integer values)");
  std::vector<void *> bufs(host_buffers, host_buffers + (n_buffers > 0 ? n_buffers : 0));
  return guarded([&] {
    auto r = ctx->exec->run_host(kernel, map, bufs);
    return r ? 0 : set_error(r.error());
  });
}

int kh_synchronize(kh_context *ctx, void *stream) {
  if (int rc = need_ctx(ctx)) return rc;
  auto r = ctx->exec->synchronize(stream);
  return r ? 0 : set_error(r.error());
}

int kh_module_launch(kh_context *ctx, const void *image, size_t image_size, const char *entry,
                     const uint32_t grid[3], const uint32_t block[3], size_t dynamic_smem,
                     const uint64_t *ptrs, const int64_t *shapes, const int *ranks, int n_memrefs,
                     void *stream) {
  if (int rc = need_ctx(ctx)) return rc;
  if (entry == nullptr || grid == nullptr || block == nullptr)
    return set_error(2, "kh_module_launch: null entry, grid or block");
  return guarded([&] {
    auto backend = ctx->exec->backend_ptr();
    if (auto r = backend->make_current(); !r) return set_error(r.error());
    auto module = kh::GpuModule::load(backend, image, image_size);
    if (!module) return set_error(module.error());
    auto fn = module->get_function(entry);
    if (!fn) return set_error(fn.error());
    kh::KernelLaunch launch(backend);
    launch.grid(grid[0], grid[1], grid[2]).block(block[0], block[1], block[2]).shared_mem_bytes(dynamic_smem).stream(stream);
    const int64_t *sp = shapes;
    for (int i = 0; i < n_memrefs; ++i) {
      launch.memref_arg(reinterpret_cast<const void *>(ptrs[i]), std::vector<int64_t>(sp, sp + ranks[i]));
      sp += ranks[i];
    }
    auto r = launch.launch(*fn);
    if (!r) return set_error(r.error());
    // the module is unloaded when this scope ends: wait for the kernel first
    if (auto s = backend->stream_synchronize(stream); !s) return set_error(s.error());
    return 0;
  });
}

int kh_profile_enable(kh_context *ctx, int on) {
  if (int rc = need_ctx(ctx)) return rc;
  ctx->exec->profile_enable(on != 0);
  return 0;
}
int kh_profile_report(kh_context *ctx, char *buf, int cap) {
  if (int rc = need_ctx(ctx)) return rc;
  auto r = ctx->exec->profile_report();
  if (!r) return set_error(r.error());
  copy_out(*r, buf, cap);
  return 0;
}
int kh_launch_count(kh_context *ctx, uint64_t *count) {
  if (int rc = need_ctx(ctx)) return rc;
  if (count) *count = ctx->exec->launches_issued();
  return 0;
}

int kh_vecadd(kh_context *ctx, const float *a, const float *b, float *c, int64_t n, void *stream) {
  return launch_named(ctx, "vecadd", {{"n", n}},
                      {const_cast<float *>(a), const_cast<float *>(b), c}, stream);
}
int kh_fused_gelu(kh_context *ctx, const float *x, float *out, int64_t n, void *stream) {
  return launch_named(ctx, "fused_gelu", {{"n", n}}, {const_cast<float *>(x), nullptr, out}, stream);
}
int kh_fused_gelu_bias(kh_context *ctx, const float *x, const float *bias, float *out, int64_t n,
                       void *stream) {
  return launch_named(ctx, "fused_gelu", {{"n", n}, {"bias", 1}},
                      {const_cast<float *>(x), const_cast<float *>(bias), out}, stream);
}
int kh_scan(kh_context *ctx, const float *x, float *y, int64_t n, void *stream) {
  return launch_named(ctx, "scan", {{"n", n}}, {const_cast<float *>(x), y}, stream);
}
int kh_scan_lookback_probe(kh_context *ctx, const float *x, float *y, int64_t n, uint32_t poll_limit, void *stream) {
  if (int rc = need_ctx(ctx)) return rc;
  if (x == nullptr || y == nullptr) return set_error(2, "kh_scan_lookback_probe: null buffer");
  return guarded([&] {
    if (auto r = ctx->exec->backend().make_current(); !r) return set_error(r.error());
    auto r = kh::run_scan_lookback_probe(*ctx->exec, x, y, n, poll_limit, stream);
    return r ? 0 : set_error(r.error());
  });
}
int kh_wait_name(uint32_t code, char *buf, int cap) {
  copy_out(kh::Executor::wait_name(code), buf, cap);
  return 0;
}
int kh_softmax(kh_context *ctx, const float *x, float *y, int64_t rows, int64_t cols, void *stream) {
  return launch_named(ctx, "softmax", {{"rows", rows}, {"cols", cols}}, {const_cast<float *>(x), y},
                      stream);
}
int kh_layernorm(kh_context *ctx, const float *x, const float *gamma, const float *beta, float *y,
                 int64_t rows, int64_t cols, void *stream) {
  return launch_named(ctx, "layernorm", {{"rows", rows}, {"cols", cols}},
                      {const_cast<float *>(x), const_cast<float *>(gamma),
                       const_cast<float *>(beta), y},
                      stream);
}
int kh_gemm(kh_context *ctx, const float *a, const float *b, float *c, int64_t m, int64_t n,
            int64_t k, void *stream) {
  return launch_named(ctx, "gemm", {{"m", m}, {"n", n}, {"k", k}},
                      {const_cast<float *>(a), const_cast<float *>(b), c}, stream);
}
int kh_gemm_scaled(kh_context *ctx, const float *a, const float *b, float *c, int64_t m, int64_t n, int64_t k,
                   float alpha, float beta, void *stream) {
  if (int rc = need_ctx(ctx)) return rc;
  if (a == nullptr || b == nullptr || c == nullptr) return set_error(2, "kh_gemm_scaled: null buffer");
  if (m <= 0 || n <= 0 || k <= 0) return set_error(2, "kh_gemm_scaled: m, n and k must be positive");
  return guarded([&] {
    auto r = kh::run_gemm_scaled(*ctx->exec, a, b, c, m, n, k, alpha, beta, stream);
    return r ? 0 : set_error(r.error());
  });
}
int kh_gemm_allgather(kh_context *ctx, const float *a_shard, const float *b, void *const *c_replicas,
                      int world, int rank, int64_t m_shard, int64_t n, int64_t k, void *stream) {
  if (c_replicas == nullptr || world <= 0) return set_error(2, "kh_gemm_allgather: no C replicas given");
  if (world > 8) return set_error(2, "kh_gemm_allgather: between 1 and 8 ranks are supported");
  for (int i = 0; i < world; ++i)
    if (int rc = refuse_misaligned("kh_gemm_allgather", {{"C replica", c_replicas[i]}})) return rc;
  if (int rc = need_ctx(ctx)) return rc;
  return guarded([&] {
    if (auto r = ctx->exec->backend().make_current(); !r) return set_error(r.error());
    std::vector<void *> reps(c_replicas, c_replicas + world);
    auto r = kh::run_gemm_allgather(*ctx->exec, a_shard, b, reps, nullptr, rank, world, m_shard, n, k, stream);
    return r ? 0 : set_error(r.error());
  });
}
int kh_gemm_allgather_multicast(kh_context *ctx, const float *a_shard, const float *b, float *c_local,
                                void *c_multicast, int world, int rank, int64_t m_shard, int64_t n,
                                int64_t k, void *stream) {
  if (c_multicast == nullptr || c_local == nullptr)
    return set_error(2, "kh_gemm_allgather_multicast: null C address");
  if (int rc = refuse_misaligned("kh_gemm_allgather_multicast", {{"C", c_local}, {"C multicast address", c_multicast}}))
    return rc;
  if (int rc = need_ctx(ctx)) return rc;
  if (world < 1 || world > 8 || rank < 0 || rank >= world)
    return set_error(2, "kh_gemm_allgather_multicast: rank / world out of range");
  return guarded([&] {
    if (auto r = ctx->exec->backend().make_current(); !r) return set_error(r.error());
    std::vector<void *> reps(static_cast<size_t>(world), nullptr);
    reps[static_cast<size_t>(rank)] = c_local;
    auto r = kh::run_gemm_allgather(*ctx->exec, a_shard, b, reps, c_multicast, rank, world, m_shard, n, k, stream);
    return r ? 0 : set_error(r.error());
  });
}
int kh_gemm_host_sharded_begin(kh_context *ctx, const float *a_shard_host, const float *b_slice_host,
                               void *const *b_replicas, void *b_multicast, int world, int rank, int64_t m_shard,
                               int64_t n, int64_t k) {
  if (b_replicas == nullptr || world <= 0 || world > 8)
    return set_error(2, "kh_gemm_host_sharded_begin: between 1 and 8 B replicas are expected");
  if (int rc = refuse_misaligned("kh_gemm_host_sharded_begin", {{"B multicast address", b_multicast}})) return rc;
  for (int i = 0; i < world; ++i)
    if (int rc = refuse_misaligned("kh_gemm_host_sharded_begin", {{"B replica", b_replicas[i]}})) return rc;
  if (int rc = need_ctx(ctx)) return rc;
  return guarded([&] {
    if (auto r = ctx->exec->backend().make_current(); !r) return set_error(r.error());
    std::vector<void *> reps(b_replicas, b_replicas + world);
    auto r = kh::run_gemm_host_sharded_begin(*ctx->exec, a_shard_host, b_slice_host, reps, b_multicast, rank, world,
                                             m_shard, n, k);
    return r ? 0 : set_error(r.error());
  });
}
int kh_gemm_host_sharded_finish(kh_context *ctx, float *c_shard_host) {
  if (int rc = need_ctx(ctx)) return rc;
  return guarded([&] {
    if (auto r = ctx->exec->backend().make_current(); !r) return set_error(r.error());
    auto r = kh::run_gemm_host_sharded_finish(*ctx->exec, c_shard_host);
    return r ? 0 : set_error(r.error());
  });
}
int kh_attention(kh_context *ctx, const float *q, const float *k, const float *v, float *o,
                 int64_t batch, int64_t heads, int64_t seq, int64_t head_dim, void *stream) {
  if (int rc = refuse_misaligned("kh_attention", {{"Q", q}, {"K", k}, {"V", v}, {"O", o}})) return rc;
  return launch_named(ctx, "attention",
                      {{"batch", batch}, {"heads", heads}, {"seq", seq}, {"head_dim", head_dim}},
                      {const_cast<float *>(q), const_cast<float *>(k), const_cast<float *>(v), o},
                      stream);
}

int kh_attention_allgather(kh_context *ctx, const float *q, const float *k, const float *v,
                           void *const *o_replicas, void *o_multicast, int world, int rank, int64_t slices,
                           int64_t seq, int64_t head_dim, void *stream) {
  if (o_replicas == nullptr || world <= 0) return set_error(2, "kh_attention_allgather: no output replicas given");
  if (world > 8) return set_error(2, "kh_attention_allgather: between 1 and 8 ranks are supported");
  if (head_dim != 64) return set_error(2, "kh_attention_allgather: the kernel is pinned to head_dim = 64");
  if (int rc = refuse_misaligned("kh_attention_allgather", {{"Q", q}, {"K", k}, {"V", v}, {"O multicast address", o_multicast}}))
    return rc;
  for (int i = 0; i < world; ++i)
    if (int rc = refuse_misaligned("kh_attention_allgather", {{"O replica", o_replicas[i]}})) return rc;
  if (int rc = need_ctx(ctx)) return rc;
  return guarded([&] {
    if (auto r = ctx->exec->backend().make_current(); !r) return set_error(r.error());
    std::vector<void *> reps(o_replicas, o_replicas + world);
    auto r = kh::run_attention_allgather(*ctx->exec, q, k, v, reps, o_multicast, rank, world, slices, seq, stream);
    return r ? 0 : set_error(r.error());
  });
}

int kh_malloc(kh_context *ctx, size_t bytes, void **out) {
  if (int rc = need_ctx(ctx)) return rc;
  if (out == nullptr) return set_error(2, "kh_malloc: null out pointer");
  (void)ctx->exec->backend().make_current();
  auto p = ctx->exec->backend().malloc(bytes);
  if (!p) return set_error(p.error());
  *out = *p;
  return 0;
}
int kh_free(kh_context *ctx, void *ptr) {
  if (int rc = need_ctx(ctx)) return rc;
  (void)ctx->exec->backend().make_current();
  auto r = ctx->exec->backend().free(ptr);
  return r ? 0 : set_error(r.error());
}
int kh_memcpy_h2d(kh_context *ctx, void *dst, const void *src, size_t bytes) {
  if (int rc = need_ctx(ctx)) return rc;
  (void)ctx->exec->backend().make_current();
  auto r = ctx->exec->backend().memcpy_h2d(dst, src, bytes);
  return r ? 0 : set_error(r.error());
}
int kh_memcpy_d2h(kh_context *ctx, void *dst, const void *src, size_t bytes) {
  if (int rc = need_ctx(ctx)) return rc;
  (void)ctx->exec->backend().make_current();
  auto r = ctx->exec->backend().memcpy_d2h(dst, src, bytes);
  return r ? 0 : set_error(r.error());
}

int kh_bench_row(kh_context *ctx, const char *kernel, const char *shape, int warmup, int iters,
                 double *ms_median, double *rate, int *rate_is_gflops) {
  if (int rc = need_ctx(ctx)) return rc;
  return guarded([&] {
    const kh::ShapeMap map = kh::parse_shape_text(shape ? shape : "");
    if (map.empty()) return set_error(2, "kh_bench_row: malformed shape text");
    kh::Executor &ex = *ctx->exec;
    const kh::KernelPlan plan = kh::find_kernel(kernel).plan(map, ex.limits());
    std::vector<kh::Buffer> owned;
    std::vector<void *> bufs;
    for (const kh::TensorArg &t : plan.tensors) {
      auto b = kh::Buffer::allocate(ex.backend_ptr(), static_cast<size_t>(t.elements()) * 4);
      if (!b) return set_error(b.error());
      // 0x3c003c00 is the fp32 value 0.0078..., finite and harmless for every kernel
      if (auto r = ex.backend().memset32_async(b->data(), 0x3c003c00u, static_cast<size_t>(t.elements()), nullptr); !r)
        return set_error(r.error());
      bufs.push_back(b->data());
      owned.push_back(std::move(*b));
    }
    auto ms = kh::bench::time_launch_median(
        ex.backend_ptr(), [&] { return ex.run(kernel, map, bufs, nullptr); }, warmup, iters, nullptr);
    if (!ms) return set_error(ms.error());
    if (auto r = ex.synchronize(nullptr); !r) return set_error(r.error());
    if (ms_median) *ms_median = *ms;
    if (rate)
      *rate = plan.work_is_flops ? kh::bench::gflops_from_ms(plan.work, *ms)
                                 : kh::bench::gbps_from_ms(plan.work, *ms);
    if (rate_is_gflops) *rate_is_gflops = plan.work_is_flops ? 1 : 0;
    return 0;
  });
}

int kh_arm_arrival_flags(kh_context *ctx, void *const *flag_arrays, int world, uint64_t epoch) {
  if (int rc = need_ctx(ctx)) return rc;
  if (flag_arrays == nullptr || world < 2 || world > 8)
    return set_error(2, "kh_arm_arrival_flags: between 2 and 8 flag arrays are expected");
  if (epoch == 0) return set_error(2, "kh_arm_arrival_flags: the epoch must be positive (and grow from call to call)");
  ctx->exec->arm_arrival_flags(std::vector<void *>(flag_arrays, flag_arrays + world), epoch);
  return 0;
}

int kh_arm_arrival_flags_overlapped(kh_context *ctx, void *const *flag_arrays, int world, uint64_t epoch) {
  if (int rc = kh_arm_arrival_flags(ctx, flag_arrays, world, epoch)) return rc;
  ctx->exec->arm_arrival_flags(std::vector<void *>(flag_arrays, flag_arrays + world), epoch, /*overlap=*/true);
  return 0;
}

int kh_join_arrivals(kh_context *ctx, void *stream) {
  if (int rc = need_ctx(ctx)) return rc;
  auto r = ctx->exec->join_arrival_wait(stream);
  return r ? 0 : set_error(r.error());
}

int kh_gemm_clock(kh_context *ctx, uint64_t *sm_cycles, uint64_t *nanoseconds) {
  if (int rc = need_ctx(ctx)) return rc;
  uint64_t record[2] = {0, 0};
  auto r = ctx->exec->backend().memcpy_d2h(record, reinterpret_cast<char *>(ctx->exec->status_word()) + 32, sizeof record);
  if (!r) return set_error(r.error());
  if (sm_cycles) *sm_cycles = record[0];
  if (nanoseconds) *nanoseconds = record[1];
  return 0;
}

int kh_enable_peer_access(kh_context *ctx, kh_context *peer) {
  if (int rc = need_ctx(ctx)) return rc;
  if (int rc = need_ctx(peer)) return rc;
  return guarded([&] {
    auto r = ctx->exec->backend().enable_peer_access(peer->exec->backend());
    return r ? 0 : set_error(r.error());
  });
}

int kh_bench_sharded(int gpus, const char *kernel, const char *shape, int warmup, int iters, double *ms_median,
                     double *rate, int *rate_is_gflops) {
  if (gpus < 1 || gpus > 8) return set_error(2, "kh_bench_sharded: between 1 and 8 GPUs are supported");
  if (kernel == nullptr || shape == nullptr) return set_error(2, "kh_bench_sharded: kernel name and shape text are required");
  const std::string name = kernel;
  if (name != "gemm" && name != "attention")
    return set_error(2, "kh_bench_sharded: only gemm (M-row blocks) and attention ((batch, head) slices) are partitioned; "
                        "the other kernels run as independent replicas");
  if (warmup < 0 || iters < 1) return set_error(2, "kh_bench_sharded: iters must be at least 1");
  return guarded([&] {
    const kh::ShapeMap map = kh::parse_shape_text(shape);
    if (map.empty()) return set_error(2, "kh_bench_sharded: malformed shape text");
    {
      int have = 0;
      if (int rc = kh_device_count(&have)) return rc;
      if (have < gpus)
        return set_error(kh::kDriverUnavailable, "kh_bench_sharded: " + std::to_string(gpus) + " GPUs asked for, " +
                                                     std::to_string(have) + " visible");
    }
    // one context per GPU, every GPU mapped into every other
    struct Rank {
      std::unique_ptr<kh::Executor> exec;
      std::vector<kh::Buffer> owned;
      std::vector<void *> in;       // this rank's inputs
      void *out = nullptr;          // its replica of the whole output
      kh::EventHandle start = nullptr, stop = nullptr;
    };
    std::vector<Rank> ranks(static_cast<size_t>(gpus));
    for (int d = 0; d < gpus; ++d) {
      auto backend = kh::make_cuda_backend();
      if (!backend) return set_error(backend.error());
      auto exec = kh::Executor::create(*backend, d);
      if (!exec) return set_error(exec.error());
      ranks[d].exec = std::move(*exec);
    }
    for (int d = 0; d < gpus; ++d)
      for (int e = 0; e < gpus; ++e)
        if (auto r = ranks[d].exec->backend().enable_peer_access(ranks[e].exec->backend()); !r) return set_error(r.error());

    // the plan of the WHOLE problem gives the shapes and the work; each rank runs its shard of it
    const kh::KernelPlan plan = kh::find_kernel(name).plan(map, ranks[0].exec->limits());
    int64_t m = 0, n = 0, k = 0, slices = 0, seq = 0;
    if (name == "gemm") {
      m = map.at("m"), n = map.at("n"), k = map.at("k");
      if (m % (256 * gpus) != 0)
        return set_error(2, "kh_bench_sharded: gemm rows must split into whole 256-row tiles per GPU (m = " +
                                std::to_string(m) + ", " + std::to_string(gpus) + " GPUs)");
    } else {
      slices = map.at("batch") * map.at("heads"), seq = map.at("seq");
      if (slices % gpus != 0)
        return set_error(2, "kh_bench_sharded: batch * heads must be a multiple of the GPU count");
    }
    const auto filled = [&](Rank &r, int64_t elements) -> kh::Result<void *> {
      auto b = kh::Buffer::allocate(r.exec->backend_ptr(), static_cast<size_t>(elements) * 4);
      if (!b) return std::unexpected(b.error());
      // 0x3c003c00 is the fp32 value 0.0078..., finite and harmless for every kernel
      if (auto w = r.exec->backend().memset32_async(b->data(), 0x3c003c00u, static_cast<size_t>(elements), nullptr); !w)
        return std::unexpected(w.error());
      void *p = b->data();
      r.owned.push_back(std::move(*b));
      return p;
    };
    for (Rank &r : ranks) {
      if (auto c = r.exec->backend().make_current(); !c) return set_error(c.error());
      const std::vector<int64_t> inputs = name == "gemm" ? std::vector<int64_t>{m / gpus * k, k * n}
                                                         : std::vector<int64_t>(3, slices / gpus * seq * 64);
      for (int64_t elements : inputs) {
        auto p = filled(r, elements);
        if (!p) return set_error(p.error());
        r.in.push_back(*p);
      }
      auto o = filled(r, name == "gemm" ? m * n : slices * seq * 64);
      if (!o) return set_error(o.error());
      r.out = *o;
      for (kh::EventHandle *e : {&r.start, &r.stop}) {
        auto made = r.exec->backend().event_create();
        if (!made) return set_error(made.error());
        *e = *made;
      }
      if (auto done = r.exec->backend().device_synchronize(); !done) return set_error(done.error());
    }
    std::vector<void *> replicas;
    for (Rank &r : ranks) replicas.push_back(r.out);

    // One step: every rank's launch is enqueued (they run concurrently, each storing its tiles into
    // every replica with plain peer stores), then the host waits for all of them: the barrier after
    // which every replica holds the whole output. The step's time is the slowest rank's, by events.
    std::vector<double> times;
    for (int it = 0; it < warmup + iters; ++it) {
      for (int d = 0; d < gpus; ++d) {
        Rank &r = ranks[d];
        kh::Backend &be = r.exec->backend();
        if (auto c = be.make_current(); !c) return set_error(c.error());
        if (auto e = be.event_record(r.start, nullptr); !e) return set_error(e.error());
        kh::Result<void> launched =
            name == "gemm" ? kh::run_gemm_allgather(*r.exec, r.in[0], r.in[1], replicas, nullptr, d, gpus, m / gpus, n, k, nullptr)
                           : kh::run_attention_allgather(*r.exec, r.in[0], r.in[1], r.in[2], replicas, nullptr, d, gpus,
                                                         slices / gpus, seq, nullptr);
        if (!launched) return set_error(launched.error());
        if (auto e = be.event_record(r.stop, nullptr); !e) return set_error(e.error());
      }
      double slowest = 0.0;
      for (Rank &r : ranks) {
        if (auto c = r.exec->backend().make_current(); !c) return set_error(c.error());
        if (auto done = r.exec->synchronize(nullptr); !done) return set_error(done.error());
        auto ms = r.exec->backend().event_elapsed_time(r.start, r.stop);
        if (!ms) return set_error(ms.error());
        slowest = std::max(slowest, static_cast<double>(*ms));
      }
      if (it >= warmup) times.push_back(slowest);
    }
    for (Rank &r : ranks) {
      (void)r.exec->backend().make_current();
      (void)r.exec->backend().event_destroy(r.start);
      (void)r.exec->backend().event_destroy(r.stop);
    }
    std::sort(times.begin(), times.end());
    const double median = times.size() % 2 ? times[times.size() / 2]
                                           : 0.5 * (times[times.size() / 2 - 1] + times[times.size() / 2]);
    if (ms_median) *ms_median = median;
    if (rate) *rate = kh::bench::gflops_from_ms(plan.work, median);
    if (rate_is_gflops) *rate_is_gflops = 1;
    return 0;
  });
}

int kh_register_kernel(const char *name, const void *image, size_t image_size, const char *entry, kh_plan_fn plan,
                       void *user) {
  if (name == nullptr || *name == '\0' || image == nullptr || image_size == 0 || entry == nullptr || plan == nullptr)
    return set_error(2, "kh_register_kernel: name, code object, entry symbol and plan callback are all required");
  return guarded([&] {
    static std::atomic<uint64_t> serial{0};
    auto bytes = std::make_shared<const std::vector<unsigned char>>(static_cast<const unsigned char *>(image),
                                                                    static_cast<const unsigned char *>(image) + image_size);
    kh::KernelRecord rec;
    rec.name = name;
    // a key of its own for the executors' module caches: a later registration under the same name is a new module
    rec.code_object = std::string("user:") + name + "#" + std::to_string(serial.fetch_add(1));
    rec.image = bytes;
    const std::string kernel = name, symbol = entry;
    rec.plan = [kernel, symbol, plan, user](const kh::ShapeMap &shape, const kh::DeviceLimits &limits) {
      kh_custom_plan out;
      std::memset(&out, 0, sizeof out);
      char why[512] = {0};
      const long sms = kh::query_cu_count(limits);
      const int rc = plan(kh::shape_to_text(shape).c_str(), static_cast<int>(sms > 0 ? sms : limits.cu_count), &out, why,
                          static_cast<int>(sizeof why), user);
      if (rc != 0)
        throw std::runtime_error(kernel + " template: " + (why[0] ? why : "the plan callback refused the shape"));
      if (out.n_buffers < 1 || out.n_buffers > 8)
        throw std::runtime_error(kernel + " template: the plan callback must describe 1 to 8 buffers");
      kh::KernelPlan p;
      p.kernel = kernel;
      p.shape = shape;
      for (int i = 0; i < out.n_buffers; ++i)
        p.tensors.push_back({"arg" + std::to_string(i), {out.elements[i]}, out.is_output[i] != 0});
      kh::LaunchStep s;
      s.entry = symbol;
      s.grid = {out.grid[0], std::max(out.grid[1], 1u), std::max(out.grid[2], 1u)};
      s.block = {out.block[0], std::max(out.block[1], 1u), std::max(out.block[2], 1u)};
      s.dynamic_smem = out.dynamic_smem;
      s.param_count = 5 * out.n_buffers;
      p.steps = {s};
      p.work = out.work;
      p.work_is_flops = out.work_is_flops != 0;
      return p;
    };
    const std::string key = rec.code_object;
    rec.run = [bytes, key](kh::Executor &ex, const kh::KernelPlan &p, const std::vector<void *> &b,
                           kh::StreamHandle stream) -> kh::Result<void> {
      auto fn = ex.function_from_image(key, bytes->data(), bytes->size(), p.steps[0].entry);
      if (!fn) return std::unexpected(fn.error());
      kh::LaunchArgs args;
      for (size_t i = 0; i < p.tensors.size(); ++i) args.add_memref(b[i], p.tensors[i].shape);
      return ex.launch(*fn, p.steps[0], args, stream);
    };
    kh::register_kernel(std::move(rec));
    return 0;
  });
}

int kh_unregister_kernel(const char *name) {
  return guarded([&] {
    if (name == nullptr || !kh::unregister_kernel(name))
      return set_error(2, std::string("kh_unregister_kernel: '") + (name ? name : "") +
                              "' was not registered through kh_register_kernel");
    return 0;
  });
}

int kh_registered_kernels(char *buf, int cap) {
  return guarded([&] {
    std::string s;
    for (const std::string &n : kh::registered_kernels()) {
      if (!s.empty()) s += ',';
      s += n;
    }
    copy_out(s, buf, cap);
    return 0;
  });
}

int kh_plan(const char *kernel, const char *shape, const char *target_token, int sm_count,
            kh_plan_info *out) {
  if (out == nullptr) return set_error(2, "kh_plan: null out pointer");
  return guarded([&] {
    kh::DeviceLimits limits = kh::device_limits_for(target_token);
    if (sm_count > 0) limits.cu_count = sm_count;
    const kh::ShapeMap map = kh::parse_shape_text(shape ? shape : "");
    const kh::KernelPlan plan = kh::find_kernel(kernel ? kernel : "").plan(map, limits);
    std::memset(out, 0, sizeof *out);
    out->n_buffers = static_cast<int32_t>(plan.tensors.size());
    out->n_launches = static_cast<int32_t>(plan.steps.size());
    out->workspace_bytes = static_cast<int64_t>(plan.workspace_bytes);
    if (plan.steps.empty()) return 0; // a template that launches nothing (scan_totals)
    const kh::LaunchStep &s = plan.steps.back();
    copy_out(s.entry, out->entry, sizeof out->entry);
    out->grid[0] = s.grid.x; out->grid[1] = s.grid.y; out->grid[2] = s.grid.z;
    out->block[0] = s.block.x; out->block[1] = s.block.y; out->block[2] = s.block.z;
    out->dynamic_smem = static_cast<int64_t>(s.dynamic_smem);
    out->param_count = s.param_count;
    out->tmem_columns = s.tmem_columns;
    out->work = plan.work;
    out->work_is_flops = plan.work_is_flops ? 1 : 0;
    return 0;
  });
}

int kh_kernel_image(const char *kernel, const void **image, size_t *size) {
  return guarded([&] {
    const std::string name(kernel ? kernel : "");
    const kh::KernelRecord &rec = kh::find_kernel(name);
    if (rec.image) { // registered from outside: its own code object
      if (image) *image = rec.image->data();
      if (size) *size = rec.image->size();
      return 0;
    }
    const kh::CodeObject *co = kh::find_code_object(rec.code_object);
    if (co == nullptr || co->size == 0)
      return set_error(1, "no embedded sm_100a code object for kernel '" + rec.name + "'");
    if (image) *image = co->image;
    if (size) *size = co->size;
    return 0;
  });
}

int kh_parse_ptxas(const char *text, const char *entry, int64_t *fields6) {
  if (text == nullptr || fields6 == nullptr) return set_error(2, "kh_parse_ptxas: null argument");
  return guarded([&] {
    for (const kh::EntryResources &e : kh::parse_ptxas_report(text)) {
      if (entry != nullptr && *entry != '\0' && e.entry != entry) continue;
      fields6[0] = e.registers; fields6[1] = e.smem_bytes; fields6[2] = e.stack_bytes;
      fields6[3] = e.spill_store_bytes; fields6[4] = e.spill_load_bytes; fields6[5] = e.barriers;
      return 0;
    }
    return set_error(1, std::string("unparseable ptxas output: no entry '") + (entry ? entry : "") +
                            "' with a 'Used N registers' line");
  });
}

int kh_kernel_resources(const char *kernel, const char *entry, const char *target_token, char *json, int cap,
                        int64_t *fields6) {
  return guarded([&] {
    const std::string name(kernel ? kernel : "");
    const kh::KernelRecord &rec = kh::find_kernel(name);
    const kh::CodeObject *co = kh::find_code_object(rec.code_object);
    if (co == nullptr || co->ptxas_report == nullptr)
      return set_error(1, "no resource report embedded for kernel '" + rec.name + "'");
    const std::string want = (entry != nullptr && *entry != '\0') ? std::string(entry) : rec.name;
    for (const kh::EntryResources &e : kh::parse_ptxas_report(co->ptxas_report)) {
      if (e.entry != want) continue;
      if (json != nullptr) copy_out(kh::resources_json(e, rec.name, target_token ? target_token : "sm_100a"), json, cap);
      if (fields6 != nullptr) {
        fields6[0] = e.registers; fields6[1] = e.smem_bytes; fields6[2] = e.stack_bytes;
        fields6[3] = e.spill_store_bytes; fields6[4] = e.spill_load_bytes; fields6[5] = e.barriers;
      }
      return 0;
    }
    return set_error(1, "kernel '" + rec.name + "' has no entry point '" + want + "' in its resource report");
  });
}

int kh_occupancy_report(const char *kernel, const char *shape, const char *target_token, int sm_count, char *json,
                        int json_cap, char *markdown, int markdown_cap) {
  return guarded([&] {
    const std::string token(target_token ? target_token : "sm_100a");
    kh::DeviceLimits limits = kh::device_limits_for(token.c_str());
    if (sm_count > 0) limits.cu_count = sm_count;
    const std::string name(kernel ? kernel : "");
    const kh::KernelRecord &rec = kh::find_kernel(name);
    const kh::ShapeMap map = kh::parse_shape_text(shape ? shape : "");
    const kh::KernelPlan plan = rec.plan(map, limits);
    const kh::CodeObject *co = kh::find_code_object(rec.code_object);
    const std::vector<kh::EntryResources> entries =
        co != nullptr && co->ptxas_report != nullptr ? kh::parse_ptxas_report(co->ptxas_report)
                                                     : std::vector<kh::EntryResources>{};
    std::vector<kh::OccupancyReport> reports;
    for (const kh::LaunchStep &s : plan.steps) { // one report per launch of the plan
      kh::OccupancyInput in;
      in.kernel = s.entry;
      in.target = token;
      in.config = kh::shape_to_text(map);
      in.threads_per_workgroup = static_cast<int>(s.block.x * s.block.y * s.block.z);
      in.dynamic_smem_bytes = static_cast<long>(s.dynamic_smem);
      in.tmem_columns = s.tmem_columns;
      for (const kh::EntryResources &e : entries)
        if (e.entry == s.entry) {
          in.vgpr_count = e.registers;
          in.lds_bytes = e.smem_bytes;
        }
      kh::OccupancyReport r = kh::occupancy_report(in, limits);
      r.measured_note = "not measured: analytic report from the build's ptxas figures";
      reports.push_back(std::move(r));
    }
    if (json != nullptr) copy_out(reports.size() == 1 ? kh::occupancy_json(reports[0]) + "\n" : kh::occupancy_json_all(reports), json, json_cap);
    if (markdown != nullptr) copy_out(kh::occupancy_markdown(reports), markdown, markdown_cap);
    return 0;
  });
}

int kh_pack_memrefs(const uint64_t *ptrs, const int64_t *shapes, const int *ranks, int count,
                    uint64_t *slots, int cap, int *n_slots) {
  kh::LaunchArgs args;
  const int64_t *sp = shapes;
  for (int i = 0; i < count; ++i) {
    args.add_memref(reinterpret_cast<const void *>(ptrs[i]), std::vector<int64_t>(sp, sp + ranks[i]));
    sp += ranks[i];
  }
  const auto &raw = args.raw_slots();
  for (size_t i = 0; i < raw.size() && static_cast<int>(i) < cap; ++i) slots[i] = raw[i];
  if (n_slots) *n_slots = static_cast<int>(raw.size());
  return 0;
}

int kh_device_limits(const char *token, int64_t *f, char *name, int name_cap) {
  return guarded([&] {
    const kh::DeviceLimits &l = kh::device_limits_for(token);
    f[0] = l.lds_bytes_per_workgroup; f[1] = l.wavefront_size; f[2] = l.max_threads_per_workgroup;
    f[3] = l.max_grid_dim[0]; f[4] = l.max_grid_dim[1]; f[5] = l.max_grid_dim[2];
    f[6] = l.vram_bytes; f[7] = l.waves_per_cu; f[8] = l.reg_file_per_cu; f[9] = l.cu_count;
    f[10] = l.max_dynamic_smem_optin; f[11] = l.smem_per_sm; f[12] = l.max_blocks_per_sm;
    f[13] = l.tmem_columns_per_sm;
    copy_out(l.name, name, name_cap);
    return 0;
  });
}

int kh_target_token(const char *cli_target, char *buf, int cap) {
  const std::string tok = kh::device_token_for_cli_target(cli_target ? cli_target : "");
  if (tok.empty()) {
    std::string list;
    for (const std::string &t : kh::known_cli_targets()) {
      if (!list.empty()) list += ", ";
      list += t;
    }
    return set_error(2, std::string("unknown --target '") + (cli_target ? cli_target : "") +
                            "'; valid --target values: " + list);
  }
  copy_out(tok, buf, cap);
  return 0;
}

int kh_verify_launch(const char *token, int threads, int gx, int gy, int gz, uint64_t static_smem,
                     uint64_t dynamic_smem, int warps_per_sm_override, char *msg, int cap) {
  return guarded([&] {
    kh::DeviceLimits l = kh::device_limits_for(token);
    if (warps_per_sm_override > 0) l.waves_per_cu = warps_per_sm_override;
    kh::LaunchConfig c;
    c.threads_per_workgroup = threads;
    c.grid_x = gx; c.grid_y = gy; c.grid_z = gz;
    c.static_shared_bytes = static_smem;
    c.dynamic_shared_bytes = dynamic_smem;
    auto r = kh::LaunchVerifier().verify(c, l);
    if (r) {
      copy_out("", msg, cap);
      return 0;
    }
    copy_out(r.error(), msg, cap);
    g_last_error = r.error();
    return 1;
  });
}

int kh_occupancy(const char *token, int regs, int64_t static_smem, int threads, int64_t dynamic_smem,
                 int tmem_columns, int *out5, double *theoretical_pct, int *sm3) {
  return guarded([&] {
    kh::OccupancyInput in;
    in.kernel = "k";
    in.target = token ? token : "";
    in.vgpr_count = regs;
    in.lds_bytes = static_smem;
    in.threads_per_workgroup = threads;
    in.dynamic_smem_bytes = dynamic_smem;
    in.tmem_columns = tmem_columns;
    const kh::OccupancyReport r = kh::occupancy_report(in, kh::device_limits_for(token));
    if (out5) {
      out5[0] = r.vgpr_limited_waves; out5[1] = r.lds_limited_blocks; out5[2] = r.thread_limited_blocks;
      out5[3] = r.achieved_waves; out5[4] = static_cast<int>(r.limiter);
    }
    if (theoretical_pct) *theoretical_pct = r.theoretical_pct;
    if (sm3) {
      static const char *names[] = {"none", "registers", "shared memory", "warps", "block cap", "tensor memory"};
      int idx = 0;
      for (int i = 0; i < 6; ++i)
        if (r.sm_limiter == names[i]) idx = i;
      sm3[0] = r.sm_resident_blocks;
      sm3[1] = static_cast<int>(r.sm_occupancy_pct * 100.0 + 0.5);
      sm3[2] = idx;
    }
    return 0;
  });
}

double kh_metric(const char *what, int64_t a, int64_t b, int64_t c, int64_t d) {
  using namespace kh::bench;
  const std::string w(what ? what : "");
  if (w == "gemm_flops") return gemm_flops(a, b, c);
  if (w == "gemm_bytes") return gemm_bytes(a, b, c);
  if (w == "elementwise_bytes") return elementwise_bytes(a, b);
  if (w == "layernorm_bytes") return layernorm_bytes(a, b);
  if (w == "scan_bytes") return scan_bytes(a);
  if (w == "fused_gelu_bytes") return fused_gelu_bytes(a);
  if (w == "attention_flops") return attention_flops(a, b, c, d);
  if (w == "vecadd_bytes") return vecadd_bytes(a);
  return -1.0;
}

double kh_rate(int gflops, double work, double ms) {
  return gflops ? kh::bench::gflops_from_ms(work, ms) : kh::bench::gbps_from_ms(work, ms);
}

int kh_csv_header(char *buf, int cap) {
  copy_out(kh::bench::kCsvHeader, buf, cap);
  return 0;
}

int kh_csv_line(const char *kernel, const char *shape, const char *backend, double ms, double rate,
                const char *timestamp, const char *device, char *buf, int cap) {
  kh::bench::BenchRow r;
  r.kernel = kernel ? kernel : "";
  r.shape = shape ? shape : "";
  r.backend = backend ? backend : "";
  r.ms_median = ms;
  r.gflops_or_gbps = rate;
  r.timestamp = timestamp ? timestamp : "";
  r.device = device ? device : "";
  copy_out(kh::bench::csv_line(r), buf, cap);
  return 0;
}

int kh_csv_header_ext(char *buf, int cap) {
  copy_out(kh::bench::kCsvExtendedHeader, buf, cap);
  return 0;
}

int kh_csv_line_ext(const char *kernel, const char *shape, const char *backend, double ms, double rate,
                    const char *timestamp, const char *device, int gpus, double roofline_frac, double max_rel_err,
                    double cpu_ms, int cpu_cores, char *buf, int cap) {
  kh::bench::BenchRow r;
  r.kernel = kernel ? kernel : "";
  r.shape = shape ? shape : "";
  r.backend = backend ? backend : "";
  r.ms_median = ms;
  r.gflops_or_gbps = rate;
  r.timestamp = timestamp ? timestamp : "";
  r.device = device ? device : "";
  r.gpus = gpus;
  r.roofline_frac = roofline_frac;
  r.max_rel_err = max_rel_err;
  r.cpu_ms = cpu_ms;
  r.cpu_cores = cpu_cores;
  copy_out(kh::bench::csv_line_extended(r), buf, cap);
  return 0;
}

int kh_shape_roundtrip(const char *text, char *buf, int cap) {
  copy_out(kh::shape_to_text(kh::parse_shape_text(text ? text : "")), buf, cap);
  return 0;
}

} // extern "C"
