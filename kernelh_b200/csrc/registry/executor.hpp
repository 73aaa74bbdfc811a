// Executor: one device's launch machinery behind the kernel-name + shape
// operator surface. Owns the loaded code objects, a grow-only scratch
// allocation, the scan look-back state, the device status word that bounded
// waits report into, and a pool of device buffers for host-pointer calls.
// The path fails loudly when the driver, a code object or an entry symbol is
// missing; there is no CPU path.
#pragma once

#include "../runtime/objects.hpp"
#include "registry.hpp"

#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace kh {

// Arrival flags of a fused all-gather (see GatherTargets in kernels/gemm.cu).
struct ArrivalFlags {
  std::vector<void *> flags;
  uint64_t epoch = 0;
  bool overlap = false; // the kernel only signals; the wait runs as a launch of its own on a second stream
};

class Executor {
public:
  static Result<std::unique_ptr<Executor>> create(std::shared_ptr<Backend> backend, int ordinal);
  ~Executor();

  Backend &backend() { return *backend_; }
  const std::shared_ptr<Backend> &backend_ptr() const { return backend_; }
  const DeviceInfo &info() const { return info_; }
  const DeviceLimits &limits() const { return limits_; }

  // Plans and enqueues `kernel` for `shape` on device buffers (plan.tensors order).
  Result<void> run(const std::string &kernel, const ShapeMap &shape,
                   const std::vector<void *> &buffers, StreamHandle stream);
  // Same through host buffers: inputs are copied in, outputs copied back, the
  // device status is checked. Blocking.
  Result<void> run_host(const std::string &kernel, const ShapeMap &shape,
                        const std::vector<void *> &host_buffers);
  // Waits for `stream` and turns a recorded device-side wait timeout into an Error.
  Result<void> synchronize(StreamHandle stream);

  // ---- used by the kernel records ------------------------------------------------
  Result<KernelFunction> function(const std::string &code_object, const std::string &entry);
  // The same for a code object handed in by the caller (a kernel registered from outside);
  // `code_object` is the cache key of the loaded module.
  Result<KernelFunction> function_from_image(const std::string &code_object, const void *image, size_t size,
                                             const std::string &entry);
  Result<void *> workspace(size_t bytes);
  Result<void> launch(KernelFunction fn, const LaunchStep &step, LaunchArgs &args, StreamHandle s);
  uint32_t *status_word() const { return static_cast<uint32_t *>(status_.data()); }
  // Arrival flags for the NEXT fused all-gather launch of this executor only (then disarmed): every
  // rank's flag array as mapped on this device, and the epoch to write and wait for (> 0, growing).
  void arm_arrival_flags(std::vector<void *> flags, uint64_t epoch, bool overlap = false) {
    arrival_ = {std::move(flags), epoch, overlap};
  }
  // The overlapped wait: `await` (the gemm code object's await_arrivals) goes on a second stream behind
  // what `stream` holds now; join_arrival_wait orders `stream` behind the last such wait, if any.
  Result<void> enqueue_arrival_wait(const KernelFunction &await, const void *targets, size_t bytes, StreamHandle stream);
  Result<void> join_arrival_wait(StreamHandle stream);
  ArrivalFlags take_arrival_flags() { return std::exchange(arrival_, ArrivalFlags{}); }
  // Scratch of the gemm's split last wave: partial sums and meeting flags (grow-only).
  Result<std::pair<void *, void *>> gemm_partials(size_t partial_bytes, size_t flag_bytes);
  // The three streams of the host-buffer paths (uploads, compute, downloads), created on first use.
  Result<HostStreams> host_streams();
  // Device staging buffer number `index` of the host-buffer paths, at least `bytes` large (grow-only).
  Result<void *> host_staging(size_t index, size_t bytes);
  // A two-phase host-buffer call parks its second half here between the phases.
  std::function<Result<void>(void *)> pending_host_finish;

  // Per-launch timing: while enabled, every launch is bracketed by two events
  // on its stream. profile_report() waits for them and returns
  // "entry:launches:total_ms" items joined by ';', then forgets them.
  void profile_enable(bool on) { profiling_ = on; }
  Result<std::string> profile_report();
  uint64_t launches_issued() const { return launches_issued_; }

  // Look-back state for scans of up to `tiles` tiles: counters and one descriptor per tile,
  // zeroed when allocated; the kernel keeps it consistent from launch to launch by itself.
  Result<void *> scan_state(int64_t tiles);
  // Text of a device-side wait code (the status word's low half), e.g. "scan look-back wait".
  static const char *wait_name(uint32_t code);

private:
  Executor() = default;
  struct FunctionInfo {
    KernelFunction fn;
    size_t static_smem = 0;
    size_t optin_smem = 0; // largest dynamic size already opted in
    bool large_clusters = false; // opted in to cluster sizes above eight
  };
  std::shared_ptr<Backend> backend_;
  DeviceInfo info_;
  DeviceLimits limits_{};
  std::map<std::string, GpuModule> modules_;
  std::map<std::string, FunctionInfo> functions_;
  Buffer workspace_;
  Buffer status_;
  Buffer scan_state_;
  int64_t scan_capacity_tiles_ = 0;
  struct ProfiledLaunch {
    std::string entry;
    EventHandle start, end;
  };
  ArrivalFlags arrival_;
  StreamHandle arrival_stream_ = nullptr;
  EventHandle arrival_launched_ = nullptr, arrival_seen_ = nullptr;
  bool arrival_pending_ = false;
  Buffer gemm_partials_, gemm_partial_flags_;
  bool profiling_ = false;
  std::vector<ProfiledLaunch> profiled_;
  uint64_t launches_issued_ = 0;
  std::vector<Buffer> host_pool_;
  StreamHandle host_stream_ = nullptr;
  StreamHandle host_in_stream_ = nullptr, host_out_stream_ = nullptr;
};

// builtin_kernels.cpp
// `multicast` non-null: the replicas' NVLink multicast address (then only replicas[rank] is read).
Result<void> run_gemm_allgather(Executor &ex, const void *a_shard, const void *b,
                                const std::vector<void *> &replicas, void *multicast, int rank,
                                int world, int64_t m_shard, int64_t n, int64_t k, StreamHandle stream);

// The M-row-sharded product on HOST buffers, in two phases with the caller's barrier across
// ranks in between. begin: this rank's slice of B (rows [rank * k / world, (rank + 1) * k /
// world)) is uploaded into its own replica of B and sent on to every other replica over NVLink
// (multimem.st through `b_multicast`, or peer stores), while the upload of the A shard starts;
// returns when the slice has gone out. finish (after every rank's begin has returned and a
// barrier was passed): B is split, the A blocks are split and multiplied as they arrive, and
// the rows of C go back to `c_shard_host`; returns when they are there.
Result<void> run_gemm_host_sharded_begin(Executor &ex, const void *a_shard_host, const void *b_slice_host,
                                         const std::vector<void *> &b_replicas, void *b_multicast, int rank,
                                         int world, int64_t m_shard, int64_t n, int64_t k);
Result<void> run_gemm_host_sharded_finish(Executor &ex, void *c_shard_host);

Result<void> run_gemm_scaled(Executor &ex, const void *a, const void *b, void *c, int64_t m, int64_t n, int64_t k,
                             float alpha, float beta, StreamHandle stream);
Result<void> run_scan_lookback_probe(Executor &ex, const void *x, void *y, int64_t n, uint32_t spin_limit,
                                     StreamHandle stream);

// attention_kernel.cpp
Result<void> run_attention_allgather(Executor &ex, const void *q, const void *k, const void *v,
                                     const std::vector<void *> &replicas, void *multicast, int rank,
                                     int world, int64_t slices, int64_t seq, StreamHandle stream);

} // namespace kh
