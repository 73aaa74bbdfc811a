#include "executor.hpp"

#include "../runtime/launch_verifier.hpp"

#include <algorithm>
#include <climits>
#include <cstring>

namespace kh {

Result<std::unique_ptr<Executor>> Executor::create(std::shared_ptr<Backend> backend, int ordinal) {
  if (!backend) return fail(1, "Executor::create: null backend");
  auto ctx = DeviceContext::create(backend, ordinal);
  if (!ctx) return std::unexpected(ctx.error());
  std::unique_ptr<Executor> ex(new Executor());
  ex->backend_ = backend;
  ex->info_ = ctx->info();
  if (ex->info_.cc_major != 10)
    return fail(1, "Executor::create: device '" + ex->info_.name + "' is compute capability " +
                       std::to_string(ex->info_.cc_major) + "." + std::to_string(ex->info_.cc_minor) +
                       "; the kernels are built for sm_100a only");
  ex->limits_ = resolve_limits(*backend);
  auto st = Buffer::allocate(backend, 256);
  if (!st) return std::unexpected(st.error());
  ex->status_ = std::move(*st);
  if (auto r = backend->memset32_async(ex->status_.data(), 0, 64, nullptr); !r)
    return std::unexpected(r.error());
  if (auto r = backend->device_synchronize(); !r) return std::unexpected(r.error());
  return ex;
}

Executor::~Executor() {
  for (StreamHandle s : {host_stream_, host_in_stream_, host_out_stream_, arrival_stream_})
    if (backend_ && s) (void)backend_->stream_destroy(s);
  for (EventHandle e : {arrival_launched_, arrival_seen_})
    if (backend_ && e) (void)backend_->event_destroy(e);
}

Result<KernelFunction> Executor::function(const std::string &code_object, const std::string &entry) {
  const std::string key = code_object + ":" + entry;
  if (auto it = functions_.find(key); it != functions_.end()) return it->second.fn;
  auto mod = modules_.find(code_object);
  if (mod == modules_.end()) {
    const CodeObject *co = find_code_object(code_object);
    if (co == nullptr || co->size == 0)
      return fail(1, "no embedded sm_100a code object named '" + code_object +
                         "' (the library was built without its CUDA kernels)");
    return function_from_image(code_object, co->image, co->size, entry);
  }
  auto fn = mod->second.get_function(entry.c_str());
  if (!fn) return std::unexpected(fn.error());
  FunctionInfo fi;
  fi.fn = *fn;
  if (auto attrs = backend_->function_attributes(fn->handle))
    fi.static_smem = static_cast<size_t>(attrs->static_smem_bytes);
  functions_[key] = fi;
  return *fn;
}

Result<KernelFunction> Executor::function_from_image(const std::string &code_object, const void *image,
                                                     size_t size, const std::string &entry) {
  const std::string key = code_object + ":" + entry;
  if (auto it = functions_.find(key); it != functions_.end()) return it->second.fn;
  auto mod = modules_.find(code_object);
  if (mod == modules_.end()) {
    auto loaded = GpuModule::load(backend_, image, size);
    if (!loaded) return fail(loaded.error().code, "loading code object '" + code_object + "': " +
                                                      loaded.error().message);
    mod = modules_.emplace(code_object, std::move(*loaded)).first;
  }
  auto fn = mod->second.get_function(entry.c_str());
  if (!fn) return std::unexpected(fn.error());
  FunctionInfo fi;
  fi.fn = *fn;
  if (auto attrs = backend_->function_attributes(fn->handle))
    fi.static_smem = static_cast<size_t>(attrs->static_smem_bytes);
  functions_[key] = fi;
  return *fn;
}

Result<void *> Executor::workspace(size_t bytes) {
  if (bytes == 0) bytes = 256;
  if (workspace_.size() < bytes) {
    // Work queued on any stream may still read the old allocation.
    if (auto r = backend_->device_synchronize(); !r) return std::unexpected(r.error());
    workspace_ = Buffer();
    auto b = Buffer::allocate(backend_, bytes);
    if (!b) return fail(b.error().code, "scratch allocation of " + std::to_string(bytes) +
                                            " bytes failed: " + b.error().message);
    workspace_ = std::move(*b);
  }
  return workspace_.data();
}

Result<void> Executor::launch(KernelFunction fn, const LaunchStep &step, LaunchArgs &args,
                              StreamHandle s) {
  FunctionInfo *fi = nullptr;
  for (auto &kv : functions_)
    if (kv.second.fn.handle == fn.handle) fi = &kv.second;
  LaunchConfig cfg;
  cfg.grid_x = static_cast<int>(std::min<unsigned>(step.grid.x, INT_MAX));
  cfg.grid_y = static_cast<int>(step.grid.y);
  cfg.grid_z = static_cast<int>(step.grid.z);
  cfg.threads_per_workgroup = static_cast<int>(step.block.x * step.block.y * step.block.z);
  cfg.static_shared_bytes = fi ? fi->static_smem : 0;
  cfg.dynamic_shared_bytes = step.dynamic_smem;
  cfg.cluster_size = static_cast<int>(step.cluster);
  if (step.dynamic_smem > 0 && fi != nullptr && fi->optin_smem < step.dynamic_smem &&
      cfg.static_shared_bytes + step.dynamic_smem <= static_cast<size_t>(limits_.max_dynamic_smem_optin)) {
    if (auto r = backend_->function_set_max_dynamic_smem(fn.handle, step.dynamic_smem); !r)
      return fail(r.error().code, "launch of '" + step.entry + "': dynamic shared memory opt-in failed: " +
                                      r.error().message);
    fi->optin_smem = step.dynamic_smem;
  }
  if (step.cluster > 8 && fi != nullptr && !fi->large_clusters) {
    if (auto r = backend_->function_allow_large_clusters(fn.handle); !r)
      return fail(r.error().code, "launch of '" + step.entry + "': " + r.error().message);
    fi->large_clusters = true;
  }
  // Limits are checked analytically on every launch; the driver's occupancy
  // answer is asked for by KernelLaunch::launch and the occupancy report.
  LaunchVerifier verifier;
  if (auto ok = verifier.verify(cfg, limits_, nullptr); !ok)
    return fail(1, "launch of '" + step.entry + "' refused: " + ok.error());
  ++launches_issued_;
  if (!profiling_)
    return backend_->launch_kernel(fn.handle, step.grid, step.block, step.dynamic_smem, s,
                                   args.params(), step.cluster, step.overlap_tail);
  auto e0 = backend_->event_create();
  if (!e0) return std::unexpected(e0.error());
  auto e1 = backend_->event_create();
  if (!e1) return std::unexpected(e1.error());
  if (auto r = backend_->event_record(*e0, s); !r) return r;
  auto launched = backend_->launch_kernel(fn.handle, step.grid, step.block, step.dynamic_smem, s,
                                          args.params(), step.cluster, step.overlap_tail);
  if (auto r = backend_->event_record(*e1, s); !r) return r;
  profiled_.push_back({step.entry, *e0, *e1});
  return launched;
}

Result<std::string> Executor::profile_report() {
  std::map<std::string, std::pair<int, double>> acc;
  Error first_error;
  for (const ProfiledLaunch &p : profiled_) {
    if (auto r = backend_->event_synchronize(p.end); !r && first_error.code == 0) first_error = r.error();
    if (auto ms = backend_->event_elapsed_time(p.start, p.end)) {
      acc[p.entry].first += 1;
      acc[p.entry].second += *ms;
    } else if (first_error.code == 0) {
      first_error = ms.error();
    }
    (void)backend_->event_destroy(p.start);
    (void)backend_->event_destroy(p.end);
  }
  profiled_.clear();
  if (first_error.code != 0) return std::unexpected(first_error);
  std::string out;
  for (const auto &kv : acc) {
    if (!out.empty()) out += ';';
    out += kv.first + ":" + std::to_string(kv.second.first) + ":" + std::to_string(kv.second.second);
  }
  return out;
}

Result<void *> Executor::scan_state(int64_t tiles) {
  if (tiles > scan_capacity_tiles_) {
    const int64_t cap = std::max<int64_t>(tiles, 4096);
    if (auto r = backend_->device_synchronize(); !r) return std::unexpected(r.error());
    scan_state_ = Buffer();
    const size_t words = 4 + 2 * static_cast<size_t>(cap);
    auto b = Buffer::allocate(backend_, words * 8);
    if (!b) return std::unexpected(b.error());
    scan_state_ = std::move(*b);
    if (auto r = backend_->memset32_async(scan_state_.data(), 0, words * 2, nullptr); !r)
      return std::unexpected(r.error());
    if (auto r = backend_->device_synchronize(); !r) return std::unexpected(r.error());
    scan_capacity_tiles_ = cap;
  }
  return scan_state_.data();
}

const char *Executor::wait_name(uint32_t code) {
  static const char *names[] = {"ok", "scan look-back wait", "TMA (full-stage) wait",
                                "MMA (accumulator) wait", "epilogue wait", "empty-stage wait",
                                "wait for another GPU's arrival flag (detail = its rank)"};
  return code < 7 ? names[code] : "unknown wait";
}

Result<void> Executor::run(const std::string &kernel, const ShapeMap &shape,
                           const std::vector<void *> &buffers, StreamHandle stream) {
  if (auto r = backend_->make_current(); !r) return r;
  const KernelRecord *rec = nullptr;
  KernelPlan plan;
  try {
    rec = &find_kernel(kernel);
    plan = rec->plan(shape, limits_);
  } catch (const std::exception &e) {
    return fail(2, e.what());
  }
  if (buffers.size() != plan.tensors.size())
    return fail(2, "kernel '" + kernel + "' takes " + std::to_string(plan.tensors.size()) +
                       " buffers, got " + std::to_string(buffers.size()));
  for (size_t i = 0; i < buffers.size(); ++i)
    if (buffers[i] == nullptr && plan.tensors[i].name != "tmp")
      return fail(2, "kernel '" + kernel + "': buffer '" + plan.tensors[i].name + "' is null");
  return rec->run(*this, plan, buffers, stream);
}

Result<void> Executor::synchronize(StreamHandle stream) {
  if (auto r = backend_->make_current(); !r) return r;
  if (auto r = backend_->stream_synchronize(stream); !r) return r;
  if (arrival_pending_) { // a wait for the peers that runs on the second stream: it belongs to this work
    arrival_pending_ = false;
    if (auto r = backend_->stream_synchronize(arrival_stream_); !r) return r;
  }
  uint32_t host[2] = {0, 0};
  if (auto r = backend_->memcpy_d2h(host, status_.data(), sizeof host); !r) return r;
  uint32_t scan_host[2] = {0, 0};
  if (scan_state_.data() != nullptr) {
    if (auto r = backend_->memcpy_d2h(scan_host, static_cast<char *>(scan_state_.data()) + 8,
                                      sizeof scan_host);
        !r)
      return r;
  }
  if (host[0] == 0 && scan_host[0] == 0) return {};
  // Clear so that the next launch starts clean. The scan kernel's last block restored the
  // look-back state's counters and advanced its epoch even though the launch stopped early,
  // so only the status word has to go.
  (void)backend_->memset32_async(status_.data(), 0, 2, nullptr);
  if (scan_host[0] != 0)
    (void)backend_->memset32_async(static_cast<char *>(scan_state_.data()) + 8, 0, 2, nullptr);
  (void)backend_->device_synchronize();
  const uint32_t code = host[0] ? host[0] : scan_host[0];
  const uint32_t detail = host[0] ? host[1] : scan_host[1];
  return fail(kDeviceTimeout, std::string("a device-side bounded wait ran out: ") + wait_name(code) + " (code " +
                                  std::to_string(code) + ", detail " + std::to_string(detail) +
                                  "); the kernel stopped and its output is incomplete");
}

Result<void> Executor::enqueue_arrival_wait(const KernelFunction &await, const void *targets, size_t bytes,
                                            StreamHandle stream) {
  if (arrival_stream_ == nullptr) {
    auto s = backend_->stream_create();
    if (!s) return std::unexpected(s.error());
    arrival_stream_ = *s;
    for (EventHandle *e : {&arrival_launched_, &arrival_seen_}) {
      auto made = backend_->event_create();
      if (!made) return std::unexpected(made.error());
      *e = *made;
    }
  }
  if (auto r = backend_->event_record(arrival_launched_, stream); !r) return r;
  if (auto r = backend_->stream_wait_event(arrival_stream_, arrival_launched_); !r) return r;
  LaunchStep step;
  step.entry = "await_arrivals";
  step.block = {32, 1, 1};
  step.grid = {1, 1, 1};
  step.param_count = 2;
  LaunchArgs args;
  args.add_struct_bytes(targets, bytes);
  args.add_scalar<uint64_t>(reinterpret_cast<uint64_t>(status_word()));
  if (auto r = launch(await, step, args, arrival_stream_); !r) return r;
  if (auto r = backend_->event_record(arrival_seen_, arrival_stream_); !r) return r;
  arrival_pending_ = true;
  return {};
}

Result<void> Executor::join_arrival_wait(StreamHandle stream) {
  if (!arrival_pending_) return {};
  arrival_pending_ = false;
  return backend_->stream_wait_event(stream, arrival_seen_);
}

Result<std::pair<void *, void *>> Executor::gemm_partials(size_t partial_bytes, size_t flag_bytes) {
  for (auto [buffer, bytes] : {std::pair<Buffer *, size_t>{&gemm_partials_, partial_bytes},
                               std::pair<Buffer *, size_t>{&gemm_partial_flags_, flag_bytes}}) {
    if (buffer->data() != nullptr && buffer->size() >= bytes) continue;
    // a launch that still uses the old buffer may be in flight: wait before it is replaced
    if (auto r = backend_->device_synchronize(); !r) return std::unexpected(r.error());
    auto fresh = Buffer::allocate(backend_, bytes);
    if (!fresh) return std::unexpected(fresh.error());
    *buffer = std::move(*fresh);
  }
  return std::pair<void *, void *>{gemm_partials_.data(), gemm_partial_flags_.data()};
}

Result<HostStreams> Executor::host_streams() {
  for (StreamHandle *s : {&host_in_stream_, &host_stream_, &host_out_stream_}) {
    if (*s != nullptr) continue;
    auto created = backend_->stream_create();
    if (!created) return std::unexpected(created.error());
    *s = *created;
  }
  return HostStreams{host_in_stream_, host_stream_, host_out_stream_};
}

Result<void *> Executor::host_staging(size_t index, size_t bytes) {
  if (host_pool_.size() <= index) host_pool_.resize(index + 1);
  if (host_pool_[index].size() < bytes) {
    if (auto r = backend_->device_synchronize(); !r) return std::unexpected(r.error());
    host_pool_[index] = Buffer();
    auto b = Buffer::allocate(backend_, bytes);
    if (!b) return std::unexpected(b.error());
    host_pool_[index] = std::move(*b);
  }
  return host_pool_[index].data();
}

Result<void> Executor::run_host(const std::string &kernel, const ShapeMap &shape,
                                const std::vector<void *> &host) {
  if (auto r = backend_->make_current(); !r) return r;
  KernelPlan plan;
  try {
    plan = find_kernel(kernel).plan(shape, limits_);
  } catch (const std::exception &e) {
    return fail(2, e.what());
  }
  if (host.size() != plan.tensors.size())
    return fail(2, "kernel '" + kernel + "' takes " + std::to_string(plan.tensors.size()) +
                       " buffers, got " + std::to_string(host.size()));
  if (host_stream_ == nullptr) {
    auto s = backend_->stream_create();
    if (!s) return std::unexpected(s.error());
    host_stream_ = *s;
  }
  if (host_pool_.size() < plan.tensors.size()) host_pool_.resize(plan.tensors.size());
  std::vector<void *> dev(plan.tensors.size());
  for (size_t i = 0; i < plan.tensors.size(); ++i) {
    const size_t bytes = static_cast<size_t>(plan.tensors[i].elements()) * 4;
    if (host_pool_[i].size() < bytes) {
      if (auto r = backend_->device_synchronize(); !r) return r;
      host_pool_[i] = Buffer();
      auto b = Buffer::allocate(backend_, bytes);
      if (!b) return std::unexpected(b.error());
      host_pool_[i] = std::move(*b);
    }
    dev[i] = host_pool_[i].data();
  }
  if (const KernelRecord &record = find_kernel(kernel); record.run_host) {
    for (StreamHandle *s : {&host_in_stream_, &host_out_stream_}) {
      if (*s != nullptr) continue;
      auto created = backend_->stream_create();
      if (!created) return std::unexpected(created.error());
      *s = *created;
    }
    return record.run_host(*this, plan, host, dev, HostStreams{host_in_stream_, host_stream_, host_out_stream_});
  }
  for (size_t i = 0; i < plan.tensors.size(); ++i) {
    const size_t bytes = static_cast<size_t>(plan.tensors[i].elements()) * 4;
    if (!plan.tensors[i].is_output && host[i] != nullptr)
      if (auto r = backend_->memcpy_h2d_async(dev[i], host[i], bytes, host_stream_); !r) return r;
  }
  if (auto r = run(kernel, shape, dev, host_stream_); !r) return r;
  for (size_t i = 0; i < plan.tensors.size(); ++i)
    if (plan.tensors[i].is_output && host[i] != nullptr)
      if (auto r = backend_->memcpy_d2h_async(host[i], dev[i],
                                              static_cast<size_t>(plan.tensors[i].elements()) * 4,
                                              host_stream_);
          !r)
        return r;
  return synchronize(host_stream_);
}

} // namespace kh
