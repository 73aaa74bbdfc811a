#include "objects.hpp"

#include "launch_verifier.hpp"

#include <algorithm>
#include <climits>
#include <stdexcept>
#include <utility>

namespace kh {

Result<DeviceContext> DeviceContext::create(std::shared_ptr<Backend> backend, int ordinal) {
  if (!backend) return fail(1, "DeviceContext::create: null backend");
  if (auto r = backend->init_device(ordinal); !r) return std::unexpected(r.error());
  auto info = backend->device_info();
  if (!info) return std::unexpected(info.error());
  DeviceContext ctx;
  ctx.backend_ = std::move(backend);
  ctx.info_ = *info;
  return ctx;
}

// ---- Buffer ---------------------------------------------------------------
Result<Buffer> Buffer::allocate(std::shared_ptr<Backend> backend, size_t bytes) {
  if (!backend) return fail(1, "Buffer::allocate: null backend");
  if (bytes == 0) return fail(1, "Buffer::allocate: zero-byte allocation");
  auto p = backend->malloc(bytes);
  if (!p) return std::unexpected(p.error());
  Buffer b;
  b.backend_ = std::move(backend);
  b.ptr_ = *p;
  b.bytes_ = bytes;
  return b;
}
Buffer::Buffer(Buffer &&o) noexcept
    : backend_(std::move(o.backend_)), ptr_(std::exchange(o.ptr_, nullptr)),
      bytes_(std::exchange(o.bytes_, 0)) {}
Buffer &Buffer::operator=(Buffer &&o) noexcept {
  if (this != &o) {
    release();
    backend_ = std::move(o.backend_);
    ptr_ = std::exchange(o.ptr_, nullptr);
    bytes_ = std::exchange(o.bytes_, 0);
  }
  return *this;
}
Buffer::~Buffer() { release(); }
void Buffer::release() {
  if (ptr_ && backend_) (void)backend_->free(ptr_);
  ptr_ = nullptr;
  bytes_ = 0;
}
Result<void> Buffer::copy_from_host(const void *src, size_t bytes) {
  if (!ptr_) return fail(1, "Buffer::copy_from_host: empty buffer");
  if (bytes > bytes_) return fail(1, "Buffer::copy_from_host: " + std::to_string(bytes) +
                                         " bytes exceeds the buffer size " + std::to_string(bytes_));
  return backend_->memcpy_h2d(ptr_, src, bytes);
}
Result<void> Buffer::copy_to_host(void *dst, size_t bytes) const {
  if (!ptr_) return fail(1, "Buffer::copy_to_host: empty buffer");
  if (bytes > bytes_) return fail(1, "Buffer::copy_to_host: " + std::to_string(bytes) +
                                         " bytes exceeds the buffer size " + std::to_string(bytes_));
  return backend_->memcpy_d2h(dst, ptr_, bytes);
}

// ---- GpuModule ------------------------------------------------------------
Result<GpuModule> GpuModule::load(std::shared_ptr<Backend> backend, const void *image, size_t size) {
  if (!backend) return fail(1, "GpuModule::load: null backend");
  if (image == nullptr || size == 0) return fail(1, "GpuModule::load: empty image");
  auto m = backend->module_load_data(image);
  if (!m) return std::unexpected(m.error());
  GpuModule mod;
  mod.backend_ = std::move(backend);
  mod.module_ = *m;
  return mod;
}
GpuModule::GpuModule(GpuModule &&o) noexcept
    : backend_(std::move(o.backend_)), module_(std::exchange(o.module_, nullptr)) {}
GpuModule &GpuModule::operator=(GpuModule &&o) noexcept {
  if (this != &o) {
    release();
    backend_ = std::move(o.backend_);
    module_ = std::exchange(o.module_, nullptr);
  }
  return *this;
}
GpuModule::~GpuModule() { release(); }
void GpuModule::release() {
  if (module_ && backend_) (void)backend_->module_unload(module_);
  module_ = nullptr;
}
Result<KernelFunction> GpuModule::get_function(const char *name) const {
  if (!module_) return fail(1, "GpuModule::get_function: no module loaded");
  auto f = backend_->module_get_function(module_, name);
  if (!f) return std::unexpected(f.error());
  return KernelFunction{*f};
}

// ---- EventTimer -----------------------------------------------------------
Result<EventTimer> EventTimer::create(std::shared_ptr<Backend> backend) {
  if (!backend) return fail(1, "EventTimer::create: null backend");
  auto s = backend->event_create();
  if (!s) return std::unexpected(s.error());
  auto e = backend->event_create();
  if (!e) {
    (void)backend->event_destroy(*s);
    return std::unexpected(e.error());
  }
  EventTimer t;
  t.backend_ = std::move(backend);
  t.start_ = *s;
  t.end_ = *e;
  return t;
}
EventTimer::EventTimer(EventTimer &&o) noexcept
    : backend_(std::move(o.backend_)), start_(std::exchange(o.start_, nullptr)),
      end_(std::exchange(o.end_, nullptr)) {}
EventTimer &EventTimer::operator=(EventTimer &&o) noexcept {
  if (this != &o) {
    release();
    backend_ = std::move(o.backend_);
    start_ = std::exchange(o.start_, nullptr);
    end_ = std::exchange(o.end_, nullptr);
  }
  return *this;
}
EventTimer::~EventTimer() { release(); }
void EventTimer::release() {
  if (backend_) {
    if (start_) (void)backend_->event_destroy(start_);
    if (end_) (void)backend_->event_destroy(end_);
  }
  start_ = end_ = nullptr;
}
Result<void> EventTimer::record_start(StreamHandle s) { return backend_->event_record(start_, s); }
Result<void> EventTimer::record_end(StreamHandle s) { return backend_->event_record(end_, s); }
Result<void> EventTimer::synchronize() { return backend_->event_synchronize(end_); }
Result<float> EventTimer::elapsed_ms() { return backend_->event_elapsed_time(start_, end_); }

// ---- KernelLaunch ---------------------------------------------------------
DeviceLimits resolve_limits(Backend &backend) {
  DeviceLimits limits = sm_100a_limits; // the one target this runtime launches on
  if (auto info = backend.device_info()) {
    limits.lds_bytes_per_workgroup = info->lds_bytes_per_workgroup;
    limits.wavefront_size = info->wavefront_size;
    limits.max_threads_per_workgroup = info->max_threads_per_workgroup;
    limits.cu_count = info->cu_count;
    limits.vram_bytes = info->vram_bytes;
    // Without this the live 48 KiB static limit would also cap dynamic shared memory.
    if (info->smem_optin_per_block > 0) limits.max_dynamic_smem_optin = info->smem_optin_per_block;
    if (info->smem_per_sm > 0) limits.smem_per_sm = info->smem_per_sm;
    if (info->regs_per_sm > 0) limits.reg_file_per_cu = info->regs_per_sm;
    if (info->max_blocks_per_sm > 0) limits.max_blocks_per_sm = info->max_blocks_per_sm;
    if (info->max_threads_per_sm > 0 && info->wavefront_size > 0)
      limits.waves_per_cu = info->max_threads_per_sm / info->wavefront_size;
  }
  return limits;
}

KernelLaunch::KernelLaunch(std::shared_ptr<Backend> backend) : backend_(std::move(backend)) {}
KernelLaunch &KernelLaunch::grid(unsigned x, unsigned y, unsigned z) { grid_ = {x, y, z}; return *this; }
KernelLaunch &KernelLaunch::block(unsigned x, unsigned y, unsigned z) { block_ = {x, y, z}; return *this; }
KernelLaunch &KernelLaunch::shared_mem_bytes(size_t bytes) { shared_ = bytes; return *this; }
KernelLaunch &KernelLaunch::cluster(unsigned x) { cluster_ = x; return *this; }
KernelLaunch &KernelLaunch::stream(StreamHandle s) { stream_ = s; return *this; }
KernelLaunch &KernelLaunch::memref_arg(const void *p, const std::vector<int64_t> &shape) {
  args_.add_memref(p, shape);
  return *this;
}
KernelLaunch &KernelLaunch::tensor_map_arg(const TensorMapBytes &map) {
  args_.add_tensor_map(map);
  return *this;
}

Result<void> KernelLaunch::launch(KernelFunction fn) {
  if (!backend_) return fail(1, "KernelLaunch::launch: null backend");
  if (fn.handle == nullptr) return fail(1, "KernelLaunch::launch: null kernel function handle");
  if (args_.empty()) return fail(1, "KernelLaunch::launch: no kernel arguments packed");

  const DeviceLimits limits = resolve_limits(*backend_);
  LaunchConfig cfg;
  cfg.grid_x = static_cast<int>(std::min<unsigned>(grid_.x, INT_MAX));
  cfg.grid_y = static_cast<int>(std::min<unsigned>(grid_.y, INT_MAX));
  cfg.grid_z = static_cast<int>(std::min<unsigned>(grid_.z, INT_MAX));
  cfg.threads_per_workgroup = static_cast<int>(
      std::min<long long>(1LL * block_.x * block_.y * block_.z, INT_MAX));
  cfg.dynamic_shared_bytes = shared_;
  cfg.cluster_size = static_cast<int>(cluster_);
  if (auto attrs = backend_->function_attributes(fn.handle))
    cfg.static_shared_bytes = static_cast<size_t>(attrs->static_smem_bytes);

  // The opt-in must precede the occupancy query, which otherwise reports 0
  // blocks for more than 48 KiB of dynamic shared memory.
  if (shared_ > 0 && limits.max_dynamic_smem_optin > 0 &&
      cfg.static_shared_bytes + shared_ <= static_cast<size_t>(limits.max_dynamic_smem_optin)) {
    if (auto r = backend_->function_set_max_dynamic_smem(fn.handle, shared_); !r)
      return fail(r.error().code, "KernelLaunch::launch: dynamic shared memory opt-in failed: " +
                                      r.error().message);
  }
  LaunchVerifier verifier;
  if (auto ok = verifier.verify(cfg, limits, fn.handle); !ok)
    return fail(1, "KernelLaunch::launch refused: " + ok.error());

  return backend_->launch_kernel(fn.handle, grid_, block_, shared_, stream_, args_.params(), cluster_);
}

} // namespace kh
