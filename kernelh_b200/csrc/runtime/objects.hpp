// RAII objects of the runtime, the counterparts of the reference's
// include/kernelh/runtime/{device_context,buffer,gpu_module,event_timer,
// kernel_launch}.hpp: move-only owners whose destructors release best-effort,
// and a KernelLaunch builder that packs arguments, verifies the launch against
// the device limits and refuses it with every violation listed
// (lib/runtime/kernel_launch.cpp:100-132) before handing it to the backend.
#pragma once

#include "backend.hpp"
#include "device_limits.hpp"
#include "launch_args.hpp"

#include <memory>
#include <string>
#include <vector>

namespace kh {

class DeviceContext {
public:
  static Result<DeviceContext> create(std::shared_ptr<Backend> backend, int ordinal = 0);
  const DeviceInfo &info() const { return info_; }
  const std::shared_ptr<Backend> &backend() const { return backend_; }

private:
  std::shared_ptr<Backend> backend_;
  DeviceInfo info_;
};

class Buffer {
public:
  Buffer() = default;
  static Result<Buffer> allocate(std::shared_ptr<Backend> backend, size_t bytes);
  Buffer(Buffer &&o) noexcept;
  Buffer &operator=(Buffer &&o) noexcept;
  Buffer(const Buffer &) = delete;
  Buffer &operator=(const Buffer &) = delete;
  ~Buffer();

  void *data() const { return ptr_; }
  size_t size() const { return bytes_; }
  Result<void> copy_from_host(const void *src, size_t bytes);
  Result<void> copy_to_host(void *dst, size_t bytes) const;

private:
  void release();
  std::shared_ptr<Backend> backend_;
  void *ptr_ = nullptr;
  size_t bytes_ = 0;
};

class GpuModule {
public:
  GpuModule() = default;
  // `size` is accepted for interface parity; the driver reads the image's own header.
  static Result<GpuModule> load(std::shared_ptr<Backend> backend, const void *image, size_t size);
  GpuModule(GpuModule &&o) noexcept;
  GpuModule &operator=(GpuModule &&o) noexcept;
  GpuModule(const GpuModule &) = delete;
  GpuModule &operator=(const GpuModule &) = delete;
  ~GpuModule();
  Result<KernelFunction> get_function(const char *name) const;

private:
  void release();
  std::shared_ptr<Backend> backend_;
  void *module_ = nullptr;
};

class EventTimer {
public:
  EventTimer() = default;
  static Result<EventTimer> create(std::shared_ptr<Backend> backend);
  EventTimer(EventTimer &&o) noexcept;
  EventTimer &operator=(EventTimer &&o) noexcept;
  EventTimer(const EventTimer &) = delete;
  EventTimer &operator=(const EventTimer &) = delete;
  ~EventTimer();
  Result<void> record_start(StreamHandle s = nullptr);
  Result<void> record_end(StreamHandle s = nullptr);
  Result<void> synchronize();
  Result<float> elapsed_ms();

private:
  void release();
  std::shared_ptr<Backend> backend_;
  EventHandle start_ = nullptr, end_ = nullptr;
};

// The table entry for the backend's device, with the live device's values
// laid over it (block limits, SM count, opt-in shared memory).
DeviceLimits resolve_limits(Backend &backend);

class KernelLaunch {
public:
  explicit KernelLaunch(std::shared_ptr<Backend> backend);
  KernelLaunch &grid(unsigned x, unsigned y = 1, unsigned z = 1);
  KernelLaunch &block(unsigned x, unsigned y = 1, unsigned z = 1);
  KernelLaunch &shared_mem_bytes(size_t bytes); // dynamic shared memory (default 0)
  KernelLaunch &cluster(unsigned x);
  KernelLaunch &stream(StreamHandle s);
  KernelLaunch &memref_arg(const void *dev_ptr, const std::vector<int64_t> &shape);
  KernelLaunch &tensor_map_arg(const TensorMapBytes &map);
  template <typename T> KernelLaunch &scalar(T v) {
    args_.add_scalar(v);
    return *this;
  }
  const LaunchArgs &args() const { return args_; }
  Result<void> launch(KernelFunction fn);

private:
  std::shared_ptr<Backend> backend_;
  LaunchDims grid_{}, block_{};
  size_t shared_ = 0;
  unsigned cluster_ = 1;
  StreamHandle stream_ = nullptr;
  LaunchArgs args_;
};

} // namespace kh
