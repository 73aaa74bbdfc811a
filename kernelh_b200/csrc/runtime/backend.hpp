// GPU backend interface and its one implementation, the CUDA Driver API bound
// at run time with dlopen("libcuda.so.1"). Same shape as the reference's
// include/kernelh/runtime/backend.hpp:56-96 (every call returns Result, the
// driver is never linked, a missing driver is Error{77}), widened for B200:
// streams, async copies, pinned host memory, opt-in dynamic shared memory,
// function attributes, the driver's occupancy query, TMA tensor maps, cluster
// launches and a device count. The device the backend was initialised on is
// the one device_info() describes (the reference always describes device 0,
// lib/runtime/backend_cuda.cpp:125).
#pragma once

#include "error.hpp"
#include "launch_args.hpp"

#include <cstdint>
#include <memory>
#include <string>

namespace kh {

struct DeviceInfo {
  std::string name;
  long lds_bytes_per_workgroup = 0; // static shared memory per block (no opt-in)
  int wavefront_size = 0;
  int max_threads_per_workgroup = 0;
  long cu_count = 0;
  long vram_bytes = 0;
  // added
  long smem_optin_per_block = 0;
  long smem_per_sm = 0;
  int regs_per_sm = 0;
  int max_blocks_per_sm = 0;
  int max_threads_per_sm = 0;
  long l2_bytes = 0;
  int cc_major = 0, cc_minor = 0;
  int ordinal = 0;
};

struct LaunchDims {
  unsigned x = 1, y = 1, z = 1;
};

using EventHandle = void *;
using StreamHandle = void *;

struct KernelFunction {
  void *handle = nullptr;
};

struct FunctionAttributes {
  int num_regs = 0;
  int static_smem_bytes = 0;
  int max_dynamic_smem_bytes = 0;
  int max_threads_per_block = 0;
};

// One dimension list per tensor-map rank, innermost first (TMA convention).
struct TensorMapSpec {
  const void *global_address = nullptr;
  int rank = 0;
  uint64_t dims[5] = {0, 0, 0, 0, 0};       // elements
  uint64_t strides_bytes[4] = {0, 0, 0, 0}; // strides of dims 1..rank-1
  uint32_t box[5] = {1, 1, 1, 1, 1};        // elements
  int swizzle_bytes = 0;                    // 0, 32, 64 or 128
  int elem_bytes = 4;                       // 4 = fp32, 2 = fp16
};

class Backend {
public:
  virtual ~Backend() = default;
  virtual const char *kind() const = 0;

  virtual Result<int> device_count() = 0;
  virtual Result<void> init_device(int ordinal) = 0;
  virtual Result<void> make_current() = 0;
  // The driver's context handle (opaque here), and peer mapping between two devices of one process.
  virtual void *native_context() { return nullptr; }
  virtual Result<void> enable_peer_access(Backend &peer) {
    (void)peer;
    return fail(1, "this backend has no peer access");
  }
  virtual Result<DeviceInfo> device_info() = 0;
  virtual Result<void> device_synchronize() = 0;

  virtual Result<void *> malloc(size_t bytes) = 0;
  virtual Result<void> free(void *ptr) = 0;
  virtual Result<void *> malloc_host(size_t bytes) = 0;
  virtual Result<void> free_host(void *ptr) = 0;
  virtual Result<void> memcpy_h2d(void *dst, const void *src, size_t bytes) = 0;
  virtual Result<void> memcpy_d2h(void *dst, const void *src, size_t bytes) = 0;
  virtual Result<void> memcpy_h2d_async(void *dst, const void *src, size_t bytes, StreamHandle s) = 0;
  virtual Result<void> memcpy_d2h_async(void *dst, const void *src, size_t bytes, StreamHandle s) = 0;
  virtual Result<void> memcpy_d2d_async(void *dst, const void *src, size_t bytes, StreamHandle s) = 0;
  virtual Result<void> memset32_async(void *dst, uint32_t value, size_t words, StreamHandle s) = 0;

  virtual Result<void *> module_load_data(const void *image) = 0;
  virtual Result<void *> module_get_function(void *module, const char *name) = 0;
  virtual Result<void> module_unload(void *module) = 0;
  virtual Result<FunctionAttributes> function_attributes(void *function) = 0;
  virtual Result<void> function_set_max_dynamic_smem(void *function, size_t bytes) = 0;
  // Cluster sizes above eight CTAs are not portable: a kernel has to opt in before such a launch.
  virtual Result<void> function_allow_large_clusters(void *function) = 0;
  virtual Result<int> occupancy_max_blocks(void *function, int block_size, size_t dyn_smem) = 0;
  virtual Result<TensorMapBytes> encode_tensor_map(const TensorMapSpec &spec) = 0;

  // `cluster_x` > 1: CTAs per cluster. `overlap_tail`: programmatic dependent launch - the
  // kernel may be scheduled while the previous kernel of the stream is still draining; it must
  // then wait (griddepcontrol.wait) before it touches anything that kernel may have written.
  virtual Result<void> launch_kernel(void *function, const LaunchDims &grid, const LaunchDims &block,
                                     size_t shared_bytes, StreamHandle stream, void *const *params,
                                     unsigned cluster_x = 1, bool overlap_tail = false) = 0;

  virtual Result<StreamHandle> stream_create() = 0;
  virtual Result<void> stream_destroy(StreamHandle s) = 0;
  virtual Result<void> stream_synchronize(StreamHandle s) = 0;

  virtual Result<EventHandle> event_create() = 0;
  virtual Result<void> event_record(EventHandle e, StreamHandle s) = 0;
  virtual Result<void> event_synchronize(EventHandle e) = 0;
  virtual Result<void> stream_wait_event(StreamHandle s, EventHandle e) = 0; // later work of s waits for e
  virtual Result<bool> event_query(EventHandle e) = 0; // true = complete
  virtual Result<float> event_elapsed_time(EventHandle start, EventHandle end) = 0;
  virtual Result<void> event_destroy(EventHandle e) = 0;
};

// dlopen + dlsym of every needed driver symbol. A missing library or symbol is
// Error{77}. `library_path` is for tests ("" = libcuda.so.1).
Result<std::shared_ptr<Backend>> make_cuda_backend(const std::string &library_path = "");

} // namespace kh
