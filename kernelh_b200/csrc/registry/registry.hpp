// Kernel registry: process-wide map from a kernel-template name to the record
// that knows how to plan and launch it. Same behaviour as the reference's
// registry (include/kernelh/dsl/program.hpp:64-67, lib/dsl/registry.cpp:23-42,
// lib/dsl/program.cpp:27-37): built-ins appear on first use, registering an
// existing name replaces it, names list sorted, and an unknown name throws
// std::runtime_error "unknown kernel template '<name>'; registered kernels: ...".
// The registered value here is a hand-written kernel (code object, entry
// symbols, launch plan) rather than an IR-emitting function; launch geometry
// belongs to the record, not to the caller.
#pragma once

#include "../runtime/backend.hpp"
#include "../runtime/device_limits.hpp"
#include "shape_text.hpp"

#include <functional>
#include <initializer_list>
#include <memory>
#include <utility>
#include <string>
#include <vector>

namespace kh {

class Executor;

struct TensorArg {
  std::string name;
  std::vector<int64_t> shape; // fp32 elements, row-major contiguous
  bool is_output = false;
  int64_t elements() const {
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    return n;
  }
};

struct LaunchStep {
  std::string entry;
  LaunchDims grid, block;
  size_t dynamic_smem = 0;
  unsigned cluster = 1;
  bool overlap_tail = false; // the entry waits with griddepcontrol.wait: it may be scheduled under its predecessor's tail
  int param_count = 0;   // kernel parameters (descriptor slots + extras)
  int tmem_columns = 0;
};

struct KernelPlan {
  std::string kernel;
  ShapeMap shape;
  std::vector<TensorArg> tensors; // caller-visible buffers, template order
  size_t workspace_bytes = 0;     // scratch the executor provides
  std::vector<LaunchStep> steps;
  double work = 0.0;              // flops or bytes, the reference's metric conventions
  bool work_is_flops = false;
};

// The streams a host-buffer run may spread its work over.
struct HostStreams {
  StreamHandle in = nullptr, compute = nullptr, out = nullptr;
};

struct KernelRecord {
  std::string name;
  std::string code_object; // which embedded cubin holds the entry symbols
  // Validates the shape (throws std::runtime_error naming the offending key,
  // as the reference's templates do) and lays out the launch for `limits`.
  std::function<KernelPlan(const ShapeMap &, const DeviceLimits &)> plan;
  // Enqueues the launches of `plan` on `stream`; `buffers` are device pointers
  // in plan.tensors order.
  std::function<Result<void>(Executor &, const KernelPlan &, const std::vector<void *> &,
                             StreamHandle)>
      run;
  // Optional host-buffer form that overlaps transfers with compute: `host` are
  // the caller's buffers, `dev` device staging buffers of the same sizes. It
  // returns with everything finished. Kernels without one use upload, run,
  // download on a single stream.
  std::function<Result<void>(Executor &, const KernelPlan &, const std::vector<void *> &host,
                             const std::vector<void *> &dev, const HostStreams &)>
      run_host = nullptr;
  // A record registered from outside carries its own code object instead of naming an
  // embedded one (code_object is then a unique key for the executor's module cache).
  std::shared_ptr<const std::vector<unsigned char>> image;
};

// Name of the first non-null address in `buffers` that is not 16-byte aligned,
// or nullptr. Pure host arithmetic (used before any launch of a kernel that has
// no scalar path).
inline const char *first_misaligned16(std::initializer_list<std::pair<const char *, const void *>> buffers) {
  for (const auto &[name, ptr] : buffers)
    if (ptr != nullptr && (reinterpret_cast<uintptr_t>(ptr) & 15u) != 0) return name;
  return nullptr;
}

// Adds the record, or replaces the one registered under its name (built-ins included).
void register_kernel(KernelRecord record);
// Takes a record registered over the built-ins away again: a built-in of that name comes
// back, any other name disappears. False when the name was not registered from outside.
bool unregister_kernel(const std::string &name);
std::vector<std::string> registered_kernels();
const KernelRecord &find_kernel(const std::string &name);

// Embedded code objects (one cubin per kernel source), generated at build time.
struct CodeObject {
  const char *name;
  const unsigned char *image;
  size_t size;
  const char *ptxas_report; // `ptxas -v` lines of the build that made the image
};
const CodeObject *find_code_object(const std::string &name);
std::vector<std::string> code_object_names();

} // namespace kh
