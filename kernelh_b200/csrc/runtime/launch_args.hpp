// Kernel-argument packing. Buffer arguments use the reference's device ABI
// bit for bit (lib/runtime/descriptor_packing.cpp:19-60): each buffer is the
// expanded memref descriptor (allocated ptr, aligned ptr, offset = 0,
// sizes[N], row-major contiguous strides[N]) = 2N+3 eight-byte slots, and
// scalars take one slot each. New: a 128-byte, 64-byte-aligned tensor-map
// argument (CUtensorMap) that the TMA-fed kernels take after their
// descriptors; it is one kernel parameter but not an 8-byte slot.
#pragma once

#include <cstddef>
#include <cstdint>
#include <deque>
#include <vector>

namespace kh {

struct alignas(64) TensorMapBytes {
  uint64_t opaque[16];
};

class LaunchArgs {
public:
  void add_memref(const void *dev_ptr, const std::vector<int64_t> &shape);
  void add_scalar_bytes(const void *value, size_t byte_size);
  template <typename T> void add_scalar(T value) { add_scalar_bytes(&value, sizeof(T)); }
  void add_tensor_map(const TensorMapBytes &map);
  // A by-value struct parameter of up to kMaxStructBytes (stored 64-byte aligned). A larger
  // struct is refused (std::length_error), never truncated: a kernel reading past a short copy
  // would take whatever follows it for pointers.
  static constexpr size_t kMaxStructBytes = 256;
  void add_struct_bytes(const void *value, size_t byte_size);

  // Number of kernel parameters: 8-byte slots plus tensor maps.
  size_t param_count() const { return order_.size(); }
  size_t slot_count() const { return slots_.size(); }
  size_t tensor_map_count() const { return maps_.size(); }
  const std::vector<uint64_t> &raw_slots() const { return slots_; }
  bool empty() const { return order_.empty(); }

  // kernelParams array: one pointer per parameter, in the order added.
  // Valid until the next add_* call.
  void **params();

private:
  struct Ref {
    bool is_map; // a 64-byte aligned blob (tensor map or struct) rather than an 8-byte slot
    size_t index;
  };
  struct alignas(64) Blob {
    unsigned char bytes[kMaxStructBytes];
  };
  std::vector<uint64_t> slots_;
  std::deque<Blob> maps_; // deque: stable addresses
  std::vector<Ref> order_;
  std::vector<void *> params_;
};

} // namespace kh
