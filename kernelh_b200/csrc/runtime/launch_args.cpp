#include "launch_args.hpp"

#include <cstring>
#include <stdexcept>
#include <string>

namespace kh {

void LaunchArgs::add_memref(const void *dev_ptr, const std::vector<int64_t> &shape) {
  const uint64_t p = reinterpret_cast<uint64_t>(dev_ptr);
  auto push = [&](uint64_t v) {
    order_.push_back({false, slots_.size()});
    slots_.push_back(v);
  };
  push(p); // allocated pointer
  push(p); // aligned pointer
  push(0); // offset
  for (int64_t d : shape) push(static_cast<uint64_t>(d));
  std::vector<int64_t> strides(shape.size(), 1);
  for (size_t i = shape.size(); i-- > 1;) strides[i - 1] = strides[i] * shape[i];
  for (int64_t s : strides) push(static_cast<uint64_t>(s));
}

void LaunchArgs::add_scalar_bytes(const void *value, size_t byte_size) {
  uint64_t slot = 0;
  std::memcpy(&slot, value, byte_size > 8 ? 8 : byte_size);
  order_.push_back({false, slots_.size()});
  slots_.push_back(slot);
}

void LaunchArgs::add_tensor_map(const TensorMapBytes &map) { add_struct_bytes(&map, sizeof map); }

void LaunchArgs::add_struct_bytes(const void *value, size_t byte_size) {
  if (byte_size > kMaxStructBytes)
    throw std::length_error("LaunchArgs: a by-value kernel parameter of " + std::to_string(byte_size) +
                            " bytes exceeds the " + std::to_string(kMaxStructBytes) + " bytes a parameter may have here");
  Blob blob{};
  std::memcpy(blob.bytes, value, byte_size);
  order_.push_back({true, maps_.size()});
  maps_.push_back(blob);
}

void **LaunchArgs::params() {
  params_.resize(order_.size());
  for (size_t i = 0; i < order_.size(); ++i)
    params_[i] = order_[i].is_map ? static_cast<void *>(&maps_[order_[i].index])
                                  : static_cast<void *>(&slots_[order_[i].index]);
  return params_.data();
}

} // namespace kh
