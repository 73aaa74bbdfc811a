// Error type of the runtime: every call returns Result<T>; nothing throws
// across the runtime API. Mirrors the reference's
// include/kernelh/runtime/runtime_error.hpp:20-31 (Error{code, message},
// Result<T> = std::expected<T, Error>, skip code 77 when the driver is absent).
#pragma once

#include <expected>
#include <string>
#include <utility>

namespace kh {

// "Driver not available": callers that must skip GPU work exit with this code.
inline constexpr int kDriverUnavailable = 77;
// A device-side bounded wait ran out (see csrc/kernels/kh_device.cuh).
inline constexpr int kDeviceTimeout = 1001;

struct Error {
  int code = 0;
  std::string message;
  bool is_success() const { return code == 0; }
};

template <typename T> using Result = std::expected<T, Error>;

inline std::unexpected<Error> fail(int code, std::string message) {
  return std::unexpected(Error{code, std::move(message)});
}

} // namespace kh
