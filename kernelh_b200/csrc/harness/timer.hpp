// Launch timing, the reference's method (bench/harness/timer.cpp:29-67):
// `warmup` untimed launches, a device sync, then `iters` launches each
// bracketed by start/end events and synchronised, and the median taken.
#pragma once

#include "../runtime/objects.hpp"

#include <functional>

namespace kh::bench {

constexpr int kDefaultWarmup = 5;
constexpr int kDefaultIters = 20;

Result<double> time_launch_median(const std::shared_ptr<Backend> &backend,
                                  const std::function<Result<void>()> &launch,
                                  int warmup = kDefaultWarmup, int iters = kDefaultIters,
                                  StreamHandle stream = nullptr);

} // namespace kh::bench
