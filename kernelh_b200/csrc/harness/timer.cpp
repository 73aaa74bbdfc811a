#include "timer.hpp"

#include <algorithm>
#include <vector>

namespace kh::bench {

Result<double> time_launch_median(const std::shared_ptr<Backend> &backend,
                                  const std::function<Result<void>()> &launch, int warmup, int iters,
                                  StreamHandle stream) {
  if (iters <= 0) return fail(2, "time_launch_median: iters must be positive");
  for (int i = 0; i < warmup; ++i)
    if (auto r = launch(); !r) return std::unexpected(r.error());
  if (auto r = backend->device_synchronize(); !r) return std::unexpected(r.error());
  auto timer = EventTimer::create(backend);
  if (!timer) return std::unexpected(timer.error());
  std::vector<double> ms;
  ms.reserve(static_cast<size_t>(iters));
  for (int i = 0; i < iters; ++i) {
    if (auto r = timer->record_start(stream); !r) return std::unexpected(r.error());
    if (auto r = launch(); !r) return std::unexpected(r.error());
    if (auto r = timer->record_end(stream); !r) return std::unexpected(r.error());
    if (auto r = timer->synchronize(); !r) return std::unexpected(r.error());
    auto e = timer->elapsed_ms();
    if (!e) return std::unexpected(e.error());
    ms.push_back(*e);
  }
  std::sort(ms.begin(), ms.end());
  const size_t n = ms.size();
  return n % 2 ? ms[n / 2] : 0.5 * (ms[n / 2 - 1] + ms[n / 2]);
}

} // namespace kh::bench
