// Pre-launch check of a concrete launch configuration against the device
// limits. Behaviour follows the reference's lib/compiler/launch_verifier.cpp:
// 109-172: every rule is evaluated, all violations come back in ONE
// newline-joined string, and the message texts of the five original rules are
// kept verbatim (its tests match on them). A sixth rule covers opt-in dynamic
// shared memory, which the reference never uses (it pins sharedMemBytes = 0).
#pragma once

#include "device_limits.hpp"

#include <cstddef>
#include <expected>
#include <functional>
#include <string>

namespace kh {

struct LaunchConfig {
  int threads_per_workgroup = 0;
  int grid_x = 0, grid_y = 0, grid_z = 0;
  size_t static_shared_bytes = 0;
  size_t dynamic_shared_bytes = 0; // new: opt-in dynamic shared memory
  int cluster_size = 1;            // new: CTAs per cluster (1 = no cluster)
};

// Occupancy source: resident blocks per SM for (function, block size, dynamic
// shared bytes), or -1 when no vendor answer is available. The CUDA backend
// installs one backed by cuOccupancyMaxActiveBlocksPerMultiprocessor.
using OccupancyQuery = std::function<int(void *function, int block_size, size_t dyn_shared)>;
void set_occupancy_query(OccupancyQuery query);
int query_occupancy_max_blocks_runtime(void *function, int block_size, size_t dyn_shared);

class LaunchVerifier {
public:
  std::expected<void, std::string> verify(const LaunchConfig &config, const DeviceLimits &limits,
                                          void *function = nullptr) const;
};

} // namespace kh
