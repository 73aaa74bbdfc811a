// Analytic occupancy report. The three bounds, their tie-breaking and the
// percentage are those of the reference's lib/compiler/occupancy.cpp:124-223
// (VGPR-limited warps capped at waves_per_cu, floor(LDS/block), floor(max
// threads/threads), earlier bound wins ties, unknown inputs do not limit).
// For targets that describe an SM (smem_per_sm > 0) a second, per-SM view is
// added: resident blocks limited by registers, shared memory (1 KiB reserved
// per block), warps, the block cap and tensor-memory columns.
#pragma once

#include "device_limits.hpp"

#include <string>
#include <vector>

namespace kh {

enum class OccupancyLimiter { kNone = 0, kVgpr = 1, kLds = 2, kThreads = 3 };
const char *to_string(OccupancyLimiter l);

struct OccupancyInput {
  std::string kernel, target, config;
  int vgpr_count = 0;            // registers per thread
  long lds_bytes = 0;            // static shared bytes per block
  int threads_per_workgroup = 0;
  long dynamic_smem_bytes = 0;   // new
  int tmem_columns = 0;          // new: tensor-memory columns a block allocates
};

struct OccupancyReport {
  std::string kernel, target, config;
  int vgpr_count = 0;
  long lds_bytes = 0;
  int threads_per_workgroup = 0;
  int vgpr_limited_waves = 0, lds_limited_blocks = 0, thread_limited_blocks = 0;
  int achieved_waves = 0;
  double theoretical_pct = 0.0;
  OccupancyLimiter limiter = OccupancyLimiter::kNone;
  int measured_blocks = -1;
  double measured_pct = 0.0;
  std::string measured_note;
  // per-SM view (0 / "" when the target does not describe an SM)
  int sm_blocks_by_regs = 0, sm_blocks_by_smem = 0, sm_blocks_by_warps = 0, sm_blocks_by_cap = 0,
      sm_blocks_by_tmem = 0;
  int sm_resident_blocks = 0;
  double sm_occupancy_pct = 0.0;
  std::string sm_limiter;
};

OccupancyReport occupancy_report(const OccupancyInput &input, const DeviceLimits &limits,
                                 void *function = nullptr);
std::string occupancy_json(const OccupancyReport &report);
std::string occupancy_json_all(const std::vector<OccupancyReport> &reports);
std::string occupancy_markdown(const std::vector<OccupancyReport> &reports);

} // namespace kh
