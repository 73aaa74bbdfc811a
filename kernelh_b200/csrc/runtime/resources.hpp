// Per-kernel resource figures (registers per thread, static shared memory, spills,
// barriers) read from the `ptxas -v` text of the build, and the resources.json text made
// from them. Same source and the same schema as the reference's resource reporter for NVIDIA
// targets (lib/compiler/resource_reporter.cpp:353-363 runs `ptxas -v -arch=<chip>`, 614-660
// parses "Used N registers" / "M bytes smem", 674-690 writes resources.json; the occupancy
// estimate is 228-256: floor(register file / (registers x warp)), clamped to [1, warps per SM]).
// Here the text is captured once, when the code objects are built, for every entry point.
#pragma once

#include "device_limits.hpp"

#include <string>
#include <string_view>
#include <vector>

namespace kh {

struct EntryResources {
  std::string entry;      // entry symbol
  std::string arch;       // e.g. "sm_100a"
  int registers = 0;      // per thread
  long smem_bytes = 0;    // static shared memory per block
  long stack_bytes = 0, spill_store_bytes = 0, spill_load_bytes = 0;
  int barriers = 0;
  long cmem0_bytes = 0;
};

// Every "Compiling entry function '<name>' for '<arch>'" block of a ptxas -v report.
std::vector<EntryResources> parse_ptxas_report(std::string_view text);

// resources.json of one entry: the reference's seven keys (kernel, target, vgpr_count,
// sgpr_count, lds_bytes, wavefront_size, occupancy_estimate), then the figures ptxas gives
// beyond them. `target` is a device-limits token ("sm_100a").
std::string resources_json(const EntryResources &r, const std::string &kernel, const std::string &target);

// floor(register file / (registers x warp size)) clamped to [1, warps per SM]; 0 when unknown.
int occupancy_estimate(const DeviceLimits &limits, int registers);

} // namespace kh
