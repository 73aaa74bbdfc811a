// Device-limits table: the one place device constants live. Same contract as
// the reference's include/kernelh/compiler/device_limits.hpp:50-71 (exact-token
// lookup that throws std::invalid_argument naming the token and listing the
// known ones; cu_count 0 means "ask the runtime"), with a B200 entry and the
// extra fields a B200 launch needs (opt-in dynamic shared memory, shared
// memory per SM, resident blocks per SM, tensor-memory columns).
#pragma once

#include <string>
#include <vector>

namespace kh {

struct DeviceLimits {
  // --- the reference's fields, same meaning and order ---------------------
  long lds_bytes_per_workgroup;  // static shared memory a block may use without opt-in
  int wavefront_size;            // threads per warp
  int max_threads_per_workgroup; // max block size
  long max_grid_dim[3];
  long vram_bytes;     // 0 = unknown
  int waves_per_cu;    // resident warps per SM
  int reg_file_per_cu; // 32-bit registers per SM
  long cu_count;       // 0 = runtime query required
  const char *name;
  // --- added for sm_100a (0 = the target has no such limit / unknown) -----
  long max_dynamic_smem_optin; // static + dynamic bytes a block may use after opt-in
  long smem_per_sm;            // shared memory per SM
  int max_blocks_per_sm;       // resident blocks per SM
  int tmem_columns_per_sm;     // tensor-memory columns per SM (32-bit x 128 lanes each)
};

extern const DeviceLimits gfx1101_limits;
extern const DeviceLimits sm_80_limits;
extern const DeviceLimits sm_100a_limits;

// Exact match on "gfx1101" / "sm_80" / "sm_100a"; anything else (also null or
// empty) throws std::invalid_argument.
const DeviceLimits &device_limits_for(const char *target_name);
std::vector<std::string> known_device_targets();

// CLI target token -> table token ("nvptx-sm_100a" -> "sm_100a", ...), the
// mapping of the reference's tools/kernelh/main.cpp:375-390 plus the new
// target. Returns "" for an unknown CLI token.
std::string device_token_for_cli_target(const std::string &cli_target);
std::vector<std::string> known_cli_targets();

// SM count for occupancy math: a positive runtime value wins over the table.
void set_runtime_cu_count(long count);
long query_cu_count_runtime();
long query_cu_count(const DeviceLimits &limits);

} // namespace kh
