#include "device_limits.hpp"

#include <atomic>
#include <cstring>
#include <stdexcept>

namespace kh {

// AMD Navi 32 and the A100-class cross target: the values the reference
// ships (lib/compiler/device_limits.cpp:45-54 and 81-90), kept so existing
// callers of those tokens see the same numbers. New fields are 0 there.
const DeviceLimits gfx1101_limits = {65536, 32, 1024, {2147483647, 65535, 65535}, 17163091968L,
                                     32,    6144, 0,  "AMD Navi 32 (gfx1101)",     0,
                                     0,     0,    0};

const DeviceLimits sm_80_limits = {49152, 32,    1024, {2147483647, 65535, 65535},         0L,
                                   64,    65536, 0,    "NVIDIA A100-class (sm_80, cross)", 0,
                                   0,     0,     0};

// NVIDIA B200 (compute capability 10.0, built as sm_100a).
//   lds_bytes_per_workgroup 49152: static shared memory per block without opt-in (48 KiB).
//   max_dynamic_smem_optin 232448: 227 KiB per block once the kernel opts in
//     (cuFuncSetAttribute MAX_DYNAMIC_SHARED_SIZE_BYTES).
//   smem_per_sm 233472: 228 KiB per SM (1 KiB per resident block is reserved).
//   64 resident warps, 65536 registers, 32 resident blocks per SM.
//   tmem_columns_per_sm 512: tensor memory is 128 lanes x 512 32-bit columns.
//   vram_bytes and cu_count come from the live device (148 SMs, ~180 GB).
const DeviceLimits sm_100a_limits = {49152, 32,    1024, {2147483647, 65535, 65535}, 0L,
                                     64,    65536, 0,    "NVIDIA B200 (sm_100a)",    232448,
                                     233472, 32,   512};

namespace {
struct Entry {
  const char *token;
  const DeviceLimits *limits;
};
const Entry kTable[] = {{"gfx1101", &gfx1101_limits}, {"sm_80", &sm_80_limits},
                        {"sm_100a", &sm_100a_limits}};

struct CliEntry {
  const char *cli;
  const char *token;
};
const CliEntry kCliTable[] = {{"amdgcn-gfx1101", "gfx1101"}, {"nvptx-sm_80", "sm_80"},
                              {"nvptx-sm_100a", "sm_100a"}};

std::atomic<long> g_runtime_cu_count{0};
} // namespace

std::vector<std::string> known_device_targets() {
  std::vector<std::string> out;
  for (const Entry &e : kTable) out.emplace_back(e.token);
  return out;
}

const DeviceLimits &device_limits_for(const char *target_name) {
  if (target_name != nullptr)
    for (const Entry &e : kTable)
      if (std::strcmp(e.token, target_name) == 0) return *e.limits;
  std::string list;
  for (const Entry &e : kTable) {
    if (!list.empty()) list += ", ";
    list += e.token;
  }
  throw std::invalid_argument("unknown device target \"" +
                              std::string(target_name ? target_name : "(null)") +
                              "\"; known targets: " + list);
}

std::string device_token_for_cli_target(const std::string &cli_target) {
  for (const CliEntry &e : kCliTable)
    if (cli_target == e.cli) return e.token;
  return "";
}

std::vector<std::string> known_cli_targets() {
  std::vector<std::string> out;
  for (const CliEntry &e : kCliTable) out.emplace_back(e.cli);
  return out;
}

void set_runtime_cu_count(long count) { g_runtime_cu_count.store(count); }
long query_cu_count_runtime() { return g_runtime_cu_count.load(); }
long query_cu_count(const DeviceLimits &limits) {
  const long live = query_cu_count_runtime();
  return live > 0 ? live : limits.cu_count;
}

} // namespace kh
