#include "launch_verifier.hpp"

#include <mutex>
#include <vector>

namespace kh {
namespace {
std::mutex g_mu;
OccupancyQuery g_query;

const char *name_of(const DeviceLimits &l) { return l.name ? l.name : "(unknown device)"; }

std::string analytic_occupancy(const LaunchConfig &c, const DeviceLimits &l) {
  if (l.waves_per_cu <= 0 || l.wavefront_size <= 0 || c.threads_per_workgroup <= 0) return "";
  const long need = (static_cast<long>(c.threads_per_workgroup) + l.wavefront_size - 1) /
                    l.wavefront_size;
  if (need <= l.waves_per_cu) return "";
  return "occupancy would be 0 on target '" + std::string(name_of(l)) +
         "': threads per workgroup " + std::to_string(c.threads_per_workgroup) + " needs " +
         std::to_string(need) + " wavefronts, exceeding the target's per-CU budget of " +
         std::to_string(l.waves_per_cu) + " wavefronts (waves_per_cu * wavefront_size)";
}
} // namespace

void set_occupancy_query(OccupancyQuery query) {
  std::lock_guard<std::mutex> lock(g_mu);
  g_query = std::move(query);
}

int query_occupancy_max_blocks_runtime(void *function, int block_size, size_t dyn_shared) {
  OccupancyQuery q;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    q = g_query;
  }
  return q ? q(function, block_size, dyn_shared) : -1;
}

std::expected<void, std::string> LaunchVerifier::verify(const LaunchConfig &c,
                                                        const DeviceLimits &l,
                                                        void *function) const {
  std::vector<std::string> v;
  // 1. static shared memory against the per-block budget
  if (l.lds_bytes_per_workgroup > 0 &&
      c.static_shared_bytes > static_cast<size_t>(l.lds_bytes_per_workgroup))
    v.push_back("shared memory " + std::to_string(c.static_shared_bytes) + " bytes exceeds the " +
                std::to_string(l.lds_bytes_per_workgroup) + "-byte LDS limit for target '" +
                name_of(l) + "'");
  // 2. block size against the maximum
  if (l.max_threads_per_workgroup > 0 && c.threads_per_workgroup > l.max_threads_per_workgroup)
    v.push_back("threads per workgroup " + std::to_string(c.threads_per_workgroup) +
                " exceeds the max " + std::to_string(l.max_threads_per_workgroup));
  // 3. block size a multiple of the warp size
  if (l.wavefront_size > 1 && c.threads_per_workgroup > 0 &&
      c.threads_per_workgroup % l.wavefront_size != 0)
    v.push_back("threads per workgroup " + std::to_string(c.threads_per_workgroup) +
                " is not a multiple of the wavefront size " + std::to_string(l.wavefront_size));
  // 4. grid extents
  const long grid[3] = {c.grid_x, c.grid_y, c.grid_z};
  for (int i = 0; i < 3; ++i)
    if (l.max_grid_dim[i] > 0 && grid[i] > l.max_grid_dim[i]) {
      v.push_back("grid dim (" + std::to_string(grid[0]) + "," + std::to_string(grid[1]) + "," +
                  std::to_string(grid[2]) + ") exceeds the target grid limits");
      break;
    }
  // 6. dynamic shared memory: needs an opt-in capable target, and static +
  //    dynamic must fit the opt-in budget.
  if (c.dynamic_shared_bytes > 0) {
    const size_t total = c.static_shared_bytes + c.dynamic_shared_bytes;
    if (l.max_dynamic_smem_optin <= 0) {
      if (l.lds_bytes_per_workgroup > 0 && total > static_cast<size_t>(l.lds_bytes_per_workgroup))
        v.push_back("dynamic shared memory " + std::to_string(c.dynamic_shared_bytes) +
                    " bytes: static + dynamic " + std::to_string(total) + " bytes exceeds the " +
                    std::to_string(l.lds_bytes_per_workgroup) + "-byte limit for target '" +
                    name_of(l) + "', which has no opt-in carve-out");
    } else if (total > static_cast<size_t>(l.max_dynamic_smem_optin)) {
      v.push_back("dynamic shared memory " + std::to_string(c.dynamic_shared_bytes) +
                  " bytes: static + dynamic " + std::to_string(total) + " bytes exceeds the " +
                  std::to_string(l.max_dynamic_smem_optin) +
                  "-byte opt-in limit per block for target '" + name_of(l) + "'");
    }
  }
  if (c.cluster_size > 1 && (c.grid_x % c.cluster_size) != 0)
    v.push_back("grid dim x " + std::to_string(c.grid_x) + " is not a multiple of the cluster size " +
                std::to_string(c.cluster_size));
  // 5. occupancy > 0: vendor answer when a function handle is given, else analytic
  std::string occ;
  bool answered = false;
  if (function != nullptr && c.threads_per_workgroup > 0) {
    const int blocks = query_occupancy_max_blocks_runtime(function, c.threads_per_workgroup,
                                                          c.dynamic_shared_bytes);
    if (blocks >= 0) {
      answered = true;
      if (blocks == 0)
        occ = "occupancy would be 0 on target '" + std::string(name_of(l)) +
              "': the driver's occupancy query reported 0 resident blocks per multiprocessor "
              "for threads=" + std::to_string(c.threads_per_workgroup) + ", shared=" +
              std::to_string(c.static_shared_bytes + c.dynamic_shared_bytes) + " bytes";
    }
  }
  if (!answered) occ = analytic_occupancy(c, l);
  if (!occ.empty()) v.push_back(occ);

  if (v.empty()) return {};
  std::string out;
  for (size_t i = 0; i < v.size(); ++i) {
    if (i) out += '\n';
    out += v[i];
  }
  return std::unexpected(out);
}

} // namespace kh
