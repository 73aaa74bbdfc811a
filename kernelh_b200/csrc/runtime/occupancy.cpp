#include "occupancy.hpp"

#include "launch_verifier.hpp"

#include <algorithm>
#include <climits>
#include <cstdio>
#include <sstream>

namespace kh {

const char *to_string(OccupancyLimiter l) {
  switch (l) {
  case OccupancyLimiter::kVgpr: return "vgpr";
  case OccupancyLimiter::kLds: return "lds";
  case OccupancyLimiter::kThreads: return "threads";
  default: return "none";
  }
}

namespace {
std::string pct(double v) {
  char buf[64];
  std::snprintf(buf, sizeof buf, "%.4g", v);
  return buf;
}
std::string esc(const std::string &s) {
  std::string o;
  for (char c : s) {
    if (c == '"' || c == '\\') o += '\\';
    if (c == '\n') { o += "\\n"; continue; }
    o += c;
  }
  return o;
}
int warps_per_block(const DeviceLimits &l, int threads) {
  return l.wavefront_size > 0 ? (threads + l.wavefront_size - 1) / l.wavefront_size : 0;
}
} // namespace

OccupancyReport occupancy_report(const OccupancyInput &in, const DeviceLimits &l, void *function) {
  OccupancyReport r;
  r.kernel = in.kernel;
  r.target = in.target;
  r.config = in.config;
  r.vgpr_count = in.vgpr_count;
  r.lds_bytes = in.lds_bytes;
  r.threads_per_workgroup = in.threads_per_workgroup;

  const bool have_vgpr = in.vgpr_count > 0 && l.reg_file_per_cu > 0 && l.wavefront_size > 0;
  if (have_vgpr) {
    long long w = l.reg_file_per_cu / (1LL * in.vgpr_count * l.wavefront_size);
    w = std::clamp<long long>(w, 1, l.waves_per_cu);
    r.vgpr_limited_waves = static_cast<int>(w);
  }
  const bool have_lds = in.lds_bytes > 0 && l.lds_bytes_per_workgroup > 0;
  if (have_lds) r.lds_limited_blocks = static_cast<int>(l.lds_bytes_per_workgroup / in.lds_bytes);
  const bool have_thr = in.threads_per_workgroup > 0 && l.max_threads_per_workgroup > 0;
  if (have_thr) r.thread_limited_blocks = l.max_threads_per_workgroup / in.threads_per_workgroup;

  int best = INT_MAX;
  if (have_vgpr) { best = r.vgpr_limited_waves; r.limiter = OccupancyLimiter::kVgpr; }
  if (have_lds && r.lds_limited_blocks < best) { best = r.lds_limited_blocks; r.limiter = OccupancyLimiter::kLds; }
  if (have_thr && r.thread_limited_blocks < best) { best = r.thread_limited_blocks; r.limiter = OccupancyLimiter::kThreads; }
  if (best != INT_MAX) {
    r.achieved_waves = best;
    if (l.waves_per_cu > 0) r.theoretical_pct = 100.0 * best / l.waves_per_cu;
  }

  if (function != nullptr && in.threads_per_workgroup > 0) {
    const int blocks = query_occupancy_max_blocks_runtime(function, in.threads_per_workgroup,
                                                          static_cast<size_t>(in.dynamic_smem_bytes));
    if (blocks >= 0) {
      r.measured_blocks = blocks;
      if (l.waves_per_cu > 0)
        r.measured_pct = std::min(100.0, 100.0 * blocks * warps_per_block(l, in.threads_per_workgroup) /
                                             l.waves_per_cu);
    } else {
      r.measured_note = "driver occupancy query unavailable; measured_pct = 0 (analytic only)";
    }
  } else {
    r.measured_note = "no loaded kernel function; measured_pct = 0 (analytic only)";
  }

  // Per-SM view for targets that describe an SM.
  if (l.smem_per_sm > 0 && in.threads_per_workgroup > 0) {
    const int wpb = warps_per_block(l, in.threads_per_workgroup);
    int blocks = INT_MAX;
    std::string lim = "none";
    auto take = [&](int b, const char *what) { if (b < blocks) { blocks = b; lim = what; } };
    if (in.vgpr_count > 0) {
      // registers are allocated per warp in units of 256 (8 per thread)
      const int per_thread = (in.vgpr_count + 7) / 8 * 8;
      r.sm_blocks_by_regs = l.reg_file_per_cu / (per_thread * l.wavefront_size * std::max(wpb, 1));
      take(r.sm_blocks_by_regs, "registers");
    }
    const long smem = in.lds_bytes + in.dynamic_smem_bytes;
    if (smem > 0) {
      r.sm_blocks_by_smem = static_cast<int>(l.smem_per_sm / (smem + 1024));
      take(r.sm_blocks_by_smem, "shared memory");
    }
    if (wpb > 0) { r.sm_blocks_by_warps = l.waves_per_cu / wpb; take(r.sm_blocks_by_warps, "warps"); }
    if (l.max_blocks_per_sm > 0) { r.sm_blocks_by_cap = l.max_blocks_per_sm; take(r.sm_blocks_by_cap, "block cap"); }
    if (in.tmem_columns > 0 && l.tmem_columns_per_sm > 0) {
      r.sm_blocks_by_tmem = l.tmem_columns_per_sm / in.tmem_columns;
      take(r.sm_blocks_by_tmem, "tensor memory");
    }
    if (blocks != INT_MAX) {
      r.sm_resident_blocks = blocks;
      r.sm_limiter = lim;
      if (l.waves_per_cu > 0) r.sm_occupancy_pct = std::min(100.0, 100.0 * blocks * wpb / l.waves_per_cu);
    }
  }
  return r;
}

std::string occupancy_json(const OccupancyReport &r) {
  std::ostringstream os;
  os << "{\n  \"kernel\": \"" << esc(r.kernel) << "\",\n  \"target\": \"" << esc(r.target)
     << "\",\n  \"config\": \"" << esc(r.config) << "\",\n  \"vgpr_count\": " << r.vgpr_count
     << ",\n  \"lds_bytes\": " << r.lds_bytes << ",\n  \"threads_per_workgroup\": "
     << r.threads_per_workgroup << ",\n  \"vgpr_limited_waves\": " << r.vgpr_limited_waves
     << ",\n  \"lds_limited_blocks\": " << r.lds_limited_blocks << ",\n  \"thread_limited_blocks\": "
     << r.thread_limited_blocks << ",\n  \"theoretical_waves\": " << r.achieved_waves
     << ",\n  \"theoretical_pct\": " << pct(r.theoretical_pct) << ",\n  \"limiter\": \""
     << to_string(r.limiter) << "\",\n  \"measured_blocks\": " << r.measured_blocks
     << ",\n  \"measured_pct\": " << pct(r.measured_pct) << ",\n  \"measured_note\": \""
     << esc(r.measured_note) << "\",\n  \"sm_resident_blocks\": " << r.sm_resident_blocks
     << ",\n  \"sm_occupancy_pct\": " << pct(r.sm_occupancy_pct) << ",\n  \"sm_limiter\": \""
     << esc(r.sm_limiter) << "\"\n}";
  return os.str();
}

std::string occupancy_json_all(const std::vector<OccupancyReport> &reports) {
  std::string out = "{\n  \"reports\": [\n";
  for (size_t i = 0; i < reports.size(); ++i) {
    out += occupancy_json(reports[i]);
    out += i + 1 < reports.size() ? ",\n" : "\n";
  }
  return out + "  ]\n}\n";
}

std::string occupancy_markdown(const std::vector<OccupancyReport> &reports) {
  std::ostringstream os;
  os << "# Occupancy report\n\n| kernel | config | regs | smem (B) | theoretical % | measured % | "
        "limiter | blocks/SM | SM limiter |\n| --- | --- | ---: | ---: | ---: | ---: | --- | ---: | --- |\n";
  for (const OccupancyReport &r : reports) {
    std::string cfg = r.config;
    for (size_t p = 0; (p = cfg.find('|', p)) != std::string::npos; p += 2) cfg.replace(p, 1, "\\|");
    os << "| " << r.kernel << " | " << cfg << " | " << r.vgpr_count << " | " << r.lds_bytes << " | "
       << pct(r.theoretical_pct) << " | " << (r.measured_blocks >= 0 ? pct(r.measured_pct) : "n/a")
       << " | " << to_string(r.limiter) << " | " << r.sm_resident_blocks << " | " << r.sm_limiter
       << " |\n";
  }
  return os.str();
}

} // namespace kh
