#include "resources.hpp"

#include <charconv>
#include <sstream>

namespace kh {
namespace {

// The decimal number that ends right before `marker` in `line` (e.g. "48 registers"), or -1.
long number_before(std::string_view line, std::string_view marker) {
  const size_t at = line.find(marker);
  if (at == std::string_view::npos || at == 0) return -1;
  size_t begin = at;
  while (begin > 0 && line[begin - 1] >= '0' && line[begin - 1] <= '9') --begin;
  if (begin == at) return -1;
  long value = 0;
  const auto [end, ec] = std::from_chars(line.data() + begin, line.data() + at, value);
  return ec == std::errc() && end == line.data() + at ? value : -1;
}

// Text between the n-th pair of single quotes of `line` (n = 0, 1, ...).
std::string_view quoted(std::string_view line, int n) {
  size_t pos = 0;
  for (int i = 0;; ++i) {
    const size_t open = line.find('\'', pos);
    if (open == std::string_view::npos) return {};
    const size_t close = line.find('\'', open + 1);
    if (close == std::string_view::npos) return {};
    if (i == n) return line.substr(open + 1, close - open - 1);
    pos = close + 1;
  }
}

std::string esc(const std::string &s) {
  std::string out;
  for (char c : s) {
    if (c == '"' || c == '\\') out += '\\';
    out += c;
  }
  return out;
}

} // namespace

std::vector<EntryResources> parse_ptxas_report(std::string_view text) {
  std::vector<EntryResources> out;
  size_t pos = 0;
  while (pos < text.size()) {
    size_t eol = text.find('\n', pos);
    if (eol == std::string_view::npos) eol = text.size();
    const std::string_view line = text.substr(pos, eol - pos);
    pos = eol + 1;
    if (line.find("Compiling entry function") != std::string_view::npos) {
      EntryResources e;
      e.entry = std::string(quoted(line, 0));
      e.arch = std::string(quoted(line, 1));
      out.push_back(std::move(e));
      continue;
    }
    if (out.empty()) continue; // module-level lines ("0 bytes gmem") come before the first entry
    EntryResources &e = out.back();
    if (const long v = number_before(line, " registers"); v >= 0 && line.find("Used ") != std::string_view::npos) {
      e.registers = static_cast<int>(v);
      if (const long b = number_before(line, " barriers"); b >= 0) e.barriers = static_cast<int>(b);
      if (const long s = number_before(line, " bytes smem"); s >= 0) e.smem_bytes = s;
      if (const long c = number_before(line, " bytes cmem[0]"); c >= 0) e.cmem0_bytes = c;
    }
    if (const long v = number_before(line, " bytes stack frame"); v >= 0) {
      e.stack_bytes = v;
      if (const long s = number_before(line, " bytes spill stores"); s >= 0) e.spill_store_bytes = s;
      if (const long l = number_before(line, " bytes spill loads"); l >= 0) e.spill_load_bytes = l;
    }
  }
  return out;
}

int occupancy_estimate(const DeviceLimits &l, int registers) {
  if (registers <= 0 || l.reg_file_per_cu <= 0 || l.wavefront_size <= 0 || l.waves_per_cu <= 0) return 0;
  long long warps = l.reg_file_per_cu / (1LL * registers * l.wavefront_size);
  if (warps < 1) warps = 1;
  if (warps > l.waves_per_cu) warps = l.waves_per_cu;
  return static_cast<int>(warps);
}

std::string resources_json(const EntryResources &r, const std::string &kernel, const std::string &target) {
  int warp = 0, estimate = 0;
  try {
    const DeviceLimits &l = device_limits_for(target.c_str());
    warp = l.wavefront_size;
    estimate = occupancy_estimate(l, r.registers);
  } catch (const std::exception &) {
    // unknown target: no estimate, as in the reference
  }
  std::ostringstream os;
  os << "{\n  \"kernel\": \"" << esc(kernel) << "\",\n  \"target\": \"" << esc(target) << "\",\n  \"vgpr_count\": "
     << r.registers << ",\n  \"sgpr_count\": 0,\n  \"lds_bytes\": " << r.smem_bytes << ",\n  \"wavefront_size\": " << warp
     << ",\n  \"occupancy_estimate\": " << estimate << ",\n  \"entry\": \"" << esc(r.entry) << "\",\n  \"arch\": \""
     << esc(r.arch) << "\",\n  \"barriers\": " << r.barriers << ",\n  \"stack_bytes\": " << r.stack_bytes
     << ",\n  \"spill_store_bytes\": " << r.spill_store_bytes << ",\n  \"spill_load_bytes\": " << r.spill_load_bytes
     << ",\n  \"source\": \"ptxas -v at build time\"\n}\n";
  return os.str();
}

} // namespace kh
