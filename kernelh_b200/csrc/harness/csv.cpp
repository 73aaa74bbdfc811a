#include "csv.hpp"

#include <iomanip>
#include <ostream>
#include <sstream>

namespace kh::bench {

const char *const kCsvHeader = "kernel,shape,backend,ms_median,gflops_or_gbps,timestamp,device";
const char *const kCsvExtendedHeader =
    "kernel,shape,backend,ms_median,gflops_or_gbps,timestamp,device,gpus,roofline_frac,max_rel_err,"
    "cpu_ms,cpu_cores";

std::string csv_escape(const std::string &f) {
  if (f.find_first_of(",\"\n\r") == std::string::npos) return f;
  std::string out = "\"";
  for (char c : f) {
    if (c == '"') out += '"';
    out += c;
  }
  return out + "\"";
}

namespace {
std::string num(double v) {
  std::ostringstream os;
  os << std::setprecision(10) << v;
  return os.str();
}
} // namespace

std::string csv_line(const BenchRow &r) {
  return csv_escape(r.kernel) + "," + csv_escape(r.shape) + "," + csv_escape(r.backend) + "," +
         num(r.ms_median) + "," + num(r.gflops_or_gbps) + "," + csv_escape(r.timestamp) + "," +
         csv_escape(r.device);
}

std::string csv_line_extended(const BenchRow &r) {
  return csv_line(r) + "," + std::to_string(r.gpus) + "," + num(r.roofline_frac) + "," +
         (r.max_rel_err < 0 ? std::string() : num(r.max_rel_err)) + "," +
         (r.cpu_ms < 0 ? std::string() : num(r.cpu_ms)) + "," + std::to_string(r.cpu_cores);
}

bool write_results_csv(std::ostream &out, const std::vector<BenchRow> &rows, bool extended) {
  out << (extended ? kCsvExtendedHeader : kCsvHeader) << '\n';
  for (const BenchRow &r : rows) out << (extended ? csv_line_extended(r) : csv_line(r)) << '\n';
  return out.good();
}

} // namespace kh::bench
