// results.csv writer. Header and quoting are the reference's
// (bench/harness/csv.cpp:9-57): exactly
// kernel,shape,backend,ms_median,gflops_or_gbps,timestamp,device
// Extra columns, when asked for, are appended after those seven so existing
// consumers keep parsing the first seven.
#pragma once

#include <iosfwd>
#include <string>
#include <vector>

namespace kh::bench {

struct BenchRow {
  std::string kernel, shape, backend;
  double ms_median = 0.0;
  double gflops_or_gbps = 0.0;
  std::string timestamp, device;
  // appended columns
  int gpus = 1;
  double roofline_frac = 0.0;
  double max_rel_err = -1.0; // < 0: not checked
  double cpu_ms = -1.0;      // < 0: not timed
  int cpu_cores = 0;
};

extern const char *const kCsvHeader;
extern const char *const kCsvExtendedHeader;
std::string csv_escape(const std::string &field);
std::string csv_line(const BenchRow &row);
std::string csv_line_extended(const BenchRow &row);
bool write_results_csv(std::ostream &out, const std::vector<BenchRow> &rows, bool extended = false);

} // namespace kh::bench
