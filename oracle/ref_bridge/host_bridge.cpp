// C ABI over the reference's host-pure pieces (compiled from their sources by
// oracle/Makefile): descriptor packing, device-limits table, launch verifier,
// occupancy model, bench metrics, CSV line and shape-text parsing. Used to
// check the new runtime's host logic differentially.
#include "kernelh/compiler/device_limits.hpp"
#include "kernelh/compiler/launch_verifier.hpp"
#include "kernelh/compiler/occupancy.hpp"
#include "kernelh/runtime/descriptor_packing.hpp"

#include "bench/harness/csv.hpp"
#include "bench/harness/metrics.hpp"
#include "bench/harness/shape_text.hpp"

#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace {
int copy_out(const std::string &s, char *buf, int cap) {
  if (buf != nullptr && cap > 0) {
    const size_t n = s.size() < static_cast<size_t>(cap - 1) ? s.size() : static_cast<size_t>(cap - 1);
    std::memcpy(buf, s.data(), n);
    buf[n] = '\0';
  }
  return static_cast<int>(s.size());
}
} // namespace

extern "C" int khref_pack_memrefs(const unsigned long long *ptrs, const long long *shapes,
                                  const int *ranks, int count, unsigned long long *slots,
                                  int cap) {
  kernelh::runtime::LaunchArgs args;
  const long long *sp = shapes;
  for (int i = 0; i < count; ++i) {
    std::vector<int64_t> shape(sp, sp + ranks[i]);
    sp += ranks[i];
    args.add_memref(reinterpret_cast<const void *>(ptrs[i]), shape);
  }
  const auto &raw = args.raw_slots();
  for (size_t i = 0; i < raw.size() && static_cast<int>(i) < cap; ++i) slots[i] = raw[i];
  return static_cast<int>(raw.size());
}

// out[0..10]: lds, wavefront, max_threads, grid x/y/z, vram, waves_per_cu,
// reg_file, cu_count; returns 0, or 1 with the exception text in `msg`.
extern "C" int khref_device_limits(const char *token, long long *out, char *name, int name_cap,
                                   char *msg, int msg_cap) {
  try {
    const kernelh::DeviceLimits &l = kernelh::device_limits_for(token);
    out[0] = l.lds_bytes_per_workgroup;
    out[1] = l.wavefront_size;
    out[2] = l.max_threads_per_workgroup;
    out[3] = l.max_grid_dim[0];
    out[4] = l.max_grid_dim[1];
    out[5] = l.max_grid_dim[2];
    out[6] = l.vram_bytes;
    out[7] = l.waves_per_cu;
    out[8] = l.reg_file_per_cu;
    out[9] = l.cu_count;
    copy_out(l.name, name, name_cap);
    return 0;
  } catch (const std::invalid_argument &e) {
    copy_out(e.what(), msg, msg_cap);
    return 1;
  }
}

extern "C" int khref_verify_launch(const char *token, int threads, int gx, int gy, int gz,
                                   unsigned long long shared, int waves_per_cu_override,
                                   char *msg, int msg_cap) {
  kernelh::DeviceLimits l = kernelh::device_limits_for(token);
  if (waves_per_cu_override > 0) l.waves_per_cu = waves_per_cu_override;
  kernelh::compiler::LaunchConfig c{threads, gx, gy, gz, static_cast<size_t>(shared)};
  kernelh::compiler::LaunchVerifier v;
  auto r = v.verify(c, l);
  if (r.has_value()) return 0;
  copy_out(r.error(), msg, msg_cap);
  return 1;
}

// out: vgpr_limited_waves, lds_limited_blocks, thread_limited_blocks,
// achieved_waves, limiter (0 none,1 vgpr,2 lds,3 threads); pct returned.
extern "C" double khref_occupancy(const char *token, int vgpr, long lds, int threads, int *out) {
  kernelh::compiler::OccupancyInput in;
  in.kernel = "k";
  in.target = token;
  in.vgpr_count = vgpr;
  in.lds_bytes = lds;
  in.threads_per_workgroup = threads;
  const auto r = kernelh::compiler::occupancy_report(in, kernelh::device_limits_for(token));
  out[0] = r.vgpr_limited_waves;
  out[1] = r.lds_limited_blocks;
  out[2] = r.thread_limited_blocks;
  out[3] = r.achieved_waves;
  out[4] = static_cast<int>(r.limiter);
  return r.theoretical_pct;
}

extern "C" double khref_metric(const char *what, long a, long b, long c, long d) {
  using namespace kernelh::bench;
  const std::string w(what);
  if (w == "gemm_flops") return gemm_flops(a, b, c);
  if (w == "gemm_bytes") return gemm_bytes(a, b, c);
  if (w == "elementwise_bytes") return elementwise_bytes(a, b);
  if (w == "layernorm_bytes") return layernorm_bytes(a, b);
  if (w == "scan_bytes") return scan_bytes(a);
  if (w == "fused_gelu_bytes") return fused_gelu_bytes(a);
  if (w == "attention_flops") return attention_flops(a, b, c, d);
  return -1.0;
}

extern "C" double khref_rate(int gflops, double work, double ms) {
  return gflops ? kernelh::bench::gflops_from_ms(work, ms) : kernelh::bench::gbps_from_ms(work, ms);
}

extern "C" int khref_csv_line(const char *kernel, const char *shape, const char *backend,
                              double ms, double rate, const char *ts, const char *device,
                              char *buf, int cap) {
  kernelh::bench::BenchRow row;
  row.kernel = kernel;
  row.shape = shape;
  row.backend = backend;
  row.ms_median = ms;
  row.gflops_or_gbps = rate;
  row.timestamp = ts;
  row.device = device;
  return copy_out(kernelh::bench::csv_line(row), buf, cap);
}

extern "C" int khref_csv_header(char *buf, int cap) {
  return copy_out(kernelh::bench::kCsvHeader, buf, cap);
}

// Round trip of the shape grammar: parse, then print back ("" when rejected).
extern "C" int khref_shape_roundtrip(const char *text, char *buf, int cap) {
  const auto m = kernelh::bench::parse_shape_text(text);
  return copy_out(kernelh::bench::shape_to_text(m), buf, cap);
}
