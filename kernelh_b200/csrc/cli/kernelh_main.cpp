// kernelh - command-line front end over the C ABI, with the reference CLI's
// grammar (tools/kernelh/main.cpp:129-158, 222-266): `--flag value` or
// `--flag=value`, shapes as k=v,k=v, exit codes 0 ok / 1 operational / 2 usage,
// 77 when no CUDA driver or device is usable (bench/harness/run_bench.hpp:5-10).
//
//   kernelh compile --kernel K --shape S --target nvptx-sm_100a --out DIR
//       writes DIR/K.cubin (the prebuilt sm_100a code object) and DIR/resources.json
//       (registers, shared memory, occupancy estimate of the entry point), prints
//       "wrote <file>" lines and "compile ok" like the reference's compile.
//   kernelh run     --kernel K --shape S [--target nvptx-sm_100a] [--seed N] [--dump FILE]
//       fills the inputs deterministically, launches once, prints a digest of
//       every output (new verb; the reference has none).
//   kernelh bench   --kernel K --shape S [--warmup W] [--iters N] [--gpus G] [--out DIR]
//   kernelh bench   --suite kernelh [--out DIR] [--peak-gbs G --peak-tflops T]
//       warm-up + median of event-timed launches, one results.csv row per kernel; with the
//       measured peaks also DIR/results_b200.csv, whose rows append gpus, roofline_frac,
//       max_rel_err, cpu_ms, cpu_cores after the reference's seven columns.
//   kernelh bench   --occupancy --kernel K --shape S --target T [--out DIR]
//       the analytic occupancy report of the launches the library would make, fed with
//       the registers and static shared memory ptxas reported for each entry point;
//       with --out also DIR/occupancy.json and DIR/occupancy.md.
#include "kernelh_b200.h"

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <fstream>
#include <map>
#include <string>
#include <sys/stat.h>
#include <vector>

namespace {

constexpr int kExitOk = 0, kExitFail = 1, kExitUsage = 2;

struct Flags {
  std::map<std::string, std::vector<std::string>> values;
  bool has(const std::string &k) const { return values.count(k) != 0; }
  std::string get(const std::string &k, const std::string &dflt = "") const {
    auto it = values.find(k);
    return it == values.end() || it->second.empty() ? dflt : it->second.back();
  }
};

bool parse_flags(int argc, char **argv, int first, Flags &out, std::string &error) {
  static const char *boolean[] = {"--occupancy", "--help"};
  for (int i = first; i < argc; ++i) {
    std::string a = argv[i];
    if (a.rfind("--", 0) != 0) {
      error = "unexpected argument '" + a + "'";
      return false;
    }
    const size_t eq = a.find('=');
    if (eq != std::string::npos) {
      out.values[a.substr(0, eq)].push_back(a.substr(eq + 1));
      continue;
    }
    bool is_bool = false;
    for (const char *b : boolean) is_bool = is_bool || a == b;
    if (is_bool) {
      out.values[a].push_back("1");
      continue;
    }
    if (i + 1 >= argc) {
      error = "flag '" + a + "' needs a value";
      return false;
    }
    out.values[a].push_back(argv[++i]);
  }
  return true;
}

int usage(const char *why) {
  if (why && *why) std::fprintf(stderr, "kernelh: %s\n", why);
  std::fprintf(stderr,
               "usage: kernelh <compile|run|bench> --kernel <name> --shape k=v,k=v [--target nvptx-sm_100a]\n"
               "       compile: --out <dir>      run: [--seed N] [--dump <file>]\n"
               "       bench:   [--warmup W] [--iters N] [--gpus G] [--out <dir>] | --suite kernelh | --occupancy\n");
  return kExitUsage;
}

// The reference tests' LCG (test/unit/e2e_softmax_test.cpp:67-74): values on a
// 2^16-point grid in [-1, 1).
void fill_lcg(std::vector<float> &v, uint32_t &seed) {
  for (float &x : v) {
    seed = seed * 1664525u + 1013904223u;
    x = static_cast<float>(static_cast<int32_t>(seed >> 8) & 0xffff) / 32768.0f - 1.0f;
  }
}

uint64_t fnv1a(const void *data, size_t bytes) {
  const unsigned char *p = static_cast<const unsigned char *>(data);
  uint64_t h = 0xcbf29ce484222325ull;
  for (size_t i = 0; i < bytes; ++i) {
    h ^= p[i];
    h *= 0x100000001b3ull;
  }
  return h;
}

std::string timestamp_utc() {
  const std::time_t t = std::time(nullptr);
  char buf[32];
  std::strftime(buf, sizeof buf, "%Y-%m-%dT%H:%M:%SZ", std::gmtime(&t));
  return buf;
}

bool check_target(const Flags &f, bool required, std::string &token) {
  if (!f.has("--target")) {
    if (required) {
      std::fprintf(stderr, "kernelh: --target is required (valid --target values: nvptx-sm_100a)\n");
      return false;
    }
    token = "sm_100a";
    return true;
  }
  for (const std::string &t : f.values.at("--target")) {
    char buf[64];
    if (kh_target_token(t.c_str(), buf, sizeof buf) != 0) {
      std::fprintf(stderr, "kernelh: %s\n", kh_last_error());
      return false;
    }
    if (std::string(buf) != "sm_100a") {
      std::fprintf(stderr, "kernelh: target '%s' is known but this build only carries sm_100a code "
                           "objects (valid --target values: nvptx-sm_100a)\n", t.c_str());
      return false;
    }
    token = buf;
  }
  return true;
}

// Buffer element counts per tensor, in template order, from the shape.
bool tensor_sizes(const std::string &kernel, const std::map<std::string, long long> &s,
                  std::vector<size_t> &sizes, std::vector<bool> &is_output) {
  auto g = [&](const char *k) { auto it = s.find(k); return it == s.end() ? 0ll : it->second; };
  if (kernel == "vecadd") { sizes = {size_t(g("n")), size_t(g("n")), size_t(g("n"))}; is_output = {false, false, true}; }
  else if (kernel == "fused_gelu") {
    const size_t n = g("n") ? size_t(g("n")) : size_t(g("rows") * g("cols"));
    sizes = {n, n, n}; is_output = {false, false, true};
  }
  else if (kernel == "scan") { sizes = {size_t(g("n")), size_t(g("n"))}; is_output = {false, true}; }
  else if (kernel == "softmax") { const size_t e = size_t(g("rows") * g("cols")); sizes = {e, e}; is_output = {false, true}; }
  else if (kernel == "layernorm") {
    const size_t e = size_t(g("rows") * g("cols"));
    sizes = {e, size_t(g("cols")), size_t(g("cols")), e}; is_output = {false, false, false, true};
  }
  else if (kernel == "gemm") {
    sizes = {size_t(g("m") * g("k")), size_t(g("k") * g("n")), size_t(g("m") * g("n"))};
    is_output = {false, false, true};
  }
  else if (kernel == "attention") {
    const size_t e = size_t(g("batch") * g("heads") * g("seq") * g("head_dim"));
    sizes = {e, e, e, e}; is_output = {false, false, false, true};
  }
  else return false;
  return true;
}

std::map<std::string, long long> parse_shape(const std::string &text) {
  std::map<std::string, long long> out;
  size_t pos = 0;
  while (pos <= text.size()) {
    const size_t comma = text.find(',', pos);
    const std::string item = text.substr(pos, comma == std::string::npos ? std::string::npos : comma - pos);
    const size_t eq = item.find('=');
    if (eq == std::string::npos || eq == 0 || eq + 1 >= item.size()) return {};
    char *end = nullptr;
    const long long v = std::strtoll(item.c_str() + eq + 1, &end, 10);
    if (*end != '\0') return {};
    out[item.substr(0, eq)] = v;
    if (comma == std::string::npos) break;
    pos = comma + 1;
  }
  return out;
}

int cmd_compile(const Flags &f) {
  if (!f.has("--kernel") || !f.has("--out")) return usage("compile needs --kernel and --out");
  std::string token;
  if (!check_target(f, true, token)) return kExitFail;
  const std::string kernel = f.get("--kernel"), out = f.get("--out");
  if (f.has("--shape")) {
    kh_plan_info plan;
    if (kh_plan(kernel.c_str(), f.get("--shape").c_str(), token.c_str(), 0, &plan) != 0) {
      std::fprintf(stderr, "kernelh: %s\n", kh_last_error());
      return kExitFail;
    }
  }
  const void *image = nullptr;
  size_t size = 0;
  if (kh_kernel_image(kernel.c_str(), &image, &size) != 0) {
    std::fprintf(stderr, "kernelh: %s\n", kh_last_error());
    return kExitFail;
  }
  ::mkdir(out.c_str(), 0755);
  const std::string path = out + "/" + kernel + ".cubin";
  std::ofstream file(path, std::ios::binary);
  file.write(static_cast<const char *>(image), static_cast<std::streamsize>(size));
  if (!file.good()) {
    std::fprintf(stderr, "kernelh: cannot write %s\n", path.c_str());
    return kExitFail;
  }
  std::printf("wrote %s\n", path.c_str());
  // the resource figures of the kernel's entry point, beside the code object
  std::vector<char> json(4096);
  if (kh_kernel_resources(kernel.c_str(), nullptr, token.c_str(), json.data(), static_cast<int>(json.size()), nullptr) != 0) {
    std::fprintf(stderr, "kernelh: %s\n", kh_last_error());
    return kExitFail;
  }
  const std::string rpath = out + "/resources.json";
  std::ofstream rfile(rpath, std::ios::binary);
  rfile << json.data();
  if (!rfile.good()) {
    std::fprintf(stderr, "kernelh: cannot write %s\n", rpath.c_str());
    return kExitFail;
  }
  std::printf("wrote %s\ncompile ok\n", rpath.c_str());
  return kExitOk;
}

int open_context(kh_context **ctx) {
  const int rc = kh_context_create(0, ctx);
  if (rc == 0) return 0;
  std::fprintf(stderr, "kernelh: %s\n", kh_last_error());
  return rc == 77 ? 77 : kExitFail;
}

int cmd_run(const Flags &f) {
  if (!f.has("--kernel") || !f.has("--shape")) return usage("run needs --kernel and --shape");
  std::string token;
  if (!check_target(f, false, token)) return kExitFail;
  const std::string kernel = f.get("--kernel"), shape = f.get("--shape");
  kh_plan_info plan;
  if (kh_plan(kernel.c_str(), shape.c_str(), token.c_str(), 0, &plan) != 0) {
    std::fprintf(stderr, "kernelh: %s\n", kh_last_error());
    return kExitFail;
  }
  std::vector<size_t> sizes;
  std::vector<bool> is_output;
  if (!tensor_sizes(kernel, parse_shape(shape), sizes, is_output)) return usage("unknown kernel for run");
  kh_context *ctx = nullptr;
  if (int rc = open_context(&ctx)) return rc;
  uint32_t seed = static_cast<uint32_t>(std::strtoul(f.get("--seed", "2599699").c_str(), nullptr, 0));
  std::vector<std::vector<float>> host(sizes.size());
  std::vector<void *> ptrs;
  for (size_t i = 0; i < sizes.size(); ++i) {
    host[i].assign(sizes[i], 0.f);
    if (!is_output[i]) fill_lcg(host[i], seed);
    ptrs.push_back(host[i].data());
  }
  const auto t0 = std::chrono::steady_clock::now();
  const int rc = kh_run_host(ctx, kernel.c_str(), shape.c_str(), ptrs.data(), static_cast<int>(ptrs.size()));
  const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
  if (rc != 0) {
    std::fprintf(stderr, "kernelh: %s\n", kh_last_error());
    kh_context_destroy(ctx);
    return rc == 77 ? 77 : kExitFail;
  }
  for (size_t i = 0; i < sizes.size(); ++i)
    if (is_output[i]) {
      std::printf("run: %s [%s] output %zu: %zu elements fnv1a=%016llx first=%.9g last=%.9g\n",
                  kernel.c_str(), shape.c_str(), i, sizes[i],
                  static_cast<unsigned long long>(fnv1a(host[i].data(), sizes[i] * 4)), host[i].front(),
                  host[i].back());
      if (f.has("--dump")) {
        std::ofstream d(f.get("--dump"), std::ios::binary);
        d.write(reinterpret_cast<const char *>(host[i].data()), static_cast<std::streamsize>(sizes[i] * 4));
      }
    }
  std::printf("run ok (%.3f ms including host<->device copies)\n", ms);
  kh_context_destroy(ctx);
  return kExitOk;
}

struct Row { std::string kernel, shape; };

std::vector<Row> suite_rows() {
  // bench/harness/suites.cpp:22-44
  std::vector<Row> rows;
  for (long n : {512L, 1024L, 2048L, 4096L, 8192L})
    rows.push_back({"gemm", "m=" + std::to_string(n) + ",n=" + std::to_string(n) + ",k=" + std::to_string(n)});
  for (auto rc : {std::pair<long, long>{4096, 1024}, {16384, 4096}}) {
    const std::string s = "rows=" + std::to_string(rc.first) + ",cols=" + std::to_string(rc.second);
    rows.push_back({"softmax", s});
    rows.push_back({"layernorm", s});
  }
  for (long n : {100000L, 1000000L}) rows.push_back({"scan", "n=" + std::to_string(n)});
  for (long n : {1048576L, 4194304L}) rows.push_back({"fused_gelu", "n=" + std::to_string(n)});
  for (long s : {512L, 1024L}) rows.push_back({"attention", "batch=2,heads=8,seq=" + std::to_string(s) + ",head_dim=64"});
  return rows;
}

int cmd_bench(const Flags &f) {
  std::string token;
  if (f.has("--occupancy")) {
    if (!f.has("--kernel") || !f.has("--shape")) return usage("bench --occupancy needs --kernel and --shape");
    if (!check_target(f, true, token)) return kExitFail;
    std::vector<char> json(16384), md(16384);
    if (kh_occupancy_report(f.get("--kernel").c_str(), f.get("--shape").c_str(), token.c_str(), 148, json.data(),
                            static_cast<int>(json.size()), md.data(), static_cast<int>(md.size())) != 0) {
      std::fprintf(stderr, "kernelh: %s\n", kh_last_error());
      return kExitFail;
    }
    std::fputs(json.data(), stdout);
    if (f.has("--out")) {
      ::mkdir(f.get("--out").c_str(), 0755);
      for (const auto &[name, text] : {std::pair<const char *, const char *>{"occupancy.json", json.data()},
                                       {"occupancy.md", md.data()}}) {
        const std::string path = f.get("--out") + "/" + name;
        std::ofstream file(path, std::ios::binary);
        file << text;
        if (!file.good()) {
          std::fprintf(stderr, "kernelh: cannot write %s\n", path.c_str());
          return kExitFail;
        }
        std::printf("wrote %s\n", path.c_str());
      }
    }
    return kExitOk;
  }
  std::vector<Row> rows;
  if (f.has("--suite")) {
    if (f.get("--suite") != "kernelh" && f.get("--suite") != "all")
      return usage("--suite must be 'kernelh' (the other reference suites are AMD/vendor baselines)");
    rows = suite_rows();
  } else {
    if (!f.has("--kernel") || !f.has("--shape")) return usage("bench needs --kernel and --shape, or --suite");
    rows.push_back({f.get("--kernel"), f.get("--shape")});
  }
  if (!check_target(f, false, token)) return kExitFail;
  const int warmup = std::atoi(f.get("--warmup", "5").c_str());
  const int iters = std::atoi(f.get("--iters", "20").c_str());
  const int gpus = std::atoi(f.get("--gpus", "1").c_str());
  if (gpus < 1 || gpus > 8) return usage("--gpus must be between 1 and 8");
  kh_context *ctx = nullptr;
  if (int rc = open_context(&ctx)) return rc;
  kh_device_info info;
  kh_device_info_get(ctx, &info);
  std::string csv, csv_ext;
  char line[2048];
  kh_csv_header(line, sizeof line);
  csv = std::string(line) + "\n";
  // with --peak-gbs / --peak-tflops (the measured HBM and tensor peaks) a second file carries the
  // appended columns: gpus, roofline_frac, max_rel_err, cpu_ms, cpu_cores (the last three empty here:
  // the library holds no CPU implementation to check or time against)
  const double peak_gbs = std::atof(f.get("--peak-gbs", "0").c_str());
  const double peak_gflops = std::atof(f.get("--peak-tflops", "0").c_str()) * 1e3;
  kh_csv_header_ext(line, sizeof line);
  csv_ext = std::string(line) + "\n";
  int failures = 0;
  // --gpus N (2..8): gemm and attention rows are partitioned over the GPUs (kh_bench_sharded); the
  // other kernels are not partitioned anywhere, so their rows run as N independent replicas, one
  // per GPU, and report the sum of the rates beside the slowest replica's time.
  std::vector<kh_context *> replicas;
  for (int d = 1; d < gpus; ++d) {
    kh_context *c = nullptr;
    if (int rc = kh_context_create(d, &c)) {
      std::fprintf(stderr, "kernelh: GPU %d of %d: %s\n", d, gpus, kh_last_error());
      for (kh_context *r : replicas) kh_context_destroy(r);
      kh_context_destroy(ctx);
      return rc == 77 ? 77 : kExitFail;
    }
    replicas.push_back(c);
  }
  for (const Row &r : rows) {
    double ms = 0, rate = 0;
    int is_gflops = 0;
    const bool partitioned = gpus > 1 && (r.kernel == "gemm" || r.kernel == "attention");
    int rc = 0;
    if (partitioned) {
      rc = kh_bench_sharded(gpus, r.kernel.c_str(), r.shape.c_str(), warmup, iters, &ms, &rate, &is_gflops);
    } else {
      rc = kh_bench_row(ctx, r.kernel.c_str(), r.shape.c_str(), warmup, iters, &ms, &rate, &is_gflops);
      for (kh_context *c : replicas) {
        double ms_r = 0, rate_r = 0;
        if (rc == 0) rc = kh_bench_row(c, r.kernel.c_str(), r.shape.c_str(), warmup, iters, &ms_r, &rate_r, &is_gflops);
        ms = std::max(ms, ms_r);
        rate += rate_r;
      }
    }
    if (rc != 0) {
      std::fprintf(stderr, "kernelh: bench %s [%s] failed: %s\n", r.kernel.c_str(), r.shape.c_str(), kh_last_error());
      ++failures;
      continue;
    }
    std::printf("bench: kernelh %s [%s] ms_median=%.6f rate=%.3f %s%s\n", r.kernel.c_str(), r.shape.c_str(), ms,
                rate, is_gflops ? "GFLOPS" : "GB/s",
                gpus == 1 ? "" : (partitioned ? (" gpus=" + std::to_string(gpus) + " partitioned").c_str()
                                              : (" gpus=" + std::to_string(gpus) + " replicas").c_str()));
    kh_csv_line(r.kernel.c_str(), r.shape.c_str(), "kernelh", ms, rate, timestamp_utc().c_str(), info.name, line,
                sizeof line);
    csv += std::string(line) + "\n";
    const double peak = is_gflops ? peak_gflops : peak_gbs;
    kh_csv_line_ext(r.kernel.c_str(), r.shape.c_str(), "kernelh", ms, rate, timestamp_utc().c_str(), info.name, gpus,
                    peak > 0 ? rate / (peak * gpus) : 0.0, -1.0, -1.0, 0, line, sizeof line);
    csv_ext += std::string(line) + "\n";
  }
  if (f.has("--out")) {
    ::mkdir(f.get("--out").c_str(), 0755);
    const std::string path = f.get("--out") + "/results.csv";
    std::ofstream file(path);
    file << csv;
    std::printf("wrote %s\n", path.c_str());
    if (peak_gbs > 0 || peak_gflops > 0) {
      const std::string epath = f.get("--out") + "/results_b200.csv";
      std::ofstream efile(epath);
      efile << csv_ext;
      std::printf("wrote %s\n", epath.c_str());
    }
  }
  for (kh_context *c : replicas) kh_context_destroy(c);
  kh_context_destroy(ctx);
  return failures ? kExitFail : kExitOk;
}

} // namespace

int main(int argc, char **argv) {
  if (argc < 2) return usage("missing subcommand");
  const std::string cmd = argv[1];
  Flags flags;
  std::string error;
  if (!parse_flags(argc, argv, 2, flags, error)) return usage(error.c_str());
  if (cmd == "compile") return cmd_compile(flags);
  if (cmd == "run") return cmd_run(flags);
  if (cmd == "bench") return cmd_bench(flags);
  if (cmd == "--help" || cmd == "help") { usage(""); return kExitOk; }
  return usage(("unknown subcommand '" + cmd + "'").c_str());
}
