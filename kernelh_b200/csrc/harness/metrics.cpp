#include "metrics.hpp"

namespace kh::bench {

double gflops_from_ms(double flops, double ms) { return flops * 1000.0 / ms / 1e9; }
double gbps_from_ms(double bytes, double ms) { return bytes * 1000.0 / ms / 1e9; }
double gemm_flops(long m, long n, long k) { return 2.0 * double(m) * double(n) * double(k); }
double gemm_bytes(long m, long n, long k) {
  return (double(m) * k + double(k) * n + double(m) * n) * 4.0;
}
double elementwise_bytes(long rows, long cols) { return 2.0 * double(rows) * double(cols) * 4.0; }
double layernorm_bytes(long rows, long cols) {
  return 2.0 * double(rows) * double(cols) * 4.0 + 2.0 * double(cols) * 4.0;
}
double scan_bytes(long n) { return 2.0 * double(n) * 4.0; }
double fused_gelu_bytes(long n) { return 3.0 * double(n) * 4.0; }
double attention_flops(long batch, long heads, long seq, long head_dim) {
  return 4.0 * double(batch) * double(heads) * double(seq) * double(seq) * double(head_dim);
}
double vecadd_bytes(long n) { return 3.0 * double(n) * 4.0; }

} // namespace kh::bench
