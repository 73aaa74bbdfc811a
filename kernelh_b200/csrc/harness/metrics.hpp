// Work counts and rates of the bench rows, the reference's conventions
// (bench/harness/metrics.cpp:14-52): GFLOPS = flops/s/1e9, GB/s = bytes/s/1e9.
#pragma once

namespace kh::bench {

double gflops_from_ms(double flops, double ms);
double gbps_from_ms(double bytes, double ms);
double gemm_flops(long m, long n, long k);
double gemm_bytes(long m, long n, long k);
double elementwise_bytes(long rows, long cols);
double layernorm_bytes(long rows, long cols);
double scan_bytes(long n);
double fused_gelu_bytes(long n);
double attention_flops(long batch, long heads, long seq, long head_dim);
double vecadd_bytes(long n); // new row: 3 * n * 4

} // namespace kh::bench
