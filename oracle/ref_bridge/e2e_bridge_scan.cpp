// test/unit/e2e_scan_test.cpp:63-68 through a C ABI (generator only; the fp64
// reference of that test is inline in run_scan_e2e).
#include "test/unit/e2e_scan_test.cpp"

extern "C" void khref_scan_fill(float *v, long n, unsigned seed) {
  std::vector<float> tmp(static_cast<size_t>(n));
  fill_rand(tmp, seed);
  std::copy(tmp.begin(), tmp.end(), v);
}
