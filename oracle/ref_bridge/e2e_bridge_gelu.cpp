// test/unit/e2e_fused_gelu_test.cpp:59-86 through a C ABI.
#include "test/unit/e2e_fused_gelu_test.cpp"

extern "C" void khref_gelu_fill(float *v, long n, unsigned *seed) {
  std::vector<float> tmp(static_cast<size_t>(n));
  uint32_t s = *seed;
  fill_rand(tmp, s);
  *seed = s;
  std::copy(tmp.begin(), tmp.end(), v);
}

extern "C" void khref_gelu_ref(const float *x, double *out, long n, int no_tanh) {
  for (long i = 0; i < n; ++i)
    out[i] = no_tanh ? gelu_no_tanh_reference(static_cast<double>(x[i]))
                     : gelu_reference(static_cast<double>(x[i]));
}
