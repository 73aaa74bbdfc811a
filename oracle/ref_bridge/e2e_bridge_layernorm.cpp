// test/unit/e2e_layernorm_test.cpp:57-91 through a C ABI.
#include "test/unit/e2e_layernorm_test.cpp"

extern "C" void khref_layernorm_fill(float *v, long n, unsigned *seed) {
  std::vector<float> tmp(static_cast<size_t>(n));
  uint32_t s = *seed;
  fill_rand(tmp, s);
  *seed = s;
  std::copy(tmp.begin(), tmp.end(), v);
}

extern "C" void khref_layernorm_ref(const float *x, const float *gamma, const float *beta,
                                    double *out, long rows, long cols, double eps) {
  std::vector<float> row(static_cast<size_t>(cols));
  std::vector<float> g(gamma, gamma + cols), b(beta, beta + cols);
  std::vector<double> orow(static_cast<size_t>(cols));
  for (long r = 0; r < rows; ++r) {
    std::copy(x + r * cols, x + (r + 1) * cols, row.begin());
    reference_row(row, static_cast<size_t>(cols), g, b, eps, orow);
    std::copy(orow.begin(), orow.end(), out + r * cols);
  }
}
