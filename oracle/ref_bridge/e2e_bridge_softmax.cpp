// Exposes the reference's own softmax input generator and fp64 row reference
// (test/unit/e2e_softmax_test.cpp:67-91) through a C ABI, by including that
// translation unit where it lies in the reference tree.
#include "test/unit/e2e_softmax_test.cpp"

extern "C" void khref_softmax_fill(float *v, long n, unsigned *seed) {
  std::vector<float> tmp(static_cast<size_t>(n));
  uint32_t s = *seed;
  fill_rand(tmp, s);
  *seed = s;
  std::copy(tmp.begin(), tmp.end(), v);
}

extern "C" void khref_softmax_ref(const float *x, double *out, long rows, long cols) {
  std::vector<float> row(static_cast<size_t>(cols));
  std::vector<double> orow(static_cast<size_t>(cols));
  for (long r = 0; r < rows; ++r) {
    std::copy(x + r * cols, x + (r + 1) * cols, row.begin());
    softmax_reference_row(row, static_cast<size_t>(cols), orow);
    std::copy(orow.begin(), orow.end(), out + r * cols);
  }
}
