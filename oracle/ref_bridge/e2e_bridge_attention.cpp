// test/unit/e2e_attention_test.cpp:72-122 through a C ABI.
#include "test/unit/e2e_attention_test.cpp"

extern "C" void khref_attention_fill(float *v, long n, unsigned seed) {
  std::vector<float> tmp(static_cast<size_t>(n));
  fill_rand(tmp, seed);
  std::copy(tmp.begin(), tmp.end(), v);
}

// One (batch, head) problem: q, k, v, out are [seq, head_dim].
extern "C" void khref_attention_ref(const float *q, const float *k, const float *v, double *out,
                                    long seq, long head_dim, int scaled) {
  std::vector<float> kMat(k, k + seq * head_dim), vMat(v, v + seq * head_dim);
  std::vector<float> qRow(static_cast<size_t>(head_dim));
  std::vector<double> oRow(static_cast<size_t>(head_dim));
  for (long i = 0; i < seq; ++i) {
    std::copy(q + i * head_dim, q + (i + 1) * head_dim, qRow.begin());
    attention_reference_row(qRow, kMat, vMat, oRow, head_dim, scaled != 0);
    std::copy(oRow.begin(), oRow.end(), out + i * head_dim);
  }
}
