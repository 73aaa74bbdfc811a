// test/unit/e2e_gemm_test.cpp:70-122 through a C ABI.
#include "test/unit/e2e_gemm_test.cpp"

extern "C" void khref_gemm_fill(float *a, float *b, long m, long n, long k) {
  for (long i = 0; i < m; ++i)
    for (long kk = 0; kk < k; ++kk) a[i * k + kk] = fill_a_value(i, kk);
  for (long kk = 0; kk < k; ++kk)
    for (long j = 0; j < n; ++j) b[kk * n + j] = fill_b_value(kk, j);
}

extern "C" void khref_gemm_ref(const float *a, const float *b, float *out, long m, long n, long k) {
  std::vector<float> va(a, a + m * k), vb(b, b + k * n), vr(static_cast<size_t>(m * n));
  fill_reference(va, vb, vr, m, n, k);
  std::copy(vr.begin(), vr.end(), out);
}

extern "C" double khref_gemm_rel_frobenius(const float *c, const float *ref, long count) {
  std::vector<float> vc(c, c + count), vr(ref, ref + count);
  return relative_frobenius(vc, vr, static_cast<size_t>(count));
}

// Row-sliced use of the reference's fill_reference for timing it on several
// host threads: B is held once, each call forms C rows for the A rows given.
namespace {
struct GemmPrepared {
  std::vector<float> b;
  long n = 0, k = 0;
};
} // namespace

extern "C" void *khref_gemm_prepare(const float *b, long n, long k) {
  auto *h = new GemmPrepared;
  h->b.assign(b, b + k * n);
  h->n = n;
  h->k = k;
  return h;
}

extern "C" void khref_gemm_rows(void *handle, const float *a_rows, float *out, long rows) {
  auto *h = static_cast<GemmPrepared *>(handle);
  std::vector<float> va(a_rows, a_rows + rows * h->k), vr(static_cast<size_t>(rows * h->n));
  fill_reference(va, h->b, vr, rows, h->n, h->k);
  std::copy(vr.begin(), vr.end(), out);
}

extern "C" void khref_gemm_release(void *handle) { delete static_cast<GemmPrepared *>(handle); }
