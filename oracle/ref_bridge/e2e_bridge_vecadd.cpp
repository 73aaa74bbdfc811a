// test/unit/e2e_vecadd_test.cpp:40-46 through a C ABI. (The fp64 reference of
// that test is inline in the test body, so only the generator can be taken
// from the reference's own code.)
#include "test/unit/e2e_vecadd_test.cpp"

extern "C" void khref_vecadd_fill(float *a, float *b, long n) {
  std::vector<float> va(static_cast<size_t>(n)), vb(static_cast<size_t>(n));
  fill_inputs(va, vb);
  std::copy(va.begin(), va.end(), a);
  std::copy(vb.begin(), vb.end(), b);
}
