// Scaled fp16 hi/lo splits of fp32 data, shared by the tensor-core kernels.
//
// A group of values (a row of A, a column of B, one (batch, head) slice of Q, K
// or V) is scaled by an exact power of two that brings its largest magnitude
// into [2^14, 2^15), the upper part of the fp16 range; a scaled value x is then
// split into hi = fp16(x) (round to nearest) and lo = fp16(x - hi) (the
// difference is exact in fp32): 22 significand bits for every element within
// 2^-17 of the group's largest, an absolute floor of 2^-38 of the largest below.
#pragma once

#include <cuda_fp16.h>

#include "kh_device.cuh"

namespace khd {

constexpr int kTargetExponent = 14; // scaled maxima lie in [2^14, 2^15)

// Power-of-two exponent that brings a group whose largest magnitude is
// `amax` into the target range; 0 for an all-zero or non-finite row.
__device__ __forceinline__ int scale_shift(float amax) {
  if (!(amax > 0.f) || amax > 3.402823466e+38f) return 0;
  return kTargetExponent - ilogbf(amax);
}

// x * 2^e for |e| up to 378, exact unless the result leaves the normal fp32
// range: 2^e is applied as three factors, each a normal fp32 power of two.
__device__ __forceinline__ float pow2f(int e) { return __int_as_float((e + 127) << 23); }
__device__ __forceinline__ float scale_pow2(float x, int e) {
  const int e1 = max(-126, min(127, e));
  const int r = e - e1;
  const int e2 = max(-126, min(127, r));
  return x * pow2f(e1) * pow2f(e2) * pow2f(r - e2);
}

// The power of two a row (column) is scaled by, prepared once per row: one
// factor when 2^shift is a normal fp32 number, three otherwise.
struct RowScale {
  float f1, f2, f3;
  bool single;
};
__device__ __forceinline__ RowScale row_scale(int shift) {
  const int e1 = max(-126, min(127, shift));
  const int r = shift - e1;
  const int e2 = max(-126, min(127, r));
  return {pow2f(e1), pow2f(e2), pow2f(r - e2), r == 0};
}
// Two scaled values -> their fp16 hi parts and the fp16 of what hi left over.
// (x - hi is exact in fp32. An infinite input gives hi = inf and lo = NaN: the
// products are non-finite either way.)
__device__ __forceinline__ void split_fp16x2(float x0, float x1, const RowScale &sc, __half2 &hi, __half2 &lo) {
  float s0 = x0 * sc.f1, s1 = x1 * sc.f1;
  if (!sc.single) {
    s0 = s0 * sc.f2 * sc.f3;
    s1 = s1 * sc.f2 * sc.f3;
  }
  hi = __floats2half2_rn(s0, s1);
  const float2 h = __half22float2(hi);
  lo = __floats2half2_rn(s0 - h.x, s1 - h.y);
}

// The same for a group of pairs that share one scale, with the packed two-wide fp32 instructions
// of sm_100a (one multiply and one subtract per PAIR) and the rare three-factor scaling behind
// ONE branch for the whole group instead of predicated multiplies on every value: the split
// kernels are instruction-issue bound before they are HBM bound, and this halves their fp32 work.
template <int kPairs>
__device__ __forceinline__ void split_fp16_pairs(const float2 (&x)[kPairs], const RowScale &sc, __half2 (&hi)[kPairs],
                                                 __half2 (&lo)[kPairs]) {
  float2 s[kPairs];
  const float2 f1 = make_float2(sc.f1, sc.f1);
#pragma unroll
  for (int j = 0; j < kPairs; ++j) s[j] = __fmul2_rn(x[j], f1);
  if (!sc.single) {
    const float2 f2 = make_float2(sc.f2, sc.f2), f3 = make_float2(sc.f3, sc.f3);
#pragma unroll
    for (int j = 0; j < kPairs; ++j) s[j] = __fmul2_rn(__fmul2_rn(s[j], f2), f3);
  }
  const float2 minus_one = make_float2(-1.f, -1.f);
#pragma unroll
  for (int j = 0; j < kPairs; ++j) {
    hi[j] = __float22half2_rn(s[j]);
    lo[j] = __float22half2_rn(__ffma2_rn(__half22float2(hi[j]), minus_one, s[j])); // s - hi, exact
  }
}

struct alignas(16) Half8 {
  __half2 v[4];
};

} // namespace khd
