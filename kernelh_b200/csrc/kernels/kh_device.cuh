// Shared device-side definitions for the sm_100a kernels.
//
// Device ABI. Every tensor argument arrives as the expanded memref descriptor
// the reference's code generator emits for a kernel parameter
// (lib/compiler/emitter.cpp:712-725): allocated pointer, aligned pointer,
// offset, sizes[N], strides[N] - 2N+3 eight-byte parameters, packed on the
// host by LaunchArgs::add_memref. The entry symbol equals the kernel name.
// The macros below declare those parameters; data is read at aligned+offset,
// and shapes are taken from the descriptor, not from compile-time constants.
#pragma once

#include <cstdint>

#define KH_MEMREF1(T, name)                                                                        \
  T *name##_alloc, T *name##_ptr, int64_t name##_off, int64_t name##_size0, int64_t name##_stride0
#define KH_MEMREF2(T, name)                                                                        \
  T *name##_alloc, T *name##_ptr, int64_t name##_off, int64_t name##_size0, int64_t name##_size1,  \
      int64_t name##_stride0, int64_t name##_stride1
#define KH_MEMREF4(T, name)                                                                        \
  T *name##_alloc, T *name##_ptr, int64_t name##_off, int64_t name##_size0, int64_t name##_size1,  \
      int64_t name##_size2, int64_t name##_size3, int64_t name##_stride0, int64_t name##_stride1,  \
      int64_t name##_stride2, int64_t name##_stride3
#define KH_DATA(name) ((name##_ptr) + (name##_off))

namespace khd {

// Status word protocol for kernels with waits (scan look-back, mbarrier
// pipelines): status[0] == 0 means clean; a wait that runs out of its
// iteration budget stores a non-zero code (first writer wins) and the kernel
// stops issuing work and returns. The host reads the word after the stream
// sync and maps it to an error. No trap, no device assert.
enum : uint32_t {
  kStatusOk = 0,
  kStatusScanLookbackTimeout = 1,
  kStatusTmaWaitTimeout = 2,
  kStatusMmaWaitTimeout = 3,
  kStatusEpilogueWaitTimeout = 4,
  kStatusEmptyWaitTimeout = 5,
  kStatusPeerArrivalTimeout = 6, // another GPU's arrival flag after a fused all-gather
};

__device__ __forceinline__ void report_status(uint32_t *status, uint32_t code, uint32_t detail) {
  if (status != nullptr && atomicCAS(status, 0u, code) == 0u) status[1] = detail;
}

// Programmatic dependent launch. A kernel launched with the "may overlap its predecessor's
// tail" attribute is scheduled while the previous kernel of the stream is still draining;
// grid_dependency_wait() holds it until that kernel has completed and its writes are visible
// (call it before the first global access), and grid_dependents_may_launch() tells the
// scheduler that the NEXT kernel's blocks may be placed as this kernel's blocks retire.
// Both are no-ops in a launch without the attribute.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependents_may_launch() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ bool is_aligned16(const void *p) {
  return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// The warp's maximum in one instruction (sm_100a's floating-point redux); NaN if any lane holds one.
__device__ __forceinline__ float warp_max_redux(float v) {
  float r;
  asm volatile("redux.sync.max.NaN.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}
// The same, NaN lanes ignored (the result is the largest number any lane holds).
__device__ __forceinline__ float warp_max_redux_numbers(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}
// 2^x by the special-function unit alone (about 2 ulp; denormal results flush to zero).
__device__ __forceinline__ float exp2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

} // namespace khd
