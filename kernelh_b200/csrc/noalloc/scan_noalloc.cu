// kh_scan_noalloc: the inclusive prefix sum for callers that are not allowed to
// allocate device memory.
//
// Who needs this. The ordinary scan entry points keep their look-back scratch
// (a ticket counter plus two 64-bit words per 4096-element tile) in a buffer
// the context allocates with cuMemAlloc on first use and grows on demand. Some
// hosts cannot do that: code running inside a memory pool or arena that owns
// every byte of the device and forbids side allocations, plugin callbacks that
// must not call an allocator because an allocation may synchronise the device,
// and code whose device memory budget is fixed and audited up front. For them
// the scratch here is a file-scope __device__ array that is part of the
// library's image: every GPU that loads the library carries it (65,552 bytes)
// until the process exits, and nothing is allocated or freed by the call.
//
// Limits and rules
//   * n <= kh_scan_noalloc_max_elements() (16,777,216); larger sizes are
//     refused with a usage error, never truncated.
//   * The first call on a device looks up the array's device address and the
//     SM count and raises the kernel's shared-memory limit (once per device,
//     with that device current). Make that first
//     call outside any stream capture.
//   * All calls on a device share the one array. The part a call uses is
//     cleared on the stream before its kernel, so a call never sees an earlier
//     call's contents; two calls that overlap on the GPU (different streams
//     without ordering) race on it and must be serialised by the caller.
//   * The device that owns x and y must be current; the call enqueues on
//     `stream` and returns without waiting.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

// The kernel is the library's scan kernel, compiled a second time into this
// translation unit under another entry name so that the existing code object
// and its launch path stay exactly as they are.
#define scan kh_scan_noalloc_kernel
#include "scan.cu"
#undef scan

extern "C" int kh_detail_set_error(int code, const char *message); // capi.cpp

namespace {

constexpr int64_t kMaxElements = int64_t(1) << 24;
constexpr int64_t kMaxTiles = kMaxElements / kTile; // 4096
constexpr int64_t kStateWords = 2 + 2 * kMaxTiles;

// The scratch itself. In host code this name is only a handle for
// cudaGetSymbolAddress, never a pointer a kernel could use.
static __device__ __align__(256) unsigned long long g_scan_scratch[kStateWords];

constexpr int kMaxDevices = 64;
struct PerDevice {
  unsigned long long *scratch = nullptr; // device address of g_scan_scratch on that device
  int sm_count = 0;
};
PerDevice g_devices[kMaxDevices];

int fail_cuda(const char *what, cudaError_t e) {
  char msg[256];
  std::snprintf(msg, sizeof msg, "kh_scan_noalloc: %s failed: %s", what, cudaGetErrorString(e));
  return kh_detail_set_error(static_cast<int>(e), msg);
}

} // namespace

extern "C" int64_t kh_scan_noalloc_max_elements(void) { return kMaxElements; }

extern "C" int kh_scan_noalloc(const float *x, float *y, int64_t n, void *stream) {
  if (x == nullptr || y == nullptr) return kh_detail_set_error(2, "kh_scan_noalloc: null buffer");
  if (n <= 0) return kh_detail_set_error(2, "kh_scan_noalloc: n must be positive");
  if (n > kMaxElements) {
    char msg[192];
    std::snprintf(msg, sizeof msg,
                  "kh_scan_noalloc: n = %lld exceeds the fixed scratch of this entry point "
                  "(at most %lld elements); use kh_scan, which allocates its scratch",
                  static_cast<long long>(n), static_cast<long long>(kMaxElements));
    return kh_detail_set_error(2, msg);
  }
  int device = 0;
  if (cudaError_t e = cudaGetDevice(&device); e != cudaSuccess) return fail_cuda("cudaGetDevice", e);
  if (device < 0 || device >= kMaxDevices)
    return kh_detail_set_error(2, "kh_scan_noalloc: device ordinal out of range");
  PerDevice &d = g_devices[device];
  if (d.scratch == nullptr) {
    // once per device, with that device current
    void *p = nullptr;
    if (cudaError_t e = cudaGetSymbolAddress(&p, g_scan_scratch); e != cudaSuccess)
      return fail_cuda("cudaGetSymbolAddress", e);
    int sms = 0;
    if (cudaError_t e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        e != cudaSuccess)
      return fail_cuda("cudaDeviceGetAttribute", e);
    // the kernel's ring of tile buffers is dynamic shared memory beyond the default limit
    if (cudaError_t e = cudaFuncSetAttribute(kh_scan_noalloc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kSlots * kTile * 4);
        e != cudaSuccess)
      return fail_cuda("cudaFuncSetAttribute", e);
    d.sm_count = sms > 0 ? sms : 1;
    d.scratch = static_cast<unsigned long long *>(p);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t tiles = (n + kTile - 1) / kTile;
  const int64_t words = 2 + 2 * tiles;
  // The array keeps what the last call left: clear the part this call reads.
  if (cudaError_t e = cudaMemsetAsync(d.scratch, 0, static_cast<size_t>(words) * 8, s); e != cudaSuccess)
    return fail_cuda("cudaMemsetAsync", e);
  const int64_t want = static_cast<int64_t>(d.sm_count) * 4;
  const unsigned grid = static_cast<unsigned>(tiles < want ? tiles : want);
  kh_scan_noalloc_kernel<<<grid, kThreads, kSlots * kTile * 4, s>>>(
      x, x, 0, n, 1,                      // x as a rank-1 memref descriptor
      y, y, 0, n, 1,                      // y
      d.scratch, d.scratch, 0, words, 1,  // state
      /*epoch=*/1u, /*ticket_base=*/0ull);
  if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return fail_cuda("kernel launch", e);
  return 0;
}
