// kh_scan_noalloc: the inclusive prefix sum for callers that are not allowed to
// allocate device memory.
//
// Who needs this. The ordinary scan entry points keep their look-back scratch
// (four counter words plus one 16-byte descriptor per 12288-element tile) in a
// buffer the context allocates with cuMemAlloc on first use and grows on demand.
// Some hosts cannot do that: code running inside a memory pool or arena that owns
// every byte of the device and forbids side allocations, plugin callbacks that
// must not call an allocator because an allocation may synchronise the device,
// and code whose device memory budget is fixed and audited up front. For them
// the scratch here is a file-scope __device__ array that is part of the
// library's image: every GPU that loads the library carries it (21,888 bytes)
// until the process exits, and nothing is allocated or freed by the call.
//
// Limits and rules
//   * n <= kh_scan_noalloc_max_elements() (16,777,216); larger sizes are
//     refused with a usage error, never truncated.
//   * The first call on a device looks up the array's device address, the SM
//     count and the driver's tensor-map encoder and raises the kernel's
//     shared-memory limit (once per device, with that device current, under a
//     lock, so concurrent first calls are safe). Make that first call outside
//     any stream capture.
//   * All calls on a device share the one array. The part a call uses is
//     cleared on the stream before its kernel, so a call never sees an earlier
//     call's contents; two calls that overlap on the GPU (different streams
//     without ordering) race on it and must be serialised by the caller.
//   * The device that owns x and y must be current; the call enqueues on
//     `stream` and returns without waiting.
//   * A look-back that runs out of its poll budget stops the kernel and leaves y
//     incomplete, as in kh_scan. Nothing reports that by itself here (there is no
//     context to ask): kh_scan_noalloc_status(stream) waits for the stream and
//     returns 1001 when the last call on the current device ended that way.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>

// The kernel is the library's scan kernel, compiled a second time into this
// translation unit under another entry name so that the existing code object
// and its launch path stay exactly as they are.
#define scan kh_scan_noalloc_kernel
#include "scan.cu"
#undef scan

extern "C" int kh_detail_set_error(int code, const char *message); // capi.cpp

namespace {

constexpr int64_t kMaxElements = int64_t(1) << 24;
constexpr int64_t kMaxTiles = (kMaxElements + kTile - 1) / kTile; // 1366
constexpr int64_t kStateWords = 4 + 2 * kMaxTiles;
constexpr size_t kDynamicSmem = static_cast<size_t>(kSlots) * kTile * 4 + 1024;

// The scratch itself. In host code this name is only a handle for
// cudaGetSymbolAddress, never a pointer a kernel could use.
static __device__ __align__(256) unsigned long long g_scan_scratch[kStateWords];

using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

constexpr int kMaxDevices = 64;
struct PerDevice {
  unsigned long long *scratch = nullptr; // device address of g_scan_scratch on that device
  int sm_count = 0;
};
PerDevice g_devices[kMaxDevices];
EncodeTiled g_encode = nullptr;
std::mutex g_setup_lock;

int fail_cuda(const char *what, cudaError_t e) {
  char msg[256];
  std::snprintf(msg, sizeof msg, "kh_scan_noalloc: %s failed: %s", what, cudaGetErrorString(e));
  return kh_detail_set_error(static_cast<int>(e), msg);
}

// x or y seen as [n / 32 rows][32 floats]; false when the buffer cannot be copied by tensor map
// (the kernel then uses plain loads / stores for that side).
bool tensor_map(const float *p, int64_t n, khd::TensorMap *out) {
  std::memset(out, 0, sizeof *out);
  if (g_encode == nullptr || (reinterpret_cast<uintptr_t>(p) & 15u) != 0 || n < kLaneElems) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(kLaneElems), static_cast<cuuint64_t>(n / kLaneElems)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(kLaneElems) * 4};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kLaneElems), 32}, elem_strides[2] = {1, 1};
  static_assert(sizeof(CUtensorMap) == sizeof(khd::TensorMap), "tensor map size");
  return g_encode(reinterpret_cast<CUtensorMap *>(out), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(p),
                  dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Once per device, with that device current. Returns 0 or an error code.
int set_up(int device, PerDevice **out) {
  if (device < 0 || device >= kMaxDevices)
    return kh_detail_set_error(2, "kh_scan_noalloc: device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_setup_lock);
  PerDevice &d = g_devices[device];
  if (d.scratch == nullptr) {
    void *p = nullptr;
    if (cudaError_t e = cudaGetSymbolAddress(&p, g_scan_scratch); e != cudaSuccess)
      return fail_cuda("cudaGetSymbolAddress", e);
    int sms = 0;
    if (cudaError_t e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device); e != cudaSuccess)
      return fail_cuda("cudaDeviceGetAttribute", e);
    // the kernel's ring of tile buffers is dynamic shared memory beyond the default limit
    if (cudaError_t e = cudaFuncSetAttribute(kh_scan_noalloc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(kDynamicSmem));
        e != cudaSuccess)
      return fail_cuda("cudaFuncSetAttribute", e);
    if (g_encode == nullptr) {
      void *fn = nullptr;
      cudaDriverEntryPointQueryResult found;
      if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found) == cudaSuccess &&
          found == cudaDriverEntryPointSuccess)
        g_encode = reinterpret_cast<EncodeTiled>(fn); // without it every call takes the plain-access path
    }
    d.sm_count = sms > 0 ? sms : 1;
    d.scratch = static_cast<unsigned long long *>(p);
  }
  *out = &d;
  return 0;
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
  PerDevice *d = nullptr;
  if (int rc = set_up(device, &d)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t tiles = (n + kTile - 1) / kTile;
  const int64_t words = 4 + 2 * tiles;
  // The array keeps what the last call left: clear the part this call reads.
  if (cudaError_t e = cudaMemsetAsync(d->scratch, 0, static_cast<size_t>(words) * 8, s); e != cudaSuccess)
    return fail_cuda("cudaMemsetAsync", e);
  khd::TensorMap x_map, y_map;
  uint32_t flags = 0;
  if (tensor_map(x, n, &x_map)) flags |= kFlagTmaIn;
  if (tensor_map(y, n, &y_map)) flags |= kFlagTmaOut;
  const unsigned grid = static_cast<unsigned>(tiles < d->sm_count ? tiles : d->sm_count);
  kh_scan_noalloc_kernel<<<grid, (kWarps + 1) * 32, kDynamicSmem, s>>>(
      x, x, 0, n, 1,                        // x as a rank-1 memref descriptor
      y, y, 0, n, 1,                        // y
      d->scratch, d->scratch, 0, words, 1,  // state
      /*spin_limit=*/0u, /*tile_bias=*/0u, x_map, y_map, flags);
  if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return fail_cuda("kernel launch", e);
  return 0;
}

extern "C" int kh_scan_noalloc_status(void *stream) {
  int device = 0;
  if (cudaError_t e = cudaGetDevice(&device); e != cudaSuccess) return fail_cuda("cudaGetDevice", e);
  PerDevice *d = nullptr;
  if (int rc = set_up(device, &d)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint32_t word[2] = {0, 0}; // the status word lives in word 1 of the array: no allocation to read it
  if (cudaError_t e = cudaMemcpyAsync(word, d->scratch + 1, sizeof word, cudaMemcpyDeviceToHost, s); e != cudaSuccess)
    return fail_cuda("cudaMemcpyAsync", e);
  if (cudaError_t e = cudaStreamSynchronize(s); e != cudaSuccess) return fail_cuda("cudaStreamSynchronize", e);
  if (word[0] == 0) return 0;
  char msg[224];
  std::snprintf(msg, sizeof msg,
                "kh_scan_noalloc: a device-side bounded wait ran out (code %u, detail %u); the kernel stopped "
                "and its output is incomplete",
                word[0], word[1]);
  return kh_detail_set_error(1001, msg);
}
