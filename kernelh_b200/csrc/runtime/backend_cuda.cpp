// CUDA Driver API backend, resolved at run time (see backend.hpp). Types come
// from <cuda.h>; the library itself is only ever dlopen'ed.
#include "backend.hpp"

#include "device_limits.hpp"
#include "launch_verifier.hpp"

#include <cuda.h>
#include <dlfcn.h>

#include <cstring>
#include <type_traits>

namespace kh {
namespace {

// name in the table, exported symbol, signature
#define KH_DRIVER_SYMBOLS(X)                                                                       \
  X(Init, "cuInit", CUresult (*)(unsigned))                                                        \
  X(DeviceGetCount, "cuDeviceGetCount", CUresult (*)(int *))                                       \
  X(DeviceGet, "cuDeviceGet", CUresult (*)(CUdevice *, int))                                       \
  X(DeviceGetName, "cuDeviceGetName", CUresult (*)(char *, int, CUdevice))                         \
  X(DeviceGetAttribute, "cuDeviceGetAttribute", CUresult (*)(int *, CUdevice_attribute, CUdevice)) \
  X(DeviceTotalMem, "cuDeviceTotalMem_v2", CUresult (*)(size_t *, CUdevice))                       \
  X(PrimaryCtxRetain, "cuDevicePrimaryCtxRetain", CUresult (*)(CUcontext *, CUdevice))             \
  X(CtxSetCurrent, "cuCtxSetCurrent", CUresult (*)(CUcontext))                                     \
  X(CtxSynchronize, "cuCtxSynchronize", CUresult (*)())                                            \
  X(CtxEnablePeerAccess, "cuCtxEnablePeerAccess", CUresult (*)(CUcontext, unsigned))               \
  X(DeviceCanAccessPeer, "cuDeviceCanAccessPeer", CUresult (*)(int *, CUdevice, CUdevice))         \
  X(MemAlloc, "cuMemAlloc_v2", CUresult (*)(CUdeviceptr *, size_t))                                \
  X(MemFree, "cuMemFree_v2", CUresult (*)(CUdeviceptr))                                            \
  X(MemHostAlloc, "cuMemHostAlloc", CUresult (*)(void **, size_t, unsigned))                       \
  X(MemFreeHost, "cuMemFreeHost", CUresult (*)(void *))                                            \
  X(MemcpyHtoD, "cuMemcpyHtoD_v2", CUresult (*)(CUdeviceptr, const void *, size_t))                \
  X(MemcpyDtoH, "cuMemcpyDtoH_v2", CUresult (*)(void *, CUdeviceptr, size_t))                      \
  X(MemcpyHtoDAsync, "cuMemcpyHtoDAsync_v2",                                                       \
    CUresult (*)(CUdeviceptr, const void *, size_t, CUstream))                                     \
  X(MemcpyDtoHAsync, "cuMemcpyDtoHAsync_v2", CUresult (*)(void *, CUdeviceptr, size_t, CUstream))  \
  X(MemcpyDtoDAsync, "cuMemcpyDtoDAsync_v2",                                                       \
    CUresult (*)(CUdeviceptr, CUdeviceptr, size_t, CUstream))                                      \
  X(MemsetD32Async, "cuMemsetD32Async", CUresult (*)(CUdeviceptr, unsigned, size_t, CUstream))     \
  X(ModuleLoadData, "cuModuleLoadData", CUresult (*)(CUmodule *, const void *))                    \
  X(ModuleGetFunction, "cuModuleGetFunction", CUresult (*)(CUfunction *, CUmodule, const char *))  \
  X(ModuleUnload, "cuModuleUnload", CUresult (*)(CUmodule))                                        \
  X(FuncGetAttribute, "cuFuncGetAttribute", CUresult (*)(int *, CUfunction_attribute, CUfunction)) \
  X(FuncSetAttribute, "cuFuncSetAttribute", CUresult (*)(CUfunction, CUfunction_attribute, int))   \
  X(OccupancyMaxActiveBlocks, "cuOccupancyMaxActiveBlocksPerMultiprocessor",                       \
    CUresult (*)(int *, CUfunction, int, size_t))                                                  \
  X(TensorMapEncodeTiled, "cuTensorMapEncodeTiled",                                                \
    CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,       \
                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,                       \
                 CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,                \
                 CUtensorMapFloatOOBfill))                                                         \
  X(LaunchKernel, "cuLaunchKernel",                                                                \
    CUresult (*)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,           \
                 unsigned, CUstream, void **, void **))                                            \
  X(LaunchKernelEx, "cuLaunchKernelEx",                                                            \
    CUresult (*)(const CUlaunchConfig *, CUfunction, void **, void **))                            \
  X(StreamCreate, "cuStreamCreate", CUresult (*)(CUstream *, unsigned))                            \
  X(StreamDestroy, "cuStreamDestroy_v2", CUresult (*)(CUstream))                                   \
  X(StreamSynchronize, "cuStreamSynchronize", CUresult (*)(CUstream))                              \
  X(StreamWaitEvent, "cuStreamWaitEvent", CUresult (*)(CUstream, CUevent, unsigned))               \
  X(EventCreate, "cuEventCreate", CUresult (*)(CUevent *, unsigned))                               \
  X(EventRecord, "cuEventRecord", CUresult (*)(CUevent, CUstream))                                 \
  X(EventSynchronize, "cuEventSynchronize", CUresult (*)(CUevent))                                 \
  X(EventQuery, "cuEventQuery", CUresult (*)(CUevent))                                             \
  X(EventElapsedTime, "cuEventElapsedTime", CUresult (*)(float *, CUevent, CUevent))               \
  X(EventDestroy, "cuEventDestroy_v2", CUresult (*)(CUevent))                                      \
  X(GetErrorString, "cuGetErrorString", CUresult (*)(CUresult, const char **))                     \
  X(GetErrorName, "cuGetErrorName", CUresult (*)(CUresult, const char **))

struct DriverApi {
  void *handle = nullptr;
#define KH_FIELD(name, sym, sig) std::type_identity_t<sig> name = nullptr;
  KH_DRIVER_SYMBOLS(KH_FIELD)
#undef KH_FIELD
};

class CudaBackend final : public Backend {
public:
  explicit CudaBackend(DriverApi api) : api_(api) {}

  const char *kind() const override { return "cuda"; }

  Result<int> device_count() override {
    if (auto r = ensure_init(); !r) return std::unexpected(r.error());
    int n = 0;
    if (CUresult r = api_.DeviceGetCount(&n); r != CUDA_SUCCESS) return err(r, "cuDeviceGetCount");
    return n;
  }

  Result<void> init_device(int ordinal) override {
    if (auto r = ensure_init(); !r) return r;
    if (CUresult r = api_.DeviceGet(&dev_, ordinal); r != CUDA_SUCCESS) return err(r, "cuDeviceGet");
    if (CUresult r = api_.PrimaryCtxRetain(&ctx_, dev_); r != CUDA_SUCCESS)
      return err(r, "cuDevicePrimaryCtxRetain");
    if (CUresult r = api_.CtxSetCurrent(ctx_); r != CUDA_SUCCESS) return err(r, "cuCtxSetCurrent");
    ordinal_ = ordinal;
    int sms = 0;
    if (api_.DeviceGetAttribute(&sms, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT, dev_) == CUDA_SUCCESS)
      set_runtime_cu_count(sms);
    // The launch verifier and the occupancy report ask the driver through this.
    auto *api = &api_;
    set_occupancy_query([api](void *fn, int block, size_t dyn) {
      int blocks = -1;
      if (fn == nullptr) return -1;
      if (api->OccupancyMaxActiveBlocks(&blocks, static_cast<CUfunction>(fn), block, dyn) !=
          CUDA_SUCCESS)
        return -1;
      return blocks;
    });
    return {};
  }

  Result<void> make_current() override {
    if (ctx_ == nullptr) return fail(1, "CudaBackend: no device initialised");
    if (CUresult r = api_.CtxSetCurrent(ctx_); r != CUDA_SUCCESS) return err(r, "cuCtxSetCurrent");
    return {};
  }

  void *native_context() override { return ctx_; }

  // Maps the memory of `peer`'s device into this device's address space (unified addressing:
  // the peer's pointers are then valid in kernels launched here). Already enabled counts as done.
  Result<void> enable_peer_access(Backend &peer) override {
    if (ctx_ == nullptr || peer.native_context() == nullptr)
      return fail(1, "CudaBackend::enable_peer_access: a device is not initialised");
    if (&peer == this) return {};
    auto peer_info = peer.device_info();
    if (!peer_info) return std::unexpected(peer_info.error());
    CUdevice other;
    if (CUresult r = api_.DeviceGet(&other, peer_info->ordinal); r != CUDA_SUCCESS) return err(r, "cuDeviceGet");
    int can = 0;
    if (CUresult r = api_.DeviceCanAccessPeer(&can, dev_, other); r != CUDA_SUCCESS)
      return err(r, "cuDeviceCanAccessPeer");
    if (!can)
      return fail(1, "device " + std::to_string(ordinal_) + " cannot map the memory of device " +
                         std::to_string(peer_info->ordinal) + " (no peer access between them)");
    if (CUresult r = api_.CtxSetCurrent(ctx_); r != CUDA_SUCCESS) return err(r, "cuCtxSetCurrent");
    const CUresult r = api_.CtxEnablePeerAccess(static_cast<CUcontext>(peer.native_context()), 0);
    if (r != CUDA_SUCCESS && r != CUDA_ERROR_PEER_ACCESS_ALREADY_ENABLED) return err(r, "cuCtxEnablePeerAccess");
    return {};
  }

  Result<DeviceInfo> device_info() override {
    if (ctx_ == nullptr) return fail(1, "CudaBackend::device_info: no device initialised");
    DeviceInfo info;
    info.ordinal = ordinal_;
    char name[256] = {0};
    if (CUresult r = api_.DeviceGetName(name, sizeof name, dev_); r != CUDA_SUCCESS)
      return err(r, "cuDeviceGetName");
    info.name = name;
    size_t total = 0;
    if (CUresult r = api_.DeviceTotalMem(&total, dev_); r != CUDA_SUCCESS)
      return err(r, "cuDeviceTotalMem");
    info.vram_bytes = static_cast<long>(total);
    auto attr = [&](CUdevice_attribute a) -> Result<int> {
      int v = 0;
      if (CUresult r = api_.DeviceGetAttribute(&v, a, dev_); r != CUDA_SUCCESS)
        return err(r, "cuDeviceGetAttribute");
      return v;
    };
#define KH_ATTR(dst, id)                                                                           \
  if (auto v = attr(id); v)                                                                        \
    dst = *v;                                                                                      \
  else                                                                                             \
    return std::unexpected(v.error());
    KH_ATTR(info.lds_bytes_per_workgroup, CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_BLOCK)
    KH_ATTR(info.wavefront_size, CU_DEVICE_ATTRIBUTE_WARP_SIZE)
    KH_ATTR(info.max_threads_per_workgroup, CU_DEVICE_ATTRIBUTE_MAX_THREADS_PER_BLOCK)
    KH_ATTR(info.cu_count, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT)
    KH_ATTR(info.smem_optin_per_block, CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_BLOCK_OPTIN)
    KH_ATTR(info.smem_per_sm, CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_MULTIPROCESSOR)
    KH_ATTR(info.regs_per_sm, CU_DEVICE_ATTRIBUTE_MAX_REGISTERS_PER_MULTIPROCESSOR)
    KH_ATTR(info.max_blocks_per_sm, CU_DEVICE_ATTRIBUTE_MAX_BLOCKS_PER_MULTIPROCESSOR)
    KH_ATTR(info.max_threads_per_sm, CU_DEVICE_ATTRIBUTE_MAX_THREADS_PER_MULTIPROCESSOR)
    KH_ATTR(info.l2_bytes, CU_DEVICE_ATTRIBUTE_L2_CACHE_SIZE)
    KH_ATTR(info.cc_major, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR)
    KH_ATTR(info.cc_minor, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR)
#undef KH_ATTR
    return info;
  }

  Result<void> device_synchronize() override {
    if (CUresult r = api_.CtxSynchronize(); r != CUDA_SUCCESS) return err(r, "cuCtxSynchronize");
    return {};
  }

  Result<void *> malloc(size_t bytes) override {
    CUdeviceptr p = 0;
    if (CUresult r = api_.MemAlloc(&p, bytes); r != CUDA_SUCCESS) return err(r, "cuMemAlloc");
    return reinterpret_cast<void *>(p);
  }
  Result<void> free(void *ptr) override {
    if (CUresult r = api_.MemFree(reinterpret_cast<CUdeviceptr>(ptr)); r != CUDA_SUCCESS)
      return err(r, "cuMemFree");
    return {};
  }
  Result<void *> malloc_host(size_t bytes) override {
    void *p = nullptr;
    if (CUresult r = api_.MemHostAlloc(&p, bytes, 0); r != CUDA_SUCCESS) return err(r, "cuMemHostAlloc");
    return p;
  }
  Result<void> free_host(void *ptr) override {
    if (CUresult r = api_.MemFreeHost(ptr); r != CUDA_SUCCESS) return err(r, "cuMemFreeHost");
    return {};
  }
  Result<void> memcpy_h2d(void *dst, const void *src, size_t bytes) override {
    if (CUresult r = api_.MemcpyHtoD(reinterpret_cast<CUdeviceptr>(dst), src, bytes); r != CUDA_SUCCESS)
      return err(r, "cuMemcpyHtoD");
    return {};
  }
  Result<void> memcpy_d2h(void *dst, const void *src, size_t bytes) override {
    if (CUresult r = api_.MemcpyDtoH(dst, reinterpret_cast<CUdeviceptr>(src), bytes); r != CUDA_SUCCESS)
      return err(r, "cuMemcpyDtoH");
    return {};
  }
  Result<void> memcpy_h2d_async(void *dst, const void *src, size_t bytes, StreamHandle s) override {
    if (CUresult r = api_.MemcpyHtoDAsync(reinterpret_cast<CUdeviceptr>(dst), src, bytes,
                                          static_cast<CUstream>(s));
        r != CUDA_SUCCESS)
      return err(r, "cuMemcpyHtoDAsync");
    return {};
  }
  Result<void> memcpy_d2h_async(void *dst, const void *src, size_t bytes, StreamHandle s) override {
    if (CUresult r = api_.MemcpyDtoHAsync(dst, reinterpret_cast<CUdeviceptr>(src), bytes,
                                          static_cast<CUstream>(s));
        r != CUDA_SUCCESS)
      return err(r, "cuMemcpyDtoHAsync");
    return {};
  }
  Result<void> memcpy_d2d_async(void *dst, const void *src, size_t bytes, StreamHandle s) override {
    if (CUresult r = api_.MemcpyDtoDAsync(reinterpret_cast<CUdeviceptr>(dst),
                                          reinterpret_cast<CUdeviceptr>(src), bytes,
                                          static_cast<CUstream>(s));
        r != CUDA_SUCCESS)
      return err(r, "cuMemcpyDtoDAsync");
    return {};
  }
  Result<void> memset32_async(void *dst, uint32_t value, size_t words, StreamHandle s) override {
    if (CUresult r = api_.MemsetD32Async(reinterpret_cast<CUdeviceptr>(dst), value, words,
                                         static_cast<CUstream>(s));
        r != CUDA_SUCCESS)
      return err(r, "cuMemsetD32Async");
    return {};
  }

  Result<void *> module_load_data(const void *image) override {
    if (image == nullptr) return fail(1, "module_load_data: null image");
    CUmodule m = nullptr;
    if (CUresult r = api_.ModuleLoadData(&m, image); r != CUDA_SUCCESS) return err(r, "cuModuleLoadData");
    return static_cast<void *>(m);
  }
  Result<void *> module_get_function(void *module, const char *name) override {
    CUfunction f = nullptr;
    if (CUresult r = api_.ModuleGetFunction(&f, static_cast<CUmodule>(module), name); r != CUDA_SUCCESS)
      return err(r, (std::string("cuModuleGetFunction(") + name + ")").c_str());
    return static_cast<void *>(f);
  }
  Result<void> module_unload(void *module) override {
    if (CUresult r = api_.ModuleUnload(static_cast<CUmodule>(module)); r != CUDA_SUCCESS)
      return err(r, "cuModuleUnload");
    return {};
  }
  Result<FunctionAttributes> function_attributes(void *function) override {
    FunctionAttributes a;
    auto f = static_cast<CUfunction>(function);
    if (CUresult r = api_.FuncGetAttribute(&a.num_regs, CU_FUNC_ATTRIBUTE_NUM_REGS, f); r != CUDA_SUCCESS)
      return err(r, "cuFuncGetAttribute(NUM_REGS)");
    api_.FuncGetAttribute(&a.static_smem_bytes, CU_FUNC_ATTRIBUTE_SHARED_SIZE_BYTES, f);
    api_.FuncGetAttribute(&a.max_dynamic_smem_bytes, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, f);
    api_.FuncGetAttribute(&a.max_threads_per_block, CU_FUNC_ATTRIBUTE_MAX_THREADS_PER_BLOCK, f);
    return a;
  }
  Result<void> function_set_max_dynamic_smem(void *function, size_t bytes) override {
    if (CUresult r = api_.FuncSetAttribute(static_cast<CUfunction>(function),
                                           CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                                           static_cast<int>(bytes));
        r != CUDA_SUCCESS)
      return err(r, "cuFuncSetAttribute(MAX_DYNAMIC_SHARED_SIZE_BYTES)");
    return {};
  }
  Result<void> function_allow_large_clusters(void *function) override {
    if (CUresult r = api_.FuncSetAttribute(static_cast<CUfunction>(function),
                                           CU_FUNC_ATTRIBUTE_NON_PORTABLE_CLUSTER_SIZE_ALLOWED, 1);
        r != CUDA_SUCCESS)
      return err(r, "cuFuncSetAttribute(NON_PORTABLE_CLUSTER_SIZE_ALLOWED)");
    return {};
  }
  Result<int> occupancy_max_blocks(void *function, int block_size, size_t dyn_smem) override {
    int blocks = 0;
    if (CUresult r = api_.OccupancyMaxActiveBlocks(&blocks, static_cast<CUfunction>(function),
                                                   block_size, dyn_smem);
        r != CUDA_SUCCESS)
      return err(r, "cuOccupancyMaxActiveBlocksPerMultiprocessor");
    return blocks;
  }

  Result<TensorMapBytes> encode_tensor_map(const TensorMapSpec &s) override {
    if (s.rank < 1 || s.rank > 5) return fail(1, "encode_tensor_map: rank must be 1..5");
    if (s.elem_bytes != 4 && s.elem_bytes != 2)
      return fail(1, "encode_tensor_map: elements must be fp32 (4 bytes) or fp16 (2 bytes)");
    const CUtensorMapDataType dtype =
        s.elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_NONE;
    switch (s.swizzle_bytes) {
    case 0: break;
    case 32: sw = CU_TENSOR_MAP_SWIZZLE_32B; break;
    case 64: sw = CU_TENSOR_MAP_SWIZZLE_64B; break;
    case 128: sw = CU_TENSOR_MAP_SWIZZLE_128B; break;
    default: return fail(1, "encode_tensor_map: swizzle must be 0, 32, 64 or 128 bytes");
    }
    cuuint64_t dims[5], strides[4];
    cuuint32_t box[5], estr[5];
    for (int i = 0; i < s.rank; ++i) {
      dims[i] = s.dims[i];
      box[i] = s.box[i];
      estr[i] = 1;
    }
    for (int i = 0; i + 1 < s.rank; ++i) strides[i] = s.strides_bytes[i];
    CUtensorMap map;
    std::memset(&map, 0, sizeof map);
    if (CUresult r = api_.TensorMapEncodeTiled(
            &map, dtype, static_cast<cuuint32_t>(s.rank),
            const_cast<void *>(s.global_address), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        r != CUDA_SUCCESS)
      return err(r, "cuTensorMapEncodeTiled");
    TensorMapBytes out;
    static_assert(sizeof(CUtensorMap) == sizeof(TensorMapBytes));
    std::memcpy(&out, &map, sizeof out);
    return out;
  }

  Result<void> launch_kernel(void *function, const LaunchDims &grid, const LaunchDims &block,
                             size_t shared_bytes, StreamHandle stream, void *const *params,
                             unsigned cluster_x, bool overlap_tail) override {
    CUresult r;
    if (cluster_x <= 1 && !overlap_tail) {
      r = api_.LaunchKernel(static_cast<CUfunction>(function), grid.x, grid.y, grid.z, block.x,
                            block.y, block.z, static_cast<unsigned>(shared_bytes),
                            static_cast<CUstream>(stream), const_cast<void **>(params), nullptr);
    } else {
      CUlaunchConfig cfg;
      std::memset(&cfg, 0, sizeof cfg);
      cfg.gridDimX = grid.x;
      cfg.gridDimY = grid.y;
      cfg.gridDimZ = grid.z;
      cfg.blockDimX = block.x;
      cfg.blockDimY = block.y;
      cfg.blockDimZ = block.z;
      cfg.sharedMemBytes = static_cast<unsigned>(shared_bytes);
      cfg.hStream = static_cast<CUstream>(stream);
      CUlaunchAttribute attrs[2];
      std::memset(attrs, 0, sizeof attrs);
      unsigned count = 0;
      if (cluster_x > 1) {
        attrs[count].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
        attrs[count].value.clusterDim.x = cluster_x;
        attrs[count].value.clusterDim.y = 1;
        attrs[count].value.clusterDim.z = 1;
        ++count;
      }
      if (overlap_tail) {
        attrs[count].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
        attrs[count].value.programmaticStreamSerializationAllowed = 1;
        ++count;
      }
      cfg.attrs = attrs;
      cfg.numAttrs = count;
      r = api_.LaunchKernelEx(&cfg, static_cast<CUfunction>(function), const_cast<void **>(params),
                              nullptr);
    }
    if (r != CUDA_SUCCESS) return err(r, "cuLaunchKernel");
    return {};
  }

  Result<StreamHandle> stream_create() override {
    CUstream s = nullptr;
    if (CUresult r = api_.StreamCreate(&s, CU_STREAM_NON_BLOCKING); r != CUDA_SUCCESS)
      return err(r, "cuStreamCreate");
    return static_cast<StreamHandle>(s);
  }
  Result<void> stream_destroy(StreamHandle s) override {
    if (CUresult r = api_.StreamDestroy(static_cast<CUstream>(s)); r != CUDA_SUCCESS)
      return err(r, "cuStreamDestroy");
    return {};
  }
  Result<void> stream_synchronize(StreamHandle s) override {
    if (CUresult r = api_.StreamSynchronize(static_cast<CUstream>(s)); r != CUDA_SUCCESS)
      return err(r, "cuStreamSynchronize");
    return {};
  }

  Result<EventHandle> event_create() override {
    CUevent e = nullptr;
    if (CUresult r = api_.EventCreate(&e, CU_EVENT_DEFAULT); r != CUDA_SUCCESS) return err(r, "cuEventCreate");
    return static_cast<EventHandle>(e);
  }
  Result<void> event_record(EventHandle e, StreamHandle s) override {
    if (CUresult r = api_.EventRecord(static_cast<CUevent>(e), static_cast<CUstream>(s)); r != CUDA_SUCCESS)
      return err(r, "cuEventRecord");
    return {};
  }
  Result<void> event_synchronize(EventHandle e) override {
    if (CUresult r = api_.EventSynchronize(static_cast<CUevent>(e)); r != CUDA_SUCCESS)
      return err(r, "cuEventSynchronize");
    return {};
  }
  Result<bool> event_query(EventHandle e) override {
    const CUresult r = api_.EventQuery(static_cast<CUevent>(e));
    if (r == CUDA_SUCCESS) return true;
    if (r == CUDA_ERROR_NOT_READY) return false;
    return err(r, "cuEventQuery");
  }
  Result<float> event_elapsed_time(EventHandle start, EventHandle end) override {
    float ms = 0.f;
    if (CUresult r = api_.EventElapsedTime(&ms, static_cast<CUevent>(start), static_cast<CUevent>(end));
        r != CUDA_SUCCESS)
      return err(r, "cuEventElapsedTime");
    return ms;
  }
  Result<void> stream_wait_event(StreamHandle s, EventHandle e) override {
    if (CUresult r = api_.StreamWaitEvent(static_cast<CUstream>(s), static_cast<CUevent>(e), 0);
        r != CUDA_SUCCESS)
      return err(r, "cuStreamWaitEvent");
    return {};
  }
  Result<void> event_destroy(EventHandle e) override {
    if (CUresult r = api_.EventDestroy(static_cast<CUevent>(e)); r != CUDA_SUCCESS)
      return err(r, "cuEventDestroy");
    return {};
  }

private:
  Result<void> ensure_init() {
    if (inited_) return {};
    if (CUresult r = api_.Init(0); r != CUDA_SUCCESS) {
      // No usable device/driver behind the library: same skip code as a missing library.
      return fail(kDriverUnavailable, "cuInit failed: " + error_string(r) + " (" +
                                          std::to_string(static_cast<int>(r)) + ")");
    }
    inited_ = true;
    return {};
  }

  std::string error_string(CUresult code) const {
    const char *s = nullptr;
    if (api_.GetErrorString && api_.GetErrorString(code, &s) == CUDA_SUCCESS && s) return s;
    return "CUDA error " + std::to_string(static_cast<int>(code));
  }
  std::unexpected<Error> err(CUresult code, const char *what) const {
    return fail(static_cast<int>(code), std::string(what) + " failed: " + error_string(code) + " (" +
                                            std::to_string(static_cast<int>(code)) + ")");
  }

  DriverApi api_;
  bool inited_ = false;
  CUdevice dev_ = 0;
  CUcontext ctx_ = nullptr;
  int ordinal_ = 0;
};

} // namespace

Result<std::shared_ptr<Backend>> make_cuda_backend(const std::string &library_path) {
  const char *path = library_path.empty() ? "libcuda.so.1" : library_path.c_str();
  void *h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (h == nullptr) {
    const char *why = dlerror();
    return fail(kDriverUnavailable, std::string("CUDA driver unavailable: dlopen(\"") + path +
                                        "\") failed: " + (why ? why : "unknown error"));
  }
  DriverApi api;
  api.handle = h;
#define KH_LOAD(name, sym, sig)                                                                    \
  api.name = reinterpret_cast<sig>(dlsym(h, sym));                                                 \
  if (api.name == nullptr)                                                                         \
    return fail(kDriverUnavailable, std::string("CUDA driver unavailable: symbol ") + sym +        \
                                        " not found in " + path);
  KH_DRIVER_SYMBOLS(KH_LOAD)
#undef KH_LOAD
  return std::shared_ptr<Backend>(std::make_shared<CudaBackend>(api));
}

} // namespace kh
