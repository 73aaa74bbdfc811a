"""kernelh_b200: kernel.h's seven launched kernel templates, hand-written for
NVIDIA B200 (sm_100a), behind kernel.h's kernel-name + shape operator surface.

This module is a thin ctypes binding of the C ABI in ``include/kernelh_b200.h``
(``libkernelh_b200.so``, built in-tree by ``kernelh_b200/csrc/build.py``). It mirrors
the reference's host interface: a device context, ``launch(kernel, shape,
buffers)`` with the CLI's ``k=v,k=v`` shape text, the launch verifier, the
device-limits table, the occupancy model, bench metrics and the results CSV
line. There is no CPU implementation behind any compute call: without the
native library this import fails, and without a B200 the compute calls raise.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libkernelh_b200.so")

DRIVER_UNAVAILABLE = 77
USAGE_ERROR = 2
DEVICE_TIMEOUT = 1001

KERNELS = ("attention", "fused_gelu", "gemm", "layernorm", "scan", "softmax", "vecadd")
# the reference also registers the second kernel of its two-launch scan; here it launches nothing
REGISTERED = tuple(sorted(KERNELS + ("scan_totals",)))


class KernelhError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code
        self.message = message


class DeviceInfo(C.Structure):
    _fields_ = [("name", C.c_char * 256), ("vram_bytes", C.c_int64),
                ("static_smem_per_block", C.c_int64), ("optin_smem_per_block", C.c_int64),
                ("smem_per_sm", C.c_int64), ("l2_bytes", C.c_int64), ("sm_count", C.c_int32),
                ("warp_size", C.c_int32), ("max_threads_per_block", C.c_int32),
                ("regs_per_sm", C.c_int32), ("max_blocks_per_sm", C.c_int32),
                ("cc_major", C.c_int32), ("cc_minor", C.c_int32), ("ordinal", C.c_int32)]


class CustomPlan(C.Structure):
    _fields_ = [("grid", C.c_uint32 * 3), ("block", C.c_uint32 * 3), ("dynamic_smem", C.c_size_t),
                ("n_buffers", C.c_int32), ("elements", C.c_int64 * 8), ("is_output", C.c_uint8 * 8),
                ("work", C.c_double), ("work_is_flops", C.c_int32)]


PLAN_FN = C.CFUNCTYPE(C.c_int, C.c_char_p, C.c_int, C.POINTER(CustomPlan), C.POINTER(C.c_char), C.c_int, C.c_void_p)


class PlanInfo(C.Structure):
    _fields_ = [("n_buffers", C.c_int32), ("n_launches", C.c_int32),
                ("workspace_bytes", C.c_int64), ("entry", C.c_char * 64),
                ("grid", C.c_uint32 * 3), ("block", C.c_uint32 * 3), ("dynamic_smem", C.c_int64),
                ("param_count", C.c_int32), ("tmem_columns", C.c_int32), ("work", C.c_double),
                ("work_is_flops", C.c_int32)]


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python kernelh_b200/csrc/build.py` "
            "(needs nvcc and g++); there is no fallback implementation")
    L = C.CDLL(LIB_PATH)
    vp, i64, f32p = C.c_void_p, C.c_int64, C.c_void_p
    L.kh_last_error.restype = C.c_char_p
    L.kh_version.restype = C.c_char_p
    L.kh_context_create.argtypes = [C.c_int, C.POINTER(vp)]
    L.kh_context_destroy.argtypes = [vp]
    L.kh_context_destroy.restype = None
    L.kh_device_count.argtypes = [C.POINTER(C.c_int)]
    L.kh_device_info_get.argtypes = [vp, C.POINTER(DeviceInfo)]
    L.kh_launch.argtypes = [vp, C.c_char_p, C.c_char_p, C.POINTER(vp), C.c_int, vp]
    L.kh_run_host.argtypes = [vp, C.c_char_p, C.c_char_p, C.POINTER(vp), C.c_int]
    L.kh_synchronize.argtypes = [vp, vp]
    L.kh_module_launch.argtypes = [vp, C.c_char_p, C.c_size_t, C.c_char_p, C.POINTER(C.c_uint32),
                                   C.POINTER(C.c_uint32), C.c_size_t, C.POINTER(C.c_uint64),
                                   C.POINTER(C.c_int64), C.POINTER(C.c_int), C.c_int, vp]
    L.kh_profile_enable.argtypes = [vp, C.c_int]
    L.kh_profile_report.argtypes = [vp, C.c_char_p, C.c_int]
    L.kh_launch_count.argtypes = [vp, C.POINTER(C.c_uint64)]
    L.kh_vecadd.argtypes = [vp, f32p, f32p, f32p, i64, vp]
    L.kh_fused_gelu.argtypes = [vp, f32p, f32p, i64, vp]
    L.kh_fused_gelu_bias.argtypes = [vp, f32p, f32p, f32p, i64, vp]
    L.kh_scan.argtypes = [vp, f32p, f32p, i64, vp]
    L.kh_scan_noalloc.argtypes = [f32p, f32p, i64, vp]
    L.kh_scan_noalloc_max_elements.restype = C.c_int64
    L.kh_scan_noalloc_status.argtypes = [vp]
    L.kh_scan_lookback_probe.argtypes = [vp, f32p, f32p, i64, C.c_uint32, vp]
    L.kh_wait_name.argtypes = [C.c_uint32, C.c_char_p, C.c_int]
    L.kh_softmax.argtypes = [vp, f32p, f32p, i64, i64, vp]
    L.kh_layernorm.argtypes = [vp, f32p, f32p, f32p, f32p, i64, i64, vp]
    L.kh_gemm.argtypes = [vp, f32p, f32p, f32p, i64, i64, i64, vp]
    L.kh_gemm_allgather.argtypes = [vp, f32p, f32p, C.POINTER(vp), C.c_int, C.c_int, i64, i64, i64, vp]
    L.kh_gemm_allgather_multicast.argtypes = [vp, f32p, f32p, f32p, vp, C.c_int, C.c_int, i64, i64, i64, vp]
    L.kh_gemm_host_sharded_begin.argtypes = [vp, f32p, f32p, C.POINTER(vp), vp, C.c_int, C.c_int, i64, i64, i64]
    L.kh_gemm_host_sharded_finish.argtypes = [vp, f32p]
    L.kh_attention.argtypes = [vp, f32p, f32p, f32p, f32p, i64, i64, i64, i64, vp]
    L.kh_attention_allgather.argtypes = [vp, f32p, f32p, f32p, C.POINTER(vp), vp, C.c_int, C.c_int, i64, i64, i64, vp]
    L.kh_malloc.argtypes = [vp, C.c_size_t, C.POINTER(vp)]
    L.kh_free.argtypes = [vp, vp]
    L.kh_memcpy_h2d.argtypes = [vp, vp, vp, C.c_size_t]
    L.kh_memcpy_d2h.argtypes = [vp, vp, vp, C.c_size_t]
    L.kh_bench_row.argtypes = [vp, C.c_char_p, C.c_char_p, C.c_int, C.c_int,
                               C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_int)]
    L.kh_enable_peer_access.argtypes = [vp, vp]
    L.kh_gemm_scaled.argtypes = [vp, f32p, f32p, f32p, i64, i64, i64, C.c_float, C.c_float, vp]
    L.kh_arm_arrival_flags.argtypes = [vp, C.POINTER(vp), C.c_int, C.c_uint64]
    L.kh_arm_arrival_flags_overlapped.argtypes = [vp, C.POINTER(vp), C.c_int, C.c_uint64]
    L.kh_join_arrivals.argtypes = [vp, vp]
    L.kh_gemm_clock.argtypes = [vp, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
    L.kh_bench_sharded.argtypes = [C.c_int, C.c_char_p, C.c_char_p, C.c_int, C.c_int,
                                   C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_int)]
    L.kh_registered_kernels.argtypes = [C.c_char_p, C.c_int]
    L.kh_register_kernel.argtypes = [C.c_char_p, C.c_char_p, C.c_size_t, C.c_char_p, PLAN_FN, C.c_void_p]
    L.kh_unregister_kernel.argtypes = [C.c_char_p]
    L.kh_plan.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p, C.c_int, C.POINTER(PlanInfo)]
    L.kh_kernel_image.argtypes = [C.c_char_p, C.POINTER(vp), C.POINTER(C.c_size_t)]
    L.kh_kernel_resources.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, C.c_int, C.POINTER(C.c_int64)]
    L.kh_parse_ptxas.argtypes = [C.c_char_p, C.c_char_p, C.POINTER(C.c_int64)]
    L.kh_occupancy_report.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p, C.c_int, C.c_char_p, C.c_int,
                                      C.c_char_p, C.c_int]
    L.kh_pack_memrefs.argtypes = [C.POINTER(C.c_uint64), C.POINTER(C.c_int64), C.POINTER(C.c_int),
                                  C.c_int, C.POINTER(C.c_uint64), C.c_int, C.POINTER(C.c_int)]
    L.kh_device_limits.argtypes = [C.c_char_p, C.POINTER(C.c_int64), C.c_char_p, C.c_int]
    L.kh_target_token.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
    L.kh_verify_launch.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint64,
                                   C.c_uint64, C.c_int, C.c_char_p, C.c_int]
    L.kh_occupancy.argtypes = [C.c_char_p, C.c_int, C.c_int64, C.c_int, C.c_int64, C.c_int,
                               C.POINTER(C.c_int), C.POINTER(C.c_double), C.POINTER(C.c_int)]
    L.kh_metric.argtypes = [C.c_char_p, i64, i64, i64, i64]
    L.kh_metric.restype = C.c_double
    L.kh_rate.argtypes = [C.c_int, C.c_double, C.c_double]
    L.kh_rate.restype = C.c_double
    L.kh_csv_header.argtypes = [C.c_char_p, C.c_int]
    L.kh_csv_line.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p, C.c_double, C.c_double,
                              C.c_char_p, C.c_char_p, C.c_char_p, C.c_int]
    L.kh_csv_header_ext.argtypes = [C.c_char_p, C.c_int]
    L.kh_csv_line_ext.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p, C.c_double, C.c_double, C.c_char_p, C.c_char_p,
                                  C.c_int, C.c_double, C.c_double, C.c_double, C.c_int, C.c_char_p, C.c_int]
    L.kh_shape_roundtrip.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
    return L


lib = _load()


def _check(rc: int) -> None:
    if rc != 0:
        raise KernelhError(rc, (lib.kh_last_error() or b"").decode(errors="replace"))


def _ptr(x) -> int | None:
    """Device or host address of a torch tensor / numpy array / int / None."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if hasattr(x, "ctypes"):
        return x.ctypes.data
    raise TypeError(f"cannot take the address of {type(x)!r}")


def shape_text(**shape: int) -> str:
    return ",".join(f"{k}={int(v)}" for k, v in shape.items())


class Context:
    """A device context: the reference's ``make_cuda_backend()`` +
    ``DeviceContext::create(backend, ordinal)``, plus the launch machinery."""

    def __init__(self, device_ordinal: int = 0):
        h = C.c_void_p()
        _check(lib.kh_context_create(device_ordinal, C.byref(h)))
        self._h = h

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib.kh_context_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def device_info(self) -> DeviceInfo:
        info = DeviceInfo()
        _check(lib.kh_device_info_get(self._h, C.byref(info)))
        return info

    # ---- operator surface ----------------------------------------------------
    def launch(self, kernel: str, shape: str, buffers, stream: int | None = None) -> None:
        """Enqueue `kernel` for the CLI-style `shape` text on DEVICE buffers."""
        arr = (C.c_void_p * len(buffers))(*[_ptr(b) for b in buffers])
        _check(lib.kh_launch(self._h, kernel.encode(), shape.encode(), arr, len(buffers), stream))

    def run_host(self, kernel: str, shape: str, buffers) -> None:
        """Same on HOST buffers: copy in, launch, copy out, wait."""
        arr = (C.c_void_p * len(buffers))(*[_ptr(b) for b in buffers])
        _check(lib.kh_run_host(self._h, kernel.encode(), shape.encode(), arr, len(buffers)))

    def synchronize(self, stream: int | None = None) -> None:
        _check(lib.kh_synchronize(self._h, stream))

    def module_launch(self, image: bytes, entry: str, grid, block, buffers, shapes,
                      dynamic_smem: int = 0, stream: int | None = None) -> None:
        """The reference runtime's sequence with caller-chosen geometry: load the
        code object, look up `entry`, pack `buffers` as memref descriptors of
        `shapes`, verify the launch against the device limits, launch, wait."""
        flat = [d for s_ in shapes for d in s_]
        _check(lib.kh_module_launch(
            self._h, image, len(image), entry.encode(), (C.c_uint32 * 3)(*grid), (C.c_uint32 * 3)(*block),
            dynamic_smem, (C.c_uint64 * len(buffers))(*[_ptr(b) for b in buffers]),
            (C.c_int64 * max(len(flat), 1))(*flat), (C.c_int * len(shapes))(*[len(s_) for s_ in shapes]),
            len(buffers), stream))

    def profile(self, on: bool) -> None:
        _check(lib.kh_profile_enable(self._h, int(on)))

    def profile_report(self) -> dict:
        """{entry: (launches, total_ms)} of the launches made while profiling."""
        buf = C.create_string_buffer(4096)
        _check(lib.kh_profile_report(self._h, buf, 4096))
        out = {}
        for item in filter(None, buf.value.decode().split(";")):
            name, count, ms = item.split(":")
            out[name] = (int(count), float(ms))
        return out

    def launch_count(self) -> int:
        n = C.c_uint64()
        _check(lib.kh_launch_count(self._h, C.byref(n)))
        return n.value

    def bench_row(self, kernel: str, shape: str, warmup: int = 5, iters: int = 20):
        ms, rate, is_gflops = C.c_double(), C.c_double(), C.c_int()
        _check(lib.kh_bench_row(self._h, kernel.encode(), shape.encode(), warmup, iters,
                                C.byref(ms), C.byref(rate), C.byref(is_gflops)))
        return ms.value, rate.value, bool(is_gflops.value)

    def gemm_scaled(self, a, b, c, m, n, k, alpha, beta, stream=None):
        """C = alpha * A.B + beta * C (beta = 0 never reads C)."""
        _check(lib.kh_gemm_scaled(self._h, _ptr(a), _ptr(b), _ptr(c), m, n, k, alpha, beta, stream))

    def arm_arrival_flags(self, flag_arrays, epoch: int, overlapped: bool = False):
        """The next gemm_allgather / gemm_allgather_multicast call of this context ends with the
        barrier itself: `flag_arrays` are every rank's eight-word int64 arrays (addresses as mapped
        here, e.g. a symmetric-memory buffer's `buffer_ptrs`), `epoch` a positive, growing number.
        `overlapped`: the kernel only signals; the wait runs on a second stream beside what is enqueued
        next (see join_arrivals)."""
        arr = (C.c_void_p * len(flag_arrays))(*[C.c_void_p(int(p)) for p in flag_arrays])
        fn = lib.kh_arm_arrival_flags_overlapped if overlapped else lib.kh_arm_arrival_flags
        _check(fn(self._h, arr, len(flag_arrays), epoch))

    def join_arrivals(self, stream=None):
        """Orders `stream` behind the wait of the last overlapped arrival barrier, if one is running."""
        _check(lib.kh_join_arrivals(self._h, stream))

    def gemm_clock(self):
        """(SM cycles, nanoseconds) block 0 of the last gemm launch counted over its life; call after
        synchronize. cycles / ns * 1000 is the SM clock in MHz while the tensor cores were busy."""
        cycles, ns = C.c_uint64(), C.c_uint64()
        _check(lib.kh_gemm_clock(self._h, C.byref(cycles), C.byref(ns)))
        return cycles.value, ns.value

    def enable_peer_access(self, peer: "Context"):
        """Maps the memory of `peer`'s GPU into this context's GPU (both in this process)."""
        _check(lib.kh_enable_peer_access(self._h, peer._h))

    # ---- typed entry points ----------------------------------------------------
    def vecadd(self, a, b, c, n, stream=None):
        _check(lib.kh_vecadd(self._h, _ptr(a), _ptr(b), _ptr(c), n, stream))

    def fused_gelu(self, x, out, n, stream=None):
        _check(lib.kh_fused_gelu(self._h, _ptr(x), _ptr(out), n, stream))

    def fused_gelu_bias(self, x, bias, out, n, stream=None):
        _check(lib.kh_fused_gelu_bias(self._h, _ptr(x), _ptr(bias), _ptr(out), n, stream))

    def scan(self, x, y, n, stream=None):
        _check(lib.kh_scan(self._h, _ptr(x), _ptr(y), n, stream))

    def scan_lookback_probe(self, x, y, n, poll_limit, stream=None):
        """Diagnostic: a scan whose first look-back runs out of `poll_limit` polls on purpose
        (no fault: the kernel stops and returns; `synchronize` then raises code 1001)."""
        _check(lib.kh_scan_lookback_probe(self._h, _ptr(x), _ptr(y), n, poll_limit, stream))

    def softmax(self, x, y, rows, cols, stream=None):
        _check(lib.kh_softmax(self._h, _ptr(x), _ptr(y), rows, cols, stream))

    def layernorm(self, x, gamma, beta, y, rows, cols, stream=None):
        _check(lib.kh_layernorm(self._h, _ptr(x), _ptr(gamma), _ptr(beta), _ptr(y), rows, cols,
                                stream))

    def gemm(self, a, b, c, m, n, k, stream=None):
        _check(lib.kh_gemm(self._h, _ptr(a), _ptr(b), _ptr(c), m, n, k, stream))

    def gemm_allgather(self, a_shard, b, c_replicas, rank, m_shard, n, k, stream=None):
        """Sharded gemm whose epilogue stores every C tile into all ranks' full C
        (`c_replicas`: addresses mapped on this device, this rank's own included)."""
        arr = (C.c_void_p * len(c_replicas))(*[_ptr(p) for p in c_replicas])
        _check(lib.kh_gemm_allgather(self._h, _ptr(a_shard), _ptr(b), arr, len(c_replicas), rank,
                                     m_shard, n, k, stream))

    def gemm_allgather_multicast(self, a_shard, b, c_local, c_multicast, world, rank, m_shard, n, k, stream=None):
        """Sharded gemm whose epilogue stores every C tile to `c_local` (this rank's
        full C) and sends it once through the replicas' NVLink multicast address
        (`c_multicast`), reaching all ranks' full C."""
        _check(lib.kh_gemm_allgather_multicast(self._h, _ptr(a_shard), _ptr(b), _ptr(c_local),
                                               C.c_void_p(int(c_multicast)), world, rank, m_shard, n, k, stream))

    def gemm_host_sharded_begin(self, a_shard_host, b_slice_host, b_replicas, b_multicast, rank, m_shard, n, k):
        """Phase 1 of the sharded gemm on HOST buffers: upload this rank's rows of B into its
        replica and send them to the other replicas, start the upload of the A shard. A barrier
        across the ranks must follow before `gemm_host_sharded_finish`."""
        arr = (C.c_void_p * len(b_replicas))(*[(None if p is None else _ptr(p)) for p in b_replicas])
        _check(lib.kh_gemm_host_sharded_begin(self._h, _ptr(a_shard_host), _ptr(b_slice_host), arr,
                                              C.c_void_p(int(b_multicast)) if b_multicast else None,
                                              len(b_replicas), rank, m_shard, n, k))

    def gemm_host_sharded_finish(self, c_shard_host):
        """Phase 2: prepare B, multiply, copy this rank's rows of C to `c_shard_host`; blocking."""
        _check(lib.kh_gemm_host_sharded_finish(self._h, _ptr(c_shard_host)))

    def attention(self, q, k, v, o, batch, heads, seq, head_dim, stream=None):
        _check(lib.kh_attention(self._h, _ptr(q), _ptr(k), _ptr(v), _ptr(o), batch, heads, seq,
                                head_dim, stream))

    def attention_allgather(self, q, k, v, o_replicas, o_multicast, rank, slices, seq, head_dim=64, stream=None):
        """Attention over this rank's `slices` (batch, head) problems whose output tiles also go to
        every other rank's copy of the whole output (`o_replicas`: addresses mapped on this device;
        `o_multicast`: the copies' NVLink multicast address, or 0 for plain peer stores)."""
        arr = (C.c_void_p * len(o_replicas))(*[(None if p is None else _ptr(p)) for p in o_replicas])
        _check(lib.kh_attention_allgather(self._h, _ptr(q), _ptr(k), _ptr(v), arr,
                                          C.c_void_p(int(o_multicast)) if o_multicast else None,
                                          len(o_replicas), rank, slices, seq, head_dim, stream))

    # ---- raw device memory -------------------------------------------------------
    def malloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        _check(lib.kh_malloc(self._h, nbytes, C.byref(p)))
        return p.value

    def free(self, ptr: int) -> None:
        _check(lib.kh_free(self._h, ptr))

    def memcpy_h2d(self, dst: int, src, nbytes: int) -> None:
        _check(lib.kh_memcpy_h2d(self._h, dst, _ptr(src), nbytes))

    def memcpy_d2h(self, dst, src: int, nbytes: int) -> None:
        _check(lib.kh_memcpy_d2h(self._h, _ptr(dst), src, nbytes))


def scan_noalloc(x, y, n: int, stream: int | None = None) -> None:
    """Inclusive prefix sum without any device allocation: for callers that own
    all device memory themselves or may not call an allocator. Uses a fixed
    scratch array inside the library (n <= scan_noalloc_max_elements()); the
    tensors' device must be current; calls on one device must not overlap."""
    _check(lib.kh_scan_noalloc(_ptr(x), _ptr(y), n, stream))


def scan_noalloc_max_elements() -> int:
    return int(lib.kh_scan_noalloc_max_elements())


def scan_noalloc_status(stream: int | None = None) -> None:
    """Waits for `stream`; raises code 1001 when the last scan_noalloc on the current
    device stopped on a look-back that ran out (reads 8 bytes, allocates nothing)."""
    _check(lib.kh_scan_noalloc_status(stream))


def wait_name(code: int) -> str:
    buf = C.create_string_buffer(64)
    lib.kh_wait_name(code, buf, 64)
    return buf.value.decode()


# --------------------------------------------------------------------------- host helpers
def device_count() -> int:
    n = C.c_int()
    _check(lib.kh_device_count(C.byref(n)))
    return n.value


def bench_sharded(gpus: int, kernel: str, shape: str, warmup: int = 5, iters: int = 20):
    """One partitioned bench row (gemm by M-row blocks, attention by (batch, head) slices) on
    `gpus` GPUs of this box from one process: (ms of the slowest rank, median; whole-job GFLOP/s)."""
    ms, rate, is_gflops = C.c_double(), C.c_double(), C.c_int()
    _check(lib.kh_bench_sharded(gpus, kernel.encode(), shape.encode(), warmup, iters,
                                C.byref(ms), C.byref(rate), C.byref(is_gflops)))
    return ms.value, rate.value


def registered_kernels() -> list[str]:
    buf = C.create_string_buffer(1024)
    _check(lib.kh_registered_kernels(buf, 1024))
    return buf.value.decode().split(",")


_registered_callbacks: dict[str, object] = {}


def register_kernel(name: str, image: bytes, entry: str, plan_fn) -> None:
    """The plug-in point (the reference's ``registerKernel``): add a kernel template or
    replace the one registered under `name`. `plan_fn(shape: dict, sm_count) -> dict` returns
    ``grid``, ``block``, ``elements`` (fp32 elements per buffer), ``outputs`` (indices) and
    optionally ``dynamic_smem``, ``work``, ``work_is_flops``; raising ValueError refuses the
    shape with that message."""

    def trampoline(shape_text, sm_count, out, error, error_cap, _user):
        try:
            shape = dict((k, int(v)) for k, v in (item.split("=") for item in shape_text.decode().split(",") if item))
            d = plan_fn(shape, sm_count)
            p = out.contents
            for i in range(3):
                p.grid[i] = (list(d["grid"]) + [1, 1])[i]
                p.block[i] = (list(d["block"]) + [1, 1])[i]
            p.dynamic_smem = int(d.get("dynamic_smem", 0))
            p.n_buffers = len(d["elements"])
            for i, n in enumerate(d["elements"]):
                p.elements[i] = int(n)
                p.is_output[i] = 1 if i in d.get("outputs", ()) else 0
            p.work = float(d.get("work", 0.0))
            p.work_is_flops = int(bool(d.get("work_is_flops", False)))
            return 0
        except Exception as exc:  # the message goes back through the C interface
            msg = str(exc).encode()[:max(error_cap - 1, 0)]
            C.memmove(error, msg + b"\0", len(msg) + 1)
            return 1

    cb = PLAN_FN(trampoline)
    _check(lib.kh_register_kernel(name.encode(), image, len(image), entry.encode(), cb, None))
    _registered_callbacks[name] = cb  # the library keeps calling it: keep it alive


def unregister_kernel(name: str) -> None:
    _check(lib.kh_unregister_kernel(name.encode()))
    _registered_callbacks.pop(name, None)


def plan(kernel: str, shape: str, target: str = "sm_100a", sm_count: int = 148) -> PlanInfo:
    info = PlanInfo()
    _check(lib.kh_plan(kernel.encode(), shape.encode(), target.encode(), sm_count, C.byref(info)))
    return info


def kernel_image(kernel: str) -> bytes:
    p, n = C.c_void_p(), C.c_size_t()
    _check(lib.kh_kernel_image(kernel.encode(), C.byref(p), C.byref(n)))
    return C.string_at(p.value, n.value)


RESOURCE_FIELDS = ("registers", "smem_bytes", "stack_bytes", "spill_store_bytes", "spill_load_bytes", "barriers")


def kernel_resources(kernel: str, entry: str | None = None, target: str = "sm_100a") -> tuple[dict, str]:
    """(figures, resources.json text) of an entry point, from the build's ptxas -v output."""
    buf = C.create_string_buffer(4096)
    f = (C.c_int64 * 6)()
    _check(lib.kh_kernel_resources(kernel.encode(), entry.encode() if entry else None, target.encode(), buf, 4096, f))
    return dict(zip(RESOURCE_FIELDS, [int(v) for v in f])), buf.value.decode()


def parse_ptxas(text: str, entry: str | None = None) -> dict:
    f = (C.c_int64 * 6)()
    _check(lib.kh_parse_ptxas(text.encode(), entry.encode() if entry else None, f))
    return dict(zip(RESOURCE_FIELDS, [int(v) for v in f]))


def occupancy_report(kernel: str, shape: str, target: str = "sm_100a", sm_count: int = 148) -> tuple[str, str]:
    """(occupancy.json text, occupancy.md text) for the launches the library makes."""
    js, md = C.create_string_buffer(16384), C.create_string_buffer(16384)
    _check(lib.kh_occupancy_report(kernel.encode(), shape.encode(), target.encode(), sm_count, js, 16384, md, 16384))
    return js.value.decode(), md.value.decode()


def pack_memrefs(ptrs, shapes) -> list[int]:
    flat = [d for s in shapes for d in s]
    ranks = [len(s) for s in shapes]
    P = (C.c_uint64 * len(ptrs))(*ptrs)
    S = (C.c_int64 * max(len(flat), 1))(*flat)
    R = (C.c_int * len(ranks))(*ranks)
    slots = (C.c_uint64 * 256)()
    n = C.c_int()
    _check(lib.kh_pack_memrefs(P, S, R, len(ptrs), slots, 256, C.byref(n)))
    return [int(slots[i]) for i in range(n.value)]


LIMIT_FIELDS = ("lds_bytes_per_workgroup", "wavefront_size", "max_threads_per_workgroup",
                "max_grid_x", "max_grid_y", "max_grid_z", "vram_bytes", "waves_per_cu",
                "reg_file_per_cu", "cu_count", "max_dynamic_smem_optin", "smem_per_sm",
                "max_blocks_per_sm", "tmem_columns_per_sm")


def device_limits(token: str) -> dict:
    f = (C.c_int64 * 14)()
    name = C.create_string_buffer(256)
    _check(lib.kh_device_limits(token.encode() if token is not None else None, f, name, 256))
    out = dict(zip(LIMIT_FIELDS, [int(v) for v in f]))
    out["name"] = name.value.decode()
    return out


def target_token(cli_target: str) -> str:
    buf = C.create_string_buffer(64)
    _check(lib.kh_target_token(cli_target.encode(), buf, 64))
    return buf.value.decode()


def verify_launch(token: str, threads: int, grid=(1, 1, 1), static_smem: int = 0,
                  dynamic_smem: int = 0, warps_per_sm_override: int = 0) -> str:
    """'' when the launch is acceptable, else every violation, one per line."""
    msg = C.create_string_buffer(8192)
    rc = lib.kh_verify_launch(token.encode(), threads, grid[0], grid[1], grid[2], static_smem,
                              dynamic_smem, warps_per_sm_override, msg, 8192)
    if rc not in (0, 1):
        _check(rc)
    return msg.value.decode()


def occupancy(token: str, regs: int, static_smem: int, threads: int, dynamic_smem: int = 0,
              tmem_columns: int = 0) -> dict:
    out5 = (C.c_int * 5)()
    pct = C.c_double()
    sm3 = (C.c_int * 3)()
    _check(lib.kh_occupancy(token.encode(), regs, static_smem, threads, dynamic_smem, tmem_columns,
                            out5, C.byref(pct), sm3))
    return {"vgpr_limited_waves": out5[0], "lds_limited_blocks": out5[1],
            "thread_limited_blocks": out5[2], "achieved_waves": out5[3],
            "limiter": ("none", "vgpr", "lds", "threads")[out5[4]], "theoretical_pct": pct.value,
            "sm_resident_blocks": sm3[0], "sm_occupancy_pct": sm3[1] / 100.0,
            "sm_limiter": ("none", "registers", "shared memory", "warps", "block cap",
                           "tensor memory")[sm3[2]]}


def metric(what: str, a: int = 0, b: int = 0, c: int = 0, d: int = 0) -> float:
    return lib.kh_metric(what.encode(), a, b, c, d)


def rate(gflops: bool, work: float, ms: float) -> float:
    return lib.kh_rate(int(gflops), work, ms)


def csv_header() -> str:
    buf = C.create_string_buffer(256)
    lib.kh_csv_header(buf, 256)
    return buf.value.decode()


def csv_line(kernel, shape, backend, ms, rate_, timestamp, device) -> str:
    buf = C.create_string_buffer(2048)
    lib.kh_csv_line(kernel.encode(), shape.encode(), backend.encode(), ms, rate_,
                    timestamp.encode(), device.encode(), buf, 2048)
    return buf.value.decode()


def csv_header_ext() -> str:
    buf = C.create_string_buffer(512)
    lib.kh_csv_header_ext(buf, 512)
    return buf.value.decode()


def csv_line_ext(kernel, shape, backend, ms, rate_, timestamp, device, gpus=1, roofline_frac=0.0, max_rel_err=-1.0,
                 cpu_ms=-1.0, cpu_cores=0) -> str:
    buf = C.create_string_buffer(2048)
    lib.kh_csv_line_ext(kernel.encode(), shape.encode(), backend.encode(), ms, rate_, timestamp.encode(),
                        device.encode(), gpus, roofline_frac, max_rel_err, cpu_ms, cpu_cores, buf, 2048)
    return buf.value.decode()


def shape_roundtrip(text: str) -> str:
    buf = C.create_string_buffer(1024)
    lib.kh_shape_roundtrip(text.encode(), buf, 1024)
    return buf.value.decode()
