/*
 * kernelh_b200 - C ABI of the B200 (sm_100a) implementation of kernel.h's
 * seven launched kernel templates.
 *
 * This header is the drop-in boundary. kernel.h itself is a C++23 program with
 * no foreign-function interface; what a replacement of its launch path must
 * offer is (a) the kernel-name + shape-map operator surface of its template
 * registry and CLI, (b) its runtime's launch objects, and (c) the pure host
 * helpers its harness and tests use. Each entry point below names the
 * reference interface it stands in for (paths relative to the reference
 * project root). All pointers are plain pointers, all sizes plain integers.
 *
 * Conventions
 *   - Every function returns 0 on success. 77 means "no usable CUDA driver or
 *     device" (the reference's skip code, include/kernelh/runtime/
 *     runtime_error.hpp:15-20), 2 means a usage error (unknown kernel, bad
 *     shape, wrong buffer count), 1001 means a device-side bounded wait ran
 *     out, any other value is the driver's error code.
 *   - kh_last_error() returns the message of the calling thread's last failure.
 *   - Tensors are fp32, row-major, contiguous. Device-pointer calls enqueue on
 *     `stream` (a CUstream / cudaStream_t, NULL = default stream) and return
 *     without waiting. There is no CPU path: without a B200 the compute calls
 *     fail with 77 or the driver's error.
 *   - A context is bound to one device and is not thread-safe; scratch memory
 *     (operand splits, scan state) belongs to the context, so launches of one
 *     context must not overlap on the GPU across streams.
 */
#ifndef KERNELH_B200_H
#define KERNELH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct kh_context kh_context;

const char *kh_last_error(void);
const char *kh_version(void);

/* ---- device context -------------------------------------------------------
 * make_cuda_backend() + DeviceContext::create(backend, ordinal)
 * (include/kernelh/runtime/backend.hpp:98-104, device_context.hpp:22-23). */
int kh_context_create(int device_ordinal, kh_context **out);
void kh_context_destroy(kh_context *ctx);
int kh_device_count(int *count);
/* DeviceInfo (include/kernelh/runtime/backend.hpp:32-39) plus the B200 fields. */
typedef struct {
  char name[256];
  int64_t vram_bytes;
  int64_t static_smem_per_block;
  int64_t optin_smem_per_block;
  int64_t smem_per_sm;
  int64_t l2_bytes;
  int32_t sm_count;
  int32_t warp_size;
  int32_t max_threads_per_block;
  int32_t regs_per_sm;
  int32_t max_blocks_per_sm;
  int32_t cc_major;
  int32_t cc_minor;
  int32_t ordinal;
} kh_device_info;
int kh_device_info_get(kh_context *ctx, kh_device_info *out);

/* ---- operator surface: kernel name + shape --------------------------------
 * program().kernel(name).shape(map) (include/kernelh/dsl/program.hpp:85-149)
 * followed by the runtime launch the reference's callers do by hand
 * (bench/harness/kernelh_backend.cpp:205-436). `shape` is the CLI text
 * "k=v,k=v" (tools/kernelh/main.cpp:242-266). Buffers are passed in template
 * order:
 *   vecadd     n                       a, b, c
 *   fused_gelu n | rows,cols [bias=1]  x, tmp (may be NULL), out | x, bias, out
 *   scan       n                       x, y
 *   softmax    rows, cols              x, y
 *   layernorm  rows, cols              x, gamma, beta, y
 *   gemm       m, n, k                 A, B, C
 *   attention  batch, heads, seq, head_dim   Q, K, V, O
 * Launch geometry and scratch are chosen by the library. */
int kh_launch(kh_context *ctx, const char *kernel, const char *shape, void *const *device_buffers,
              int n_buffers, void *stream);
/* Same call on host buffers: inputs are copied to the device, the kernel runs,
 * outputs are copied back; blocking. This is the path the reference's
 * end-to-end checks take (Buffer::copy_from_host, launch, copy_to_host:
 * test/unit/e2e_gemm_test.cpp:130-206). */
int kh_run_host(kh_context *ctx, const char *kernel, const char *shape, void *const *host_buffers,
                int n_buffers);
/* Waits for `stream` and reports a device-side wait that ran out (1001). */
int kh_synchronize(kh_context *ctx, void *stream);

/* The reference runtime's own launch sequence, for callers that keep choosing
 * launch geometry themselves: GpuModule::load(image) + get_function(entry) +
 * KernelLaunch(...).grid().block().shared_mem_bytes().memref_arg()...launch()
 * (include/kernelh/runtime/gpu_module.hpp, kernel_launch.hpp; lib/runtime/
 * kernel_launch.cpp:100-132). `image` is a code object (e.g. from
 * kh_kernel_image); buffers are packed as memref descriptors (ptrs[i] with
 * ranks[i] dims taken from `shapes`). The launch is verified against the device
 * limits first and refused (code 1, "KernelLaunch::launch refused: ..." with
 * every violation) when it cannot run; a bad image gives the driver's error. */
int kh_module_launch(kh_context *ctx, const void *image, size_t image_size, const char *entry,
                     const uint32_t grid[3], const uint32_t block[3], size_t dynamic_smem,
                     const uint64_t *ptrs, const int64_t *shapes, const int *ranks, int n_memrefs,
                     void *stream);

/* Per-launch device timing (the reference times launches with GPU events,
 * include/kernelh/runtime/event_timer.hpp): while enabled, every kernel launch
 * of this context is bracketed by events on its stream. kh_profile_report
 * waits for them and writes "entry:launches:total_ms;..." into buf.
 * kh_launch_count returns how many kernels the context has launched so far. */
int kh_profile_enable(kh_context *ctx, int on);
int kh_profile_report(kh_context *ctx, char *buf, int cap);
int kh_launch_count(kh_context *ctx, uint64_t *count);

/* Typed forms of kh_launch, one per template (lib/dsl/kernels/<name>.cpp). */
int kh_vecadd(kh_context *ctx, const float *a, const float *b, float *c, int64_t n, void *stream);
int kh_fused_gelu(kh_context *ctx, const float *x, float *out, int64_t n, void *stream);
int kh_fused_gelu_bias(kh_context *ctx, const float *x, const float *bias, float *out, int64_t n,
                       void *stream);
int kh_scan(kh_context *ctx, const float *x, float *y, int64_t n, void *stream);
int kh_softmax(kh_context *ctx, const float *x, float *y, int64_t rows, int64_t cols, void *stream);
int kh_layernorm(kh_context *ctx, const float *x, const float *gamma, const float *beta, float *y,
                 int64_t rows, int64_t cols, void *stream);
int kh_gemm(kh_context *ctx, const float *a, const float *b, float *c, int64_t m, int64_t n,
            int64_t k, void *stream);
int kh_attention(kh_context *ctx, const float *q, const float *k, const float *v, float *o,
                 int64_t batch, int64_t heads, int64_t seq, int64_t head_dim, void *stream);

/* C = alpha * A.B + beta * C, the scaled store that BLAS-style callers expect (the
 * reference's gemm epilogue is a plain store, lib/dsl/kernels/gemm.cpp:47-53; this is
 * the first of its generalisations). alpha = 1, beta = 0 is kh_gemm bit for bit;
 * beta = 0 never reads C, so C may hold anything, NaN included. */
int kh_gemm_scaled(kh_context *ctx, const float *a, const float *b, float *c, int64_t m, int64_t n, int64_t k,
                   float alpha, float beta, void *stream);

/* No counterpart in the reference (which is single-GPU). The M-row-sharded gemm
 * for several GPUs of one box with the all-gather of the C shards fused into
 * the kernel's epilogue: `a_shard` is this rank's m_shard x k rows of A, `b`
 * the whole k x n B, and `c_replicas[i]` (i < world <= 8) the address, mapped
 * on this device, of rank i's full (world*m_shard) x n C, this rank's own
 * included. Every finished tile is stored to all replicas at row
 * rank*m_shard (plain peer stores over NVLink; nothing is loaded from a peer).
 * The caller runs a barrier across ranks after the kernel before reading C. */
int kh_gemm_allgather(kh_context *ctx, const float *a_shard, const float *b, void *const *c_replicas,
                      int world, int rank, int64_t m_shard, int64_t n, int64_t k, void *stream);

/* No counterpart in the reference. The same with the C replicas bound to one
 * NVLink multicast object (NVSwitch systems): `c_local` is this rank's own
 * (world*m_shard) x n C and `c_multicast` the multicast address of that buffer
 * across all ranks (e.g. torch symmetric memory's multicast_ptr). Every tile
 * is stored to c_local and then sent once with multimem.st; the switch
 * delivers it to every rank, so a rank's links carry its shard once instead
 * of world-1 times. Same barrier rule as kh_gemm_allgather. */
int kh_gemm_allgather_multicast(kh_context *ctx, const float *a_shard, const float *b, float *c_local,
                                void *c_multicast, int world, int rank, int64_t m_shard, int64_t n,
                                int64_t k, void *stream);

/* No counterpart in the reference. The M-row-sharded gemm on HOST buffers, for
 * several GPUs of one box, without uploading the whole B once per rank: in
 * phase `begin` a rank uploads only ITS slice of B, rows [rank*k/world,
 * (rank+1)*k/world) given as `b_slice_host`, into its own replica of B
 * (`b_replicas[rank]`, a full k x n device buffer) and sends it on to every
 * other replica over NVLink (multimem.st through `b_multicast`, the replicas'
 * multicast address, or plain peer stores when it is null; `b_replicas[i]` is
 * rank i's replica as mapped on this device), while the upload of the A shard
 * (m_shard x k, `a_shard_host`) starts; begin returns when the slice has left.
 * The caller then passes a barrier across the ranks, and phase `finish`
 * prepares B, multiplies the A blocks as they arrive and copies the rank's
 * m_shard x n rows of C to `c_shard_host`, returning when they are there. k
 * must be divisible by world. No other call may use the context between the
 * two phases. Results are bit-identical with kh_gemm. */
int kh_gemm_host_sharded_begin(kh_context *ctx, const float *a_shard_host, const float *b_slice_host,
                               void *const *b_replicas, void *b_multicast, int world, int rank,
                               int64_t m_shard, int64_t n, int64_t k);
int kh_gemm_host_sharded_finish(kh_context *ctx, float *c_shard_host);

/* No counterpart in the reference. Attention over (batch, head) slices sharded
 * across the GPUs of one box with the all-gather of the output fused into the
 * kernel: q, k, v are this rank's `slices` x seq x head_dim problems; every
 * rank keeps the whole (world*slices) x seq x head_dim output, `o_replicas[i]`
 * being rank i's copy as mapped on this device. Every finished 128-row tile is
 * stored to this rank's copy at slice rank*slices and sent to the others:
 * with multimem.st through `o_multicast` (the copies' NVLink multicast
 * address; then only o_replicas[rank] is read) or, when it is null, with plain
 * peer stores. Same barrier rule as kh_gemm_allgather. */
int kh_attention_allgather(kh_context *ctx, const float *q, const float *k, const float *v,
                           void *const *o_replicas, void *o_multicast, int world, int rank, int64_t slices,
                           int64_t seq, int64_t head_dim, void *stream);

/* No counterpart in the reference. The scan for callers that must not allocate
 * device memory (memory-pool owners, allocator-free plugin callbacks, fixed
 * audited budgets): same result as kh_scan, but the look-back scratch is a
 * fixed array inside the library image instead of a cuMemAlloc'ed buffer, so
 * the call allocates and frees nothing. n may not exceed
 * kh_scan_noalloc_max_elements() (16,777,216; larger n is refused with code 2).
 * The owning device must be current; the first call on a device resolves the
 * array's address (under a lock: concurrent first calls are safe) and should
 * be made outside stream capture; calls on one device share the array and
 * must not overlap on the GPU. A look-back that runs out is not reported by
 * this call: ask kh_scan_noalloc_status. */
int kh_scan_noalloc(const float *x, float *y, int64_t n, void *stream);
int64_t kh_scan_noalloc_max_elements(void);
/* No counterpart in the reference. kh_scan_noalloc has no context that could
 * report a look-back that ran out of its poll budget: this call waits for
 * `stream`, reads the status word of the fixed array on the current device
 * (an 8-byte copy, nothing is allocated) and returns 1001 when the last
 * kh_scan_noalloc there stopped early and left y incomplete, else 0. */
int kh_scan_noalloc_status(void *stream);

/* No counterpart in the reference (whose kernels have no waits). A diagnostic
 * that shows, on a healthy GPU and without any fault, what a device-side
 * bounded wait that runs out looks like: the scan is launched with every tile
 * ticket shifted by one, so tile 0 is never produced and the look-back of tile
 * 1 gives up after `poll_limit` polls (1..1048576; a few thousand take about
 * a millisecond). The kernel then stops and returns; the next kh_synchronize
 * on the stream returns 1001 with the wait named in kh_last_error(), and the
 * context stays usable. n must cover at least two 12288-element tiles; y is
 * left incomplete. */
int kh_scan_lookback_probe(kh_context *ctx, const float *x, float *y, int64_t n, uint32_t poll_limit,
                           void *stream);
/* Name of a device-side wait code as kh_synchronize reports it (1 = "scan
 * look-back wait", 2 = "TMA (full-stage) wait", ...). */
int kh_wait_name(uint32_t code, char *buf, int cap);

/* Device memory of the context's device (Buffer::allocate / copy_from_host /
 * copy_to_host, include/kernelh/runtime/buffer.hpp). */
int kh_malloc(kh_context *ctx, size_t bytes, void **out);
int kh_free(kh_context *ctx, void *ptr);
int kh_memcpy_h2d(kh_context *ctx, void *dst, const void *src, size_t bytes);
int kh_memcpy_d2h(kh_context *ctx, void *dst, const void *src, size_t bytes);

/* One timed bench row: warm-up launches, then the median of `iters`
 * event-timed launches (bench/harness/timer.cpp:29-67), and the rate by the
 * reference's metric formulas (bench/harness/metrics.cpp:14-52). Buffers are
 * allocated by the library and filled with a fixed pattern. */
int kh_bench_row(kh_context *ctx, const char *kernel, const char *shape, int warmup, int iters,
                 double *ms_median, double *rate, int *rate_is_gflops);

/* The barrier after a fused all-gather, done by the kernel itself. Arms the NEXT
 * kh_gemm_allgather / kh_gemm_allgather_multicast call of this context (that one
 * call only): flag_arrays[i] is rank i's array of eight 64-bit words, zero at the
 * start, in peer-mapped (symmetric) memory as seen from this device. The last CTA
 * of the launch writes `epoch` into word `rank` of every other rank's array after
 * a system-wide fence, then waits (two seconds at most; then kh_synchronize gives
 * 1001 naming the rank that did not arrive) until its own array holds `epoch` or
 * more in every other word. When the kernel has completed, every rank's rows are
 * in this rank's C: no separate barrier launch is needed. `epoch` must be positive
 * and grow from call to call, the same on every rank. Every rank must run on a GPU
 * of its own: kernels that wait for one another must never share a GPU. */
int kh_arm_arrival_flags(kh_context *ctx, void *const *flag_arrays, int world, uint64_t epoch);
/* The same barrier with its wait taken out of the kernel: the armed launch only signals, and the
 * wait for the peers runs as a one-thread launch on a second stream of the context, behind the
 * kernel and beside whatever the caller enqueues next - typically the next step's operand
 * preparation, which needs nothing from the peers. The next kh_gemm_allgather* call of the context
 * orders its gemm (not its preparation) behind that wait; kh_join_arrivals(ctx, stream) orders
 * `stream` behind it (call it before reading C or recording an event that should include it), and
 * kh_synchronize waits for it and reports a wait that ran out (1001) like any other. */
int kh_arm_arrival_flags_overlapped(kh_context *ctx, void *const *flag_arrays, int world, uint64_t epoch);
int kh_join_arrivals(kh_context *ctx, void *stream);

/* The SM clock the last gemm launch of this context really ran at: block 0 of the
 * kernel counts its SM's cycles against the GPU's nanosecond timer over its whole
 * life; cycles / nanoseconds * 1000 = MHz under load (the management library's
 * samples mostly fall into the gaps between kernels). Call after kh_synchronize. */
int kh_gemm_clock(kh_context *ctx, uint64_t *sm_cycles, uint64_t *nanoseconds);

/* The harness on several GPUs of one box, in ONE process (the reference's harness
 * opens ordinal 0 only, bench/harness/run_bench.cpp:146-153): a context per GPU,
 * every GPU's memory mapped into every other (kh_enable_peer_access: the driver's
 * peer mapping; afterwards a pointer of `peer` is valid in kernels of `ctx`), the
 * gemm sharded by M-row blocks with B on every GPU, attention by (batch, head)
 * slices; every rank stores its finished tiles into every replica of the output
 * with plain peer stores inside its kernel, and the host waits for all ranks, which
 * is the barrier. ms_median is the median over `iters` steps of the slowest rank's
 * event-timed step, rate the whole job's GFLOP/s. Only gemm (m a multiple of
 * 256 * gpus) and attention (batch * heads a multiple of gpus) are partitioned;
 * any other kernel name is refused with code 2. 77 when fewer GPUs are visible. */
int kh_enable_peer_access(kh_context *ctx, kh_context *peer);
int kh_bench_sharded(int gpus, const char *kernel, const char *shape, int warmup, int iters, double *ms_median,
                     double *rate, int *rate_is_gflops);

/* ---- registry ----------------------------------------------------------------
 * registeredKernels() and the unknown-name error of emit()
 * (lib/dsl/registry.cpp:23-42, lib/dsl/program.cpp:27-37). */
int kh_registered_kernels(char *buf, int cap); /* comma separated, sorted */
/* registerKernel(name, fn) (include/kernelh/dsl/program.hpp:64-67,
 * lib/dsl/registry.cpp:39-42): the plug-in point. Adds a kernel template, or
 * REPLACES the one registered under `name`, built-ins included. Where the
 * reference registers a function that emits IR, the registered value here is a
 * finished kernel: an sm_100a code object (copied), the entry symbol in it,
 * and a callback that validates a shape and lays out the launch. The entry
 * takes its buffers as rank-1 fp32 memref descriptors (five 8-byte parameters
 * each: allocated pointer, aligned pointer, offset, size, stride), in the order
 * of kh_custom_plan.elements. The callback gets the shape as "k=v,k=v" text
 * (keys sorted) and the SM count; it returns 0, or non-zero with a message in
 * `error` that surfaces as "<name> template: <message>" (code 2).
 * kh_unregister_kernel takes such a record away again: a built-in it had
 * replaced comes back, any other name disappears. */
typedef struct {
  uint32_t grid[3], block[3];
  size_t dynamic_smem;
  int32_t n_buffers;      /* 1..8 */
  int64_t elements[8];    /* fp32 elements per buffer */
  uint8_t is_output[8];
  double work;            /* flops or bytes for the bench rate */
  int32_t work_is_flops;
} kh_custom_plan;
typedef int (*kh_plan_fn)(const char *shape_text, int sm_count, kh_custom_plan *out, char *error, int error_cap,
                          void *user);
int kh_register_kernel(const char *name, const void *image, size_t image_size, const char *entry, kh_plan_fn plan,
                       void *user);
int kh_unregister_kernel(const char *name);
/* The launch plan for a shape on a device-limits token ("sm_100a"): counts of
 * caller buffers, scratch bytes, launches, and the main launch's geometry. */
typedef struct {
  int32_t n_buffers;
  int32_t n_launches;
  int64_t workspace_bytes;
  char entry[64];          /* entry symbol of the last (main) launch */
  uint32_t grid[3];
  uint32_t block[3];
  int64_t dynamic_smem;
  int32_t param_count;     /* kernel parameters of the main launch */
  int32_t tmem_columns;
  double work;             /* flops or bytes per the reference's conventions */
  int32_t work_is_flops;
} kh_plan_info;
int kh_plan(const char *kernel, const char *shape, const char *target_token, int sm_count,
            kh_plan_info *out);
/* The embedded sm_100a code object that holds a kernel's entry symbols (what
 * `kernelh compile --target nvptx-sm_100a` writes as <name>.cubin). */
int kh_kernel_image(const char *kernel, const void **image, size_t *size);

/* Resource figures of a kernel's entry point, from the `ptxas -v` output of the
 * build that made the embedded code object: the reference's resources.json
 * (lib/compiler/resource_reporter.cpp:674-690: kernel, target, vgpr_count,
 * sgpr_count, lds_bytes, wavefront_size, occupancy_estimate) followed by the
 * entry symbol, barriers, stack and spill bytes. `entry` NULL or "" = the
 * entry named like the kernel. fields6 (may be NULL): registers, static
 * shared bytes, stack bytes, spill store bytes, spill load bytes, barriers. */
int kh_kernel_resources(const char *kernel, const char *entry, const char *target_token, char *json, int cap,
                        int64_t *fields6);
/* The parser behind it, on any `ptxas -v` text (resource_reporter.cpp:614-660):
 * the figures of `entry` (NULL or "" = the first entry in the text). */
int kh_parse_ptxas(const char *text, const char *entry, int64_t *fields6);
/* `kernelh bench --occupancy` (tools/kernelh/main.cpp:2082-2126): the analytic
 * occupancy report of every launch the library makes for `shape`, fed with the
 * registers and static shared memory of kh_kernel_resources, as occupancy.json
 * and occupancy.md text (either buffer may be NULL). */
int kh_occupancy_report(const char *kernel, const char *shape, const char *target_token, int sm_count, char *json,
                        int json_cap, char *markdown, int markdown_cap);

/* ---- host helpers ----------------------------------------------------------------
 * LaunchArgs::add_memref (lib/runtime/descriptor_packing.cpp:19-39): packs
 * `count` buffers; shapes are concatenated, ranks[i] dims each. Returns the
 * slot count through *n_slots. */
int kh_pack_memrefs(const uint64_t *ptrs, const int64_t *shapes, const int *ranks, int count,
                    uint64_t *slots, int cap, int *n_slots);
/* device_limits_for(token) (lib/compiler/device_limits.cpp:122-134). fields:
 * lds, warp, max_threads, grid x/y/z, vram, warps_per_sm, regs_per_sm, sms,
 * optin_smem, smem_per_sm, max_blocks_per_sm, tmem_columns. */
int kh_device_limits(const char *token, int64_t *fields14, char *name, int name_cap);
/* CLI target -> table token (tools/kernelh/main.cpp:375-390); 2 if unknown,
 * with the list of valid targets in kh_last_error(). */
int kh_target_token(const char *cli_target, char *buf, int cap);
/* LaunchVerifier::verify (lib/compiler/launch_verifier.cpp:109-172): 0 when
 * launchable, 1 with every violation, one per line, in `msg`. */
int kh_verify_launch(const char *token, int threads, int gx, int gy, int gz, uint64_t static_smem,
                     uint64_t dynamic_smem, int warps_per_sm_override, char *msg, int cap);
/* occupancy_report (lib/compiler/occupancy.cpp:124-223). out5: register-limited
 * warps, smem-limited blocks, thread-limited blocks, achieved, limiter
 * (0 none, 1 vgpr, 2 lds, 3 threads); sm3: resident blocks per SM, per-SM
 * occupancy percent x 100, limiter index (0 none, 1 registers, 2 shared
 * memory, 3 warps, 4 block cap, 5 tensor memory). */
int kh_occupancy(const char *token, int regs, int64_t static_smem, int threads, int64_t dynamic_smem,
                 int tmem_columns, int *out5, double *theoretical_pct, int *sm3);
/* bench/harness/metrics.cpp:14-52 by name ("gemm_flops", "scan_bytes", ...). */
double kh_metric(const char *what, int64_t a, int64_t b, int64_t c, int64_t d);
double kh_rate(int gflops, double work, double ms);
/* bench/harness/csv.cpp:9-57. */
int kh_csv_header(char *buf, int cap);
int kh_csv_line(const char *kernel, const char *shape, const char *backend, double ms, double rate,
                const char *timestamp, const char *device, char *buf, int cap);
/* The same line with the columns this build appends AFTER the reference's seven (so existing
 * consumers keep parsing those): gpus, roofline_frac, max_rel_err, cpu_ms, cpu_cores. A
 * negative max_rel_err / cpu_ms means "not checked / not timed" and prints an empty field. */
int kh_csv_header_ext(char *buf, int cap);
int kh_csv_line_ext(const char *kernel, const char *shape, const char *backend, double ms, double rate,
                    const char *timestamp, const char *device, int gpus, double roofline_frac, double max_rel_err,
                    double cpu_ms, int cpu_cores, char *buf, int cap);
/* parse_shape_text + shape_to_text (bench/harness/shape_text.cpp:10-44). */
int kh_shape_roundtrip(const char *text, char *buf, int cap);

#ifdef __cplusplus
}
#endif

#endif /* KERNELH_B200_H */
