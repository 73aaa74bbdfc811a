#!/usr/bin/env python
"""Benchmark of the hot path: fp32 GEMM 8192^3 (C = A.B, 3xFP16 on tcgen05) on
1/2/4/8 B200, with the memory-bound kernels' GB/s reported beside it at N = 1.

    python bench.py --gpus N --steps K --warmup W            # this repository's kernels
    python bench.py --impl reference --gpus N --steps K ...  # the reference's fp64 CPU routine

One "step" is one pass of the path over one batch of synthetic input: the
operand preparation (scaled fp16 hi/lo splits of A and of B^T), the tensor-core
GEMM and (N > 1) the all-gather of the C row shards. Rank 0 prints ONE JSON line. Under torchrun every rank owns one GPU;
A and C are sharded by M-row blocks, B is replicated before timing (input
placement), and the NCCL all-gather of C is inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SIZE = 8192
FLOPS = 2.0 * SIZE ** 3
METRIC = "fp32 GEMM 8192^3 TFLOP/s"
SEED = 0x4B310001


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="kernelh_b200", choices=["kernelh_b200", "reference"])
    ap.add_argument("--size", type=int, default=SIZE, help=argparse.SUPPRESS)
    ap.add_argument("--gather", default="p2p", choices=["p2p", "p2p-st", "nccl"],
                    help="N > 1: 'p2p' = the gemm epilogue stores C tiles into every rank's C over NVLink "
                         "(symmetric memory; one multimem.st per tile piece through the NVSwitch multicast "
                         "address when there is one, else plain peer stores) and a barrier follows; "
                         "'p2p-st' = the same, forcing plain peer stores; 'nccl' = plain gemm + NCCL all-gather")
    ap.add_argument("--barrier", default="flags", choices=["flags", "overlap", "symm"],
                    help="N > 1 with --gather p2p: 'flags' = the gemm kernel ends with the barrier itself (arrival "
                         "flags in symmetric memory, written after its last store and awaited by its last CTA); "
                         "'overlap' = the kernel only signals and the wait for the peers runs on a second stream "
                         "beside the next step's operand preparation (measured: no faster, the kernel itself is as "
                         "long as the traffic into the GPU); 'symm' = a symmetric-memory barrier launch after the kernel")
    ap.add_argument("--csv", default="", help="N = 1: also write the rows of this run as results CSV with the "
                                              "appended columns (gpus, roofline_frac, max_rel_err, cpu_ms, cpu_cores)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the memory-bound rows, the e2e leg and the CPU baseline")
    return ap.parse_args()


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["source"] = "measured"
        return p
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples the SM clock and the clock-event reasons during the timed region:
    NVML every 5 ms (reads only), or nvidia-smi every 100 ms when NVML cannot be
    loaded."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
                   0x40: "hw_thermal_slowdown"}

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []
        self.nvml = None
        self.samples: list[tuple[float, int]] = []
        self.max_mhz = None
        self.running = False

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            self.nvml = (pynvml, handle, reasons)
            self.running = True
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE,
                stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _poll(self):
        pynvml, handle, reasons = self.nvml
        while self.running:
            try:
                self.samples.append((float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)),
                                     int(reasons(handle))))
            except Exception:
                pass
            time.sleep(0.005)

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.nvml is not None:
            self.running = False
            self.thread.join(timeout=1.0)
            sm = sorted(mhz for mhz, _ in self.samples)
            mask = 0
            for _, bits in self.samples:
                mask |= bits
            found = sorted(name for bit, name in self.REASON_BITS.items() if mask & bit)
            return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz,
                    "sm_min_mhz": sm[0] if sm else None, "samples": len(sm), "reasons": found, "source": "nvml, 5 ms"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvidia-smi, 100 ms"}


# --------------------------------------------------------------------------- CPU arm
def cpu_gemm_sample(size: int, steps: int, warmup: int):
    """Times the reference's fp64 CPU routine (test/unit/e2e_gemm_test.cpp:92-108)
    on the host cores for a bounded sample of the workload's C rows. Uses the
    reference's own code when it was compiled here (oracle/_ref), else the oracle's
    restatement of it. Returns (tflops, cores, kind, sample text, ms per step)."""
    import numpy as np

    from oracle import oracle_py as O

    cores = os.cpu_count() or 1
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        pass
    a_full_rows = None
    b = O.uniform((size, size), SEED + 1, -1, 1)
    if O.ref_available():
        kind = "reference"
        threads = min(cores, 32)
        rows_per_thread = 4
        rows = threads * rows_per_thread
        a_full_rows = O.uniform((rows, size), SEED, -1, 1)
        R = O.ref()
        handle = R.khref_gemm_prepare(b.reshape(-1), size, size)
        out = np.empty((rows, size), np.float32)

        def one_step():
            ts = []
            for t in range(threads):
                lo = t * rows_per_thread
                th = threading.Thread(target=R.khref_gemm_rows, args=(
                    handle, a_full_rows[lo:lo + rows_per_thread].reshape(-1),
                    out[lo:lo + rows_per_thread].reshape(-1), rows_per_thread))
                th.start()
                ts.append(th)
            for th in ts:
                th.join()
    else:
        kind = "port"
        threads = O.num_threads()
        rows = max(threads * 4, 8)
        a_full_rows = O.uniform((rows, size), SEED, -1, 1)

        def one_step():
            O.gemm_ref(a_full_rows, b)

    for _ in range(min(warmup, 1)):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    dt = (time.perf_counter() - t0) / steps
    tflops = 2.0 * rows * size * size / dt / 1e12
    sample = (f"{rows} of {size} rows of C per step (full K and N), fp64 accumulation, "
              f"{threads} host threads")
    return tflops, threads, kind, sample, dt * 1e3


def reference_arm(args) -> None:
    """`--impl reference`: the reference's CPU implementation of the path, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tflops, threads, kind, sample, ms = cpu_gemm_sample(args.size, max(args.steps, 1), args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic",
        "config": {"workload": f"gemm m=n=k={args.size} fp32 row-major, A,B ~ U[-1,1) seeded",
                   "sample": sample},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": kind,
                         "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def time_rotating(torch, launch, sets, iters, use_graph=True):
    """Average ms per launch while rotating through `sets` argument sets whose
    total size exceeds L2. The launches are captured once into a CUDA graph and
    the graph is replayed, so the figure is the GPU's back-to-back rate and not
    the host's launch rate (these kernels run for 5-35 us). Falls back to a plain
    launch loop when capture is not possible. Returns (ms, method)."""
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        for s in sets:
            launch(s, stream)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if use_graph:
        try:
            per_graph = max(len(sets), (32 // len(sets)) * len(sets))
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                cs = torch.cuda.current_stream().cuda_stream
                for i in range(per_graph):
                    launch(sets[i % len(sets)], cs)
            replays = max(3, iters // per_graph)
            for _ in range(2):
                g.replay()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(replays):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / (replays * per_graph), "cuda graph replay"
        except Exception as exc:  # capture refused: time the plain loop instead
            sys.stderr.write(f"bench.py: graph capture failed ({exc}); timing a launch loop\n")
            torch.cuda.synchronize()
    e0.record()
    for i in range(iters):
        launch(sets[i % len(sets)], stream)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters, "launch loop"


NOMINAL_HBM_GBS = 8000.0  # the "about 8 TB/s" of the B200 data sheet, beside the measured copy rate


def cpu_row(fn, bytes_or_flops: float, is_flops: bool, kind: str, cores: int, sample: str) -> dict:
    """Times one call of a CPU reference routine (after one untimed call)."""
    fn()
    t0 = time.perf_counter()
    fn()
    ms = (time.perf_counter() - t0) * 1e3
    rate = bytes_or_flops / ms / 1e6
    return {"ms": ms, ("gflops" if is_flops else "gbs"): rate, "cores": cores, "kind": kind, "sample": sample}


def memory_bound_rows(torch, ctx, stream, hbm_peak: float) -> dict:
    """GB/s of the five HBM-bound kernels at the benchmark configurations' sizes
    (rotating through buffer sets larger than L2) and at a large size. The benchmark-size
    rows also carry the largest floored-relative error against the CPU oracle on seeded
    inputs and the time of the reference's CPU routine for the same shape."""
    import numpy as np

    from oracle import oracle_py as O

    out = {}
    R = O.ref() if O.ref_available() else None
    kind = "reference" if R is not None else "port"

    def row(name, kernel, shape, make, bytes_per_launch, nsets, iters=200, check=None, cpu=None):
        sets = [make() for _ in range(nsets)]
        ms, method = time_rotating(torch, lambda s, st: ctx.launch(kernel, shape, s, st), sets, iters)
        gbs = bytes_per_launch / ms / 1e6
        out[name] = {"shape": shape, "ms": ms, "gbs": gbs, "frac_of_measured_hbm": gbs / hbm_peak,
                     "frac_of_nominal_8tbs": gbs / NOMINAL_HBM_GBS, "buffer_sets": nsets, "timing": method}
        if check is not None:
            inputs, ref = check()
            dev_in = [torch.from_numpy(x).cuda() if x is not None else None for x in inputs]
            res = torch.full(ref.shape, float("nan"), device="cuda")
            ctx.launch(kernel, shape, dev_in + [res], stream)
            ctx.synchronize(stream)
            c = O.compare(res.cpu().numpy(), ref)
            out[name]["max_rel_err"] = c.max_rel
            if ref.dtype == np.float32:  # vecadd and scan: the oracle's result is the fp32 answer itself
                out[name]["bit_mismatches"] = int(O.bit_mismatches(res.cpu().numpy(), ref))
        if cpu is not None:
            out[name]["cpu"] = cpu()

    f = lambda *shape: torch.randn(*shape, device="cuda")
    n = 1 << 24
    va, vb = O.uniform(n, SEED, -1, 1), O.uniform(n, SEED + 1, -1, 1)
    row("vecadd", "vecadd", f"n={n}", lambda: [f(n), f(n), f(n)], 3 * n * 4, 3,
        check=lambda: ([va, vb], O.vecadd_ref(va, vb)),
        cpu=lambda: cpu_row(lambda: O.vecadd_ref(va, vb), 3 * n * 4, False, "port", O.num_threads(), f"all {n} elements"))
    n = 1 << 22
    gx, gb = O.normal(n, SEED, 0, 1), O.normal(n, SEED + 1, 0, 1)
    row("fused_gelu_bias", "fused_gelu", f"n={n},bias=1", lambda: [f(n), f(n), f(n)], 3 * n * 4, 8,
        check=lambda: ([gx, gb], O.bias_gelu_ref(gx, gb)))
    gout = np.empty(n, np.float64)
    row("fused_gelu", "fused_gelu", f"n={n}", lambda: [f(n), None, f(n)], 2 * n * 4, 8,
        check=lambda: ([gx, None], O.fused_gelu_ref(gx)),
        cpu=lambda: cpu_row((lambda: R.khref_gelu_ref(gx, gout, n, 0)) if R else (lambda: O.fused_gelu_ref(gx)),
                            2 * n * 4, False, kind, 1 if R else O.num_threads(), f"all {n} elements, fp64"))
    r, c = 4096, 1024
    sx = O.normal((r, c), SEED, 0, 2.0)
    sout = np.empty((r, c), np.float64)
    row("softmax", "softmax", f"rows={r},cols={c}", lambda: [f(r, c), f(r, c)], 2 * r * c * 4, 8,
        check=lambda: ([sx], O.softmax_ref(sx)),
        cpu=lambda: cpu_row((lambda: R.khref_softmax_ref(sx, sout, r, c)) if R else (lambda: O.softmax_ref(sx)),
                            2 * r * c * 4, False, kind, 1 if R else O.num_threads(), f"all {r} x {c}, fp64"))
    g, b = f(c), f(c)
    lg, lb = O.uniform(c, SEED + 1, 0.5, 1.5), O.normal(c, SEED + 2, 0, 0.1)
    lx = O.normal((r, c), SEED, 0, 1)
    row("layernorm", "layernorm", f"rows={r},cols={c}", lambda: [f(r, c), g, b, f(r, c)],
        2 * r * c * 4 + 2 * c * 4, 8, check=lambda: ([lx, lg, lb], O.layernorm_ref(lx, lg, lb)),
        cpu=lambda: cpu_row((lambda: R.khref_layernorm_ref(lx, lg, lb, sout, r, c, 1e-5)) if R else
                            (lambda: O.layernorm_ref(lx, lg, lb)), 2 * r * c * 4, False, kind,
                            1 if R else O.num_threads(), f"all {r} x {c}, fp64"))
    n = 1000000
    cx = O.uniform(n, SEED, 0, 1)
    row("scan", "scan", f"n={n}", lambda: [torch.rand(n, device="cuda"), f(n)], 2 * n * 4, 24,
        check=lambda: ([cx], O.scan_ref(cx)),
        cpu=lambda: cpu_row(lambda: O.scan_ref(cx), 2 * n * 4, False, "port", 1, f"all {n} elements, fp64 running sum"))
    # The floor at the small sizes: the driver's own device-to-device copy of 16 MiB (32 MiB of
    # traffic, what softmax, layernorm and fused_gelu move at their benchmark sizes), timed the
    # same way. A kernel at this rate is bounded by launch, ramp and drain, not by its own code.
    n = 1 << 22
    sets = [[f(n), f(n)] for _ in range(8)]
    ms, method = time_rotating(torch, lambda st, _stream: st[1].copy_(st[0]), sets, 200)
    out["d2d_copy_floor"] = {"shape": f"n={n}", "ms": ms, "gbs": 2 * n * 4 / ms / 1e6,
                             "frac_of_measured_hbm": 2 * n * 4 / ms / 1e6 / hbm_peak,
                             "frac_of_nominal_8tbs": 2 * n * 4 / ms / 1e6 / NOMINAL_HBM_GBS, "buffer_sets": 8,
                             "timing": method, "note": "cudaMemcpyAsync device to device, not a kernel of this library"}
    del sets
    # large sizes: one buffer set is already far larger than L2
    n = 1 << 28
    row("vecadd_large", "vecadd", f"n={n}", lambda: [f(n), f(n), f(n)], 3 * n * 4, 1, 20)
    row("fused_gelu_bias_large", "fused_gelu", f"n={n},bias=1", lambda: [f(n), f(n), f(n)], 3 * n * 4, 1, 20)
    r = 262144
    row("softmax_large", "softmax", f"rows={r},cols={c}", lambda: [f(r, c), f(r, c)], 2 * r * c * 4, 1, 20)
    row("layernorm_large", "layernorm", f"rows={r},cols={c}", lambda: [f(r, c), g, b, f(r, c)],
        2 * r * c * 4, 1, 20)
    r, c = 16384, 4096  # the second row-kernel configuration of the reference's suite: a block per row
    g4, b4 = f(c), f(c)
    row("softmax_16384x4096", "softmax", f"rows={r},cols={c}", lambda: [f(r, c), f(r, c)], 2 * r * c * 4, 1, 20)
    row("layernorm_16384x4096", "layernorm", f"rows={r},cols={c}", lambda: [f(r, c), g4, b4, f(r, c)],
        2 * r * c * 4, 1, 20)
    n = 1 << 26
    row("scan_large", "scan", f"n={n}", lambda: [torch.rand(n, device="cuda"), f(n)], 2 * n * 4, 1, 20)
    return out


def attention_rows(torch, ctx, peaks: dict) -> dict:
    """TFLOP/s (4 b h s^2 d useful flops) of the fused attention at the reference's
    benchmark shape and at a batched one; split pass included. Every row carries its
    roofline record against ONE denominator pair, the same as the gemm's: the measured
    16-bit tensor rate (burst and sustained) divided by the three fp16 products per
    fp32-class multiply-add. The reference shape also carries the time of the reference's
    fp64 CPU routine."""
    import numpy as np

    from oracle import oracle_py as O

    out = {}
    for name, (bsz, heads, seq, dim) in (("reference_shape", (1, 1, 1024, 64)), ("batched", (8, 16, 1024, 64))):
        shape = f"batch={bsz},heads={heads},seq={seq},head_dim={dim}"
        sets = [[torch.randn(bsz, heads, seq, dim, device="cuda") for _ in range(4)] for _ in range(4)]
        ms, method = time_rotating(torch, lambda s, st: ctx.launch("attention", shape, s, st), sets, 50)
        tflops = 4.0 * bsz * heads * seq * seq * dim / ms / 1e9
        ctx.profile(True)
        for i in range(8):
            ctx.launch("attention", shape, sets[i % 4], torch.cuda.current_stream().cuda_stream)
        prof = ctx.profile_report()
        ctx.profile(False)
        out[name] = {"shape": shape, "ms": ms, "tflops": tflops, "buffer_sets": 4, "timing": method,
                     "kernels_ms": {k_: v[1] / v[0] for k_, v in prof.items()},
                     "roofline": {"bound": "tensor", "achieved": tflops, "unit": "TFLOP/s",
                                  "peak_burst": peaks["bf16_tflops"] / 3.0, "frac_of_burst": tflops / (peaks["bf16_tflops"] / 3.0),
                                  "peak_sustained": peaks["bf16_tflops_sustained"] / 3.0,
                                  "frac_of_sustained": tflops / (peaks["bf16_tflops_sustained"] / 3.0),
                                  "peak_note": f"16-bit tensor rate of {peaks['source']} / 3; split pass included in the time"}}
    q, k, v = (O.normal((1, 1, 1024, 64), SEED + i, 0, 1) for i in range(3))
    out["reference_shape"]["cpu"] = cpu_row(lambda: O.attention_ref(q, k, v), 4.0 * 1024 * 1024 * 64, True, "port",
                                            O.num_threads(), "batch 1, 1 head, seq 1024, fp64")
    return out


def gpu_arm(args) -> None:
    import torch
    import torch.distributed as dist

    import kernelh_b200 as kh
    from kernelh_b200 import sharding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if rank == 0:
            sys.stderr.write(f"bench.py: --gpus {args.gpus} needs {args.gpus} ranks (torchrun), "
                             f"found WORLD_SIZE={world}\n")
        sys.exit(2)
    if not torch.cuda.is_available():
        sys.stderr.write("bench.py: no CUDA device; the kernels have no CPU path\n")
        sys.exit(77)
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = kh.Context(local_rank)
    stream = torch.cuda.current_stream().cuda_stream
    peaks = measured_peaks()
    size = args.size
    flops = 2.0 * size ** 3
    row_lo, row_hi = sharding.gemm_shard_shape(size, size, size, world, rank)["rows"]
    rows = row_hi - row_lo

    # Synthetic inputs, identical on every rank: A, B ~ U[-1, 1), seeded.
    gen = torch.Generator(device="cuda")
    gen.manual_seed(SEED)
    a = torch.rand(size, size, device="cuda", generator=gen) * 2 - 1
    b = torch.rand(size, size, device="cuda", generator=gen) * 2 - 1
    gather = "none"
    symm = None
    c = None
    multicast = 0
    flag_arrays = None
    epoch = [0]
    if world > 1 and args.gather in ("p2p", "p2p-st"):
        # Every rank's C lives in symmetric memory, so each rank holds an address for
        # every other rank's C and the gemm epilogue can store its tiles into all of them.
        try:
            import torch.distributed._symmetric_memory as symm_mem

            c = symm_mem.empty((size, size), dtype=torch.float32, device=torch.device("cuda", local_rank))
            symm = symm_mem.rendezvous(c, dist.group.WORLD.group_name)
            replicas = [int(p) for p in symm.buffer_ptrs]
            multicast = int(getattr(symm, "multicast_ptr", 0) or 0) if args.gather == "p2p" else 0
            c.zero_()
            gather = "p2p"
            if args.barrier in ("flags", "overlap"):
                # eight 64-bit arrival words per rank, zero before the first step
                flag_words = symm_mem.empty((8,), dtype=torch.int64, device=torch.device("cuda", local_rank))
                flag_symm = symm_mem.rendezvous(flag_words, dist.group.WORLD.group_name)
                flag_words.zero_()
                flag_arrays = [int(p) for p in flag_symm.buffer_ptrs]
                torch.cuda.synchronize()
                dist.barrier()
        except Exception as exc:  # no peer mapping on this box: use the collective instead
            if rank == 0:
                sys.stderr.write(f"bench.py: symmetric memory unavailable ({exc!r}); using NCCL all-gather\n")
            c = None
    if c is None:
        c = torch.zeros(size, size, device="cuda")
        gather = "nccl" if world > 1 else "none"
    a_shard = a[row_lo:row_hi]
    c_shard = c[row_lo:row_hi]

    def barrier():
        if world > 1:
            dist.barrier()

    def fused_gather_launch():
        if flag_arrays is not None:  # every rank counts the same launches, so the epochs agree
            epoch[0] += 1
            ctx.arm_arrival_flags(flag_arrays, epoch[0], overlapped=args.barrier == "overlap")
        if multicast:
            ctx.gemm_allgather_multicast(a_shard, b, c, multicast, world, rank, rows, size, size, stream)
        else:
            ctx.gemm_allgather(a_shard, b, replicas, rank, rows, size, size, stream)
        if flag_arrays is None:
            symm.barrier()  # all ranks' stores have landed before anyone reads C

    def step():
        if gather == "p2p":
            fused_gather_launch()
        else:
            ctx.gemm(a_shard, b, c_shard, rows, size, size, stream)
            if world > 1:
                sharding.gather_output(c, c_shard, dist)

    for _ in range(max(args.warmup, 3)):
        step()
    ctx.synchronize(stream)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches_before = ctx.launch_count()
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    ctx.join_arrivals(stream)  # the last step's wait for the peers belongs to the timed region
    e1.record()
    torch.cuda.synchronize()
    barrier()
    ms_total = e0.elapsed_time(e1)
    launches = ctx.launch_count() - launches_before
    clocks = sampler.stop() if rank == 0 else None
    ctx.synchronize(stream)
    if clocks is not None:
        # the clock the last timed gemm launch really ran at, counted inside the kernel (block 0:
        # SM cycles against the GPU's nanosecond timer), beside the management library's samples
        cycles, ns = ctx.gemm_clock()
        clocks["gemm_in_kernel_sm_mhz"] = round(cycles / ns * 1e3, 1) if ns else None
        clocks["gemm_in_kernel"] = {"sm_cycles": cycles, "ns": ns}
    t = torch.tensor([ms_total], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = t.item() / args.steps
    value = flops / (ms_step * 1e-3) / 1e12

    # ---- the dominant kernel alone, per-launch, on this rank's stream -------------------
    ctx.profile(True)
    for _ in range(args.steps):
        if gather == "p2p":
            fused_gather_launch()
        else:
            ctx.gemm(a_shard, b, c_shard, rows, size, size, stream)
    prof = ctx.profile_report()
    ctx.profile(False)
    if symm is not None:
        symm.barrier()
    multiply_entries = ("gemm", "gemm_n128", "gemm_allgather", "gemm_allgather_n128")  # 256- or 128-column tiles
    multiply_key = next(k_ for k_ in prof if k_ in multiply_entries)
    gemm_launches, gemm_ms = prof[multiply_key]
    kernel_ms = gemm_ms / gemm_launches
    achieved = (flops / world) / (kernel_ms * 1e-3) / 1e12
    # 3xFP16 ceiling: the measured 16-bit tensor rate (cuBLAS bf16; fp16 runs at
    # the same rate) divided by the three products per k-step. Sustained figure:
    # the kernel is timed inside a back-to-back loop.
    peak = peaks["bf16_tflops_sustained"] / 3.0
    traffic = None
    # DRAM bytes of one 8192^3 launch, from the committed ncu capture (text summary)
    tpath = os.path.join(ROOT, "profiles", "gemm_8192_dram_traffic.md")
    if size == 8192 and os.path.exists(tpath):
        with open(tpath) as f:
            found = re.search(r"^dram_bytes_per_launch:\s*(\d+)", f.read(), re.M)
        if found:
            traffic = int(found.group(1)) / world
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "peak_burst": peaks["bf16_tflops"] / 3.0,
                "frac_of_burst": achieved / (peaks["bf16_tflops"] / 3.0), "traffic": traffic, "kernel": multiply_key + " (tcgen05 3xFP16)",
                "kernel_ms": kernel_ms, "split_ms": sum(v[1] for k_, v in prof.items() if k_ not in multiply_entries) / gemm_launches,
                "split_kernels": {k_: v[1] / v[0] for k_, v in prof.items() if k_ not in multiply_entries},
                "peak_note": f"bf16_tflops_sustained of {peaks['source']} / 3 (three fp16 products per fp32-class multiply-add)"}

    # ---- parity of the timed path, asserted on every rank (checker, not measured) ----------
    # C is overwritten with NaN on every rank, ONE more step runs, and then every rank checks
    # its own copy of the whole C: no NaN may be left (every tile of every rank's row block
    # arrived in this step, not in an earlier one), and rows sampled from every rank's row
    # block must agree with an fp64 product of the same inputs.
    parity_failures = []
    c.fill_(float("nan"))
    torch.cuda.synchronize()
    barrier()
    step()
    torch.cuda.synchronize()
    barrier()
    per_block = size // world
    sample_rows = sorted({blk * per_block + off for blk in range(world)
                          for off in (0, per_block // 3, per_block - 1)})
    pick = torch.tensor(sample_rows, device="cuda")
    ref = a[pick].double() @ b.double()
    got = c[pick].double()
    rms = ref.pow(2).mean().sqrt()
    rel_bound = 1e-5 * size ** 0.5
    gemm_check = torch.stack([
        torch.nan_to_num(((got - ref).abs() / torch.maximum(ref.abs(), rms)).max(), nan=float("inf")),
        torch.nan_to_num((got - ref).norm() / ref.norm(), nan=float("inf")),
        torch.isnan(c).sum().double(),
        torch.nan_to_num((got - ref).abs().max() / rms, nan=float("inf"))])
    if world > 1:
        every = [torch.zeros_like(gemm_check) for _ in range(world)]
        dist.all_gather(every, gemm_check)
    else:
        every = [gemm_check]
    every = [e.tolist() for e in every]
    for r, (max_rel, rel_fro, nans, _) in enumerate(every):
        if not (max_rel <= rel_bound and rel_fro <= 1e-5 and nans == 0):
            parity_failures.append(f"gemm: rank {r}'s C has max floored-relative error {max_rel:.3g} "
                                   f"(bound {rel_bound:.3g}), rel. Frobenius {rel_fro:.3g} (bound 1e-5), "
                                   f"{int(nans)} elements never written")
    err = max(e[3] for e in every)
    parity = {"gemm": {"checked": f"{len(sample_rows)} rows ({len(sample_rows) // world} from every rank's row "
                                  "block) of every rank's C against fp64, after one step on a NaN-filled C",
                       "max_rel_floored_by_rank": [e[0] for e in every], "bound": rel_bound,
                       "rel_frobenius_by_rank": [e[1] for e in every], "frobenius_bound": 1e-5,
                       "unwritten_elements_by_rank": [int(e[2]) for e in every]}}

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32 (3xFP16 tensor-core products of scaled hi/lo splits, fp32 accumulate)",
        "data": "synthetic",
        "config": {"workload": f"gemm m=n=k={size} fp32 row-major, A,B ~ U[-1,1) seeded",
                   "sharding": (f"A and C by {world} M-row blocks, B replicated before timing; " + (
                       "all-gather fused into the gemm epilogue (" + (
                           "multimem.st through the NVSwitch multicast address of every rank's C" if multicast else
                           "peer stores over NVLink into every rank's C") +
                       ") + barrier, inside the timed step" if gather == "p2p" else
                       "NCCL all-gather of C inside the timed step")) if world > 1 else "single GPU",
                   "l2": "inputs (2 x 256 MiB) and the 512 MiB operand-split scratch are larger than the 126 MB L2",
                   "step": "gemm_split_a + gemm_prep_b + " + {"none": "gemm", "nccl": "gemm + nccl all_gather",
                                                                 "p2p": ("gemm_allgather signalling its arrival, the wait for the peers on a second stream beside the "
                                                                         "next step's preparation" if args.barrier == "overlap" else
                                                                         "gemm_allgather ending with its own arrival-flag barrier") if flag_arrays is not None
                                                                 else "gemm_allgather + symmetric-memory barrier"}[gather]},
        "roofline": roofline, "gpu_launches": int(launches),
        "sampled_max_err_over_rms": err, "parity": parity,
    }
    if clocks is not None:
        line["clocks"] = clocks

    # ---- end to end through the host-buffer entry points -------------------------------------
    if not args.no_extras:
        a_h = a_shard.cpu().pin_memory()
        c_h = torch.empty(rows, size).pin_memory()
        shape = f"m={rows},n={size},k={size}"
        e2e_steps = max(3, args.steps)
        b_symm = None
        if world > 1 and gather == "p2p" and size % world == 0:
            # every rank uploads only ITS rows of B; the slices are exchanged over NVLink
            try:
                b_dev = symm_mem.empty((size, size), dtype=torch.float32, device=torch.device("cuda", local_rank))
                b_symm = symm_mem.rendezvous(b_dev, dist.group.WORLD.group_name)
                b_reps = [int(p) for p in b_symm.buffer_ptrs]
                b_mc = int(getattr(b_symm, "multicast_ptr", 0) or 0) if args.gather == "p2p" else 0
            except Exception as exc:
                if rank == 0:
                    sys.stderr.write(f"bench.py: symmetric memory for B unavailable ({exc!r}); every rank uploads all of B\n")
                b_symm = None
        if b_symm is not None:
            k_lo, k_hi = rank * (size // world), (rank + 1) * (size // world)
            b_h = b[k_lo:k_hi].cpu().pin_memory()

            def e2e_step():
                ctx.gemm_host_sharded_begin(a_h, b_h, b_reps if not b_mc else
                                            [b_dev if i == rank else None for i in range(world)],
                                            b_mc, rank, rows, size, size)
                b_symm.barrier()           # every rank's slice of B has been sent
                torch.cuda.synchronize()
                ctx.gemm_host_sharded_finish(c_h)
            e2e_note = ("kh_gemm_host_sharded_begin / _finish on pinned host buffers, per rank: H2D of this rank's 1/N of "
                        "the rows of B, sent on to every rank's B over NVLink (" + ("multimem.st" if b_mc else "peer stores") +
                        ") while the A shard goes up in row blocks; barrier; B is split, each A block is split and multiplied "
                        "as it arrives and the finished rows of C go back over the other direction of the link")
        else:
            b_h = b.cpu().pin_memory()

            def e2e_step():
                ctx.run_host("gemm", shape, [a_h, b_h, c_h])
            e2e_note = ("kh_run_host on pinned host buffers, per rank: H2D of B, then the A shard in about eight row "
                        "blocks; each block is split and multiplied while the next is on the wire and the finished rows "
                        "of C go back over the other direction of the link")
        e2e_step()
        barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.synchronize()
        dt = torch.tensor([(time.perf_counter() - t0) / e2e_steps], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        line["e2e"] = {"value": flops / dt.item() / 1e12, "unit": "TFLOP/s",
                       "h2d_bytes_per_step": int(a_h.numel() * 4 + b_h.numel() * 4),
                       "d2h_bytes_per_step": int(c_h.numel() * 4), "steps": e2e_steps,
                       "ms_per_step": dt.item() * 1e3, "note": e2e_note}
        # The rows that came back to the host against the device path's: bit for bit when both paths cut
        # the product into the same work units, and within the gemm's bound otherwise (the host path
        # multiplies row blocks as they arrive, the device path may split its last wave of tiles over K:
        # a different order of the same fp32 additions). Checked on every rank.
        dev_rows = c_shard.cpu()
        e2e_equal = torch.equal(c_h, dev_rows)
        e2e_rms = dev_rows.double().pow(2).mean().sqrt()
        e2e_diff = ((c_h.double() - dev_rows.double()).abs() / torch.maximum(dev_rows.double().abs(), e2e_rms)).max().item()
        e2e_stats = torch.tensor([1.0 if e2e_equal else 0.0, -e2e_diff], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(e2e_stats, op=dist.ReduceOp.MIN)
        line["e2e"]["bit_identical_with_device_path"] = bool(e2e_stats[0].item() == 1.0)
        line["e2e"]["max_rel_diff_from_device_path"] = -e2e_stats[1].item()
        line["e2e"]["matches_device_path"] = bool(-e2e_stats[1].item() <= rel_bound)
        if not line["e2e"]["matches_device_path"]:
            parity_failures.append(f"e2e: the rows of C that came back to the host differ from the device path's by "
                                   f"{-e2e_stats[1].item():.3e} floored-relative (bound {rel_bound:.3e})")
        del a_h, b_h, c_h

    if world > 1:
        # Batched attention sharded by (batch, head): every rank runs its share of the 8 x 16
        # independent problems and the output slices are collected with one NCCL all-gather,
        # inside the timed step.
        bsz, heads, seq, dim = 8, 16, 1024, 64
        shard = sharding.attention_shard_shape(bsz, heads, seq, dim, world, rank)
        lo, hi = shard["units"]
        even = (bsz * heads) % world == 0
        # the same seeded Q, K, V on every rank (so that any rank can check any slice); a rank
        # works on its own (batch, head) slices of them
        gen.manual_seed(SEED + 7)
        qkv_all = [torch.randn(bsz * heads, seq, dim, device="cuda", generator=gen) for _ in range(3)]
        qkv = [t[lo:hi].contiguous() if hi > lo else t[:1].contiguous() for t in qkv_all]
        o_symm = None
        att_mode = "none"
        if even and gather == "p2p":
            # the whole output lives in symmetric memory on every rank; the kernel sends its tiles there
            try:
                o_full = symm_mem.empty((bsz * heads, seq, dim), dtype=torch.float32,
                                        device=torch.device("cuda", local_rank))
                o_symm = symm_mem.rendezvous(o_full, dist.group.WORLD.group_name)
                o_reps = [int(p) for p in o_symm.buffer_ptrs]
                o_mc = int(getattr(o_symm, "multicast_ptr", 0) or 0) if args.gather == "p2p" else 0
                att_mode = "fused"
            except Exception as exc:
                if rank == 0:
                    sys.stderr.write(f"bench.py: symmetric memory for the attention output unavailable ({exc!r})\n")
                o_symm = None
        if o_symm is None:
            o_full = torch.empty(bsz * heads, seq, dim, device="cuda")
            att_mode = "nccl" if even else "none"
        o_shard = o_full[lo:hi] if even else torch.empty(max(hi - lo, 1), seq, dim, device="cuda")
        shard_shape = f"batch={hi - lo},heads=1,seq={seq},head_dim={dim}"

        def attention_step():
            if att_mode == "fused":
                ctx.attention_allgather(qkv[0], qkv[1], qkv[2], o_reps if not o_mc else
                                        [o_full if i == rank else None for i in range(world)],
                                        o_mc, rank, hi - lo, seq, dim, stream)
                o_symm.barrier()
                return
            if hi > lo:
                ctx.launch("attention", shard_shape, qkv + [o_shard], stream)
            if att_mode == "nccl":
                sharding.gather_output(o_full, o_shard, dist)

        for _ in range(3):
            attention_step()
        barrier()
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(10):
            attention_step()
        a1.record()
        torch.cuda.synchronize()
        att = torch.tensor([a0.elapsed_time(a1) / 10], device="cuda")
        dist.all_reduce(att, op=dist.ReduceOp.MAX)
        # parity, on every rank: NaN-fill the whole output, one more step, then the first and the
        # last slice of every rank's share (of this rank's own share when nothing is gathered)
        # against an fp64 evaluation; no NaN may be left anywhere a slice was due.
        o_full.fill_(float("nan"))
        if att_mode == "none":
            o_shard.fill_(float("nan"))
        torch.cuda.synchronize()
        barrier()
        attention_step()
        torch.cuda.synchronize()
        barrier()
        per = (bsz * heads) // world if even else 0
        owners = range(world) if att_mode != "none" else [rank]
        worst_rel, worst_violation = 0.0, 0.0
        for owner in owners:
            o_lo, o_hi = (owner * per, (owner + 1) * per) if even else (lo, hi)
            for sl in sorted({o_lo, o_hi - 1}) if o_hi > o_lo else []:
                q64, k64, v64 = (t[sl].double() for t in qkv_all)
                ref = torch.softmax(q64 @ k64.T / dim ** 0.5, -1) @ v64
                got = (o_full[sl] if att_mode != "none" else o_shard[sl - lo]).double()
                d = (got - ref).abs()
                rel = torch.nan_to_num((d / torch.maximum(ref.abs(), ref.pow(2).mean().sqrt())).max(), nan=float("inf"))
                vio = torch.nan_to_num((d / (2e-3 + 2e-3 * ref.abs())).max(), nan=float("inf"))
                worst_rel, worst_violation = max(worst_rel, rel.item()), max(worst_violation, vio.item())
        out_checked = o_full if att_mode != "none" else o_shard
        att_check = torch.tensor([worst_rel, worst_violation, float(torch.isnan(out_checked).sum().item())],
                                 device="cuda", dtype=torch.float64)
        att_every = [torch.zeros_like(att_check) for _ in range(world)]
        dist.all_gather(att_every, att_check)
        att_every = [e.tolist() for e in att_every]
        att_bound = 1e-5 * seq ** 0.5
        for r, (rel, vio, nans) in enumerate(att_every):
            if not (rel <= att_bound and vio <= 1.0 and nans == 0):
                parity_failures.append(f"attention_sharded: rank {r}'s output has max floored-relative error "
                                       f"{rel:.3g} (bound {att_bound:.3g}), |d| / (2e-3 + 2e-3 |ref|) = {vio:.3g} "
                                       f"(bound 1), {int(nans)} elements never written")
        parity["attention_sharded"] = {
            "checked": "first and last (batch, head) slice of every rank's share in every rank's copy of the "
                       "output against fp64, after one step on a NaN-filled output",
            "max_rel_floored_by_rank": [e[0] for e in att_every], "bound": att_bound,
            "reference_tolerance_ratio_by_rank": [e[1] for e in att_every],
            "unwritten_elements_by_rank": [int(e[2]) for e in att_every]}
        line["attention_sharded"] = {"shape": f"batch={bsz},heads={heads},seq={seq},head_dim={dim}",
                                     "sharding": f"(batch, head) slices over {world} ranks" + {
                                         "fused": "; all-gather of the output fused into the kernel (" + (
                                             "multimem.st" if att_mode == "fused" and o_mc else "peer stores") +
                                             " over NVLink) + barrier, inside the timed step",
                                         "nccl": "; output slices all-gathered (NCCL) inside the timed step",
                                         "none": "; uneven split, no gather"}[att_mode],
                                     "ms": att.item(),
                                     "tflops": 4.0 * bsz * heads * seq * seq * dim / att.item() / 1e9}

    if rank == 0 and world == 1 and not args.no_extras:
        del a, b, c
        torch.cuda.empty_cache()
        line["memory_bound"] = memory_bound_rows(torch, ctx, stream, peaks["hbm_gbs"])
        line["attention"] = attention_rows(torch, ctx, peaks)
        line["memory_bound_peak"] = {"hbm_gbs": peaks["hbm_gbs"], "source": peaks["source"],
                                     "nominal_hbm_gbs": NOMINAL_HBM_GBS}
        if args.csv:
            # the rows of this run in the harness's CSV, with the columns appended after the reference's seven
            stamp = time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())
            device = torch.cuda.get_device_name(0)
            with open(args.csv, "w") as f:
                f.write(kh.csv_header_ext() + "\n")
                f.write(kh.csv_line_ext("gemm", f"m={size},n={size},k={size}", "kernelh", ms_step, value * 1e3, stamp, device,
                                        world, roofline["frac"], parity["gemm"]["max_rel_floored_by_rank"][0]) + "\n")
                for name, r_ in line["memory_bound"].items():
                    if name == "d2d_copy_floor":  # the driver's copy, not a kernel of the harness's list
                        continue
                    kernel = name.split("_large")[0].split("_16384")[0].replace("_bias", "")
                    cpu = r_.get("cpu", {})
                    f.write(kh.csv_line_ext(kernel, r_["shape"], "kernelh", r_["ms"], r_["gbs"], stamp, device, 1,
                                            r_["frac_of_measured_hbm"], r_.get("max_rel_err", -1.0),
                                            cpu.get("ms", -1.0), cpu.get("cores", 0)) + "\n")
                for name, r_ in line["attention"].items():
                    cpu = r_.get("cpu", {})
                    f.write(kh.csv_line_ext("attention", r_["shape"], "kernelh", r_["ms"], r_["tflops"] * 1e3, stamp, device,
                                            1, r_["roofline"]["frac_of_sustained"], -1.0, cpu.get("ms", -1.0),
                                            cpu.get("cores", 0)) + "\n")
        tflops, threads, kind, sample, _ = cpu_gemm_sample(size, 2, 1)
        line["cpu_baseline"] = {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": kind,
                                "sample": sample}
    ctx.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if parity_failures:
        # identical on every rank (the figures were all-gathered): every rank exits non-zero
        if rank == 0:
            sys.stderr.write("bench.py: PARITY FAILURE, no result line printed\n" +
                             "".join(f"  {f}\n" for f in parity_failures))
        sys.exit(1)
    if rank == 0:
        print(json.dumps(line), flush=True)


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
