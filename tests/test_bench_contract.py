"""The benchmark's command-line contract on a machine without a GPU: the
reference arm (the reference's own fp64 CPU routine, timed on the host cores)
prints one JSON line with the agreed keys, and the GPU arm refuses to run
instead of falling back to anything."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True,
                          text=True, cwd=ROOT, timeout=300)


def test_reference_arm_prints_the_contract_line():
    if not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "libkernelh_ref.so")) and \
            not os.path.exists(os.path.join(ROOT, "oracle", "liboracle.so")):
        pytest.skip("the CPU oracle has not been built (make -C oracle)")
    r = run_bench("--impl", "reference", "--size", "512", "--steps", "1", "--warmup", "1")
    assert r.returncode == 0, r.stderr
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["unit"] == "TFLOP/s" and line["higher_is_better"] is True
    assert line["metric"] == "fp32 GEMM 8192^3 TFLOP/s" and line["n_gpus"] == 1
    assert line["steps"] == 1 and line["value"] > 0 and line["ms_per_step"] > 0
    assert line["vs_baseline"] is None and line["gpu_launches"] == 0 and line["data"] == "synthetic"
    base = line["cpu_baseline"]
    assert base["kind"] in ("reference", "port") and base["cores"] >= 1 and base["value"] == line["value"]
    assert "rows of C" in base["sample"] and "workload" in line["config"]
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}


def test_gpu_arm_refuses_to_run_without_a_device():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    r = run_bench("--steps", "1", "--warmup", "1")
    assert r.returncode == 77
    assert "no CPU path" in r.stderr and not [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
