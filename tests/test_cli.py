"""The `kernelh` command-line tool: the reference CLI's grammar, messages and
exit codes (tools/kernelh/main.cpp:125-158, 375-390) for the verbs that touch
this path, plus the new `run` verb."""
import os
import re
import subprocess

import numpy as np
import pytest

import kernelh_b200 as kh

CLI = os.path.join(os.path.dirname(kh.LIB_PATH), "bin", "kernelh")


def cli(*args):
    return subprocess.run([CLI, *args], capture_output=True, text=True)


def test_compile_writes_the_sm100a_code_object(tmp_path):
    r = cli("compile", "--kernel", "softmax", "--shape", "rows=4096,cols=1024", "--target",
            "nvptx-sm_100a", "--out", str(tmp_path))
    assert r.returncode == 0, r.stderr
    assert r.stdout.splitlines() == [f"wrote {tmp_path}/softmax.cubin", f"wrote {tmp_path}/resources.json",
                                     "compile ok"]
    blob = (tmp_path / "softmax.cubin").read_bytes()
    assert blob[:4] == b"\x7fELF" and b"softmax" in blob  # ELF magic; the entry symbol is in the symbol table
    assert blob == kh.kernel_image("softmax")
    # resources.json beside it: the reference's seven keys first, filled from the build's ptxas -v
    import json
    res = json.loads((tmp_path / "resources.json").read_text())
    assert list(res)[:7] == ["kernel", "target", "vgpr_count", "sgpr_count", "lds_bytes", "wavefront_size",
                             "occupancy_estimate"]
    assert res["kernel"] == "softmax" and res["target"] == "sm_100a" and res["wavefront_size"] == 32
    assert 16 <= res["vgpr_count"] <= 255 and res["sgpr_count"] == 0
    assert res["occupancy_estimate"] == min(64, 65536 // (res["vgpr_count"] * 32))
    assert res["entry"] == "softmax" and res["spill_store_bytes"] == 0
    # --flag=value form
    r = cli("compile", "--kernel=vecadd", "--target=nvptx-sm_100a", f"--out={tmp_path}")
    assert r.returncode == 0 and (tmp_path / "vecadd.cubin").exists()


def test_compile_errors_and_exit_codes(tmp_path):
    r = cli("compile", "--kernel", "gemm", "--target", "nvptx-sm_90", "--out", str(tmp_path))
    assert r.returncode == 1 and "valid --target values" in r.stderr
    r = cli("compile", "--kernel", "gemm", "--target", "nvptx-sm_80", "--out", str(tmp_path))
    assert r.returncode == 1 and "only carries sm_100a code objects" in r.stderr
    r = cli("compile", "--kernel", "nope", "--target", "nvptx-sm_100a", "--out", str(tmp_path))
    assert r.returncode == 1 and "unknown kernel template 'nope'; registered kernels:" in r.stderr
    r = cli("compile", "--kernel", "gemm", "--shape", "m=4,n=4", "--target", "nvptx-sm_100a", "--out",
            str(tmp_path))
    assert r.returncode == 1 and "shape attribute 'k' is required" in r.stderr
    assert cli("compile", "--kernel", "gemm").returncode == 2
    assert cli().returncode == 2
    assert cli("explore").returncode == 2
    assert cli("run", "--kernel").returncode == 2


def test_occupancy_report_for_the_planned_launch():
    r = cli("bench", "--occupancy", "--kernel", "attention", "--shape",
            "batch=8,heads=16,seq=1024,head_dim=64", "--target", "nvptx-sm_100a")
    assert r.returncode == 0
    import json
    reports = json.loads(r.stdout)["reports"]  # one per launch: attention_split, attention
    assert [x["kernel"] for x in reports] == ["attention_split", "attention"]
    main = reports[1]
    assert main["threads_per_workgroup"] == 512 and main["sm_resident_blocks"] == 1
    # the registers ptxas reported are fed in: the register bound is a real number, not "unknown"
    assert main["vgpr_count"] == kh.kernel_resources("attention")[0]["registers"] > 64
    assert main["vgpr_limited_waves"] == 65536 // (main["vgpr_count"] * 32)


def test_occupancy_report_files(tmp_path):
    r = cli("bench", "--occupancy", "--kernel", "gemm", "--shape", "m=8192,n=8192,k=8192", "--target",
            "nvptx-sm_100a", "--out", str(tmp_path))
    assert r.returncode == 0, r.stderr
    assert f"wrote {tmp_path}/occupancy.json" in r.stdout and f"wrote {tmp_path}/occupancy.md" in r.stdout
    import json
    reports = json.loads((tmp_path / "occupancy.json").read_text())["reports"]
    gemm = [x for x in reports if x["kernel"] == "gemm"][0]
    # 320 threads of 168 registers: one cluster CTA per SM, and the registers say so
    assert gemm["vgpr_count"] >= 128 and gemm["sm_resident_blocks"] == 1 and gemm["sm_limiter"] == "registers"
    md = (tmp_path / "occupancy.md").read_text()
    assert md.startswith("# Occupancy report") and "| gemm_prep_b |" in md and "| gemm |" in md
    # a single-launch kernel gives a single report object, like the reference's occupancy.json
    r = cli("bench", "--occupancy", "--kernel", "vecadd", "--shape", "n=16777216", "--target", "nvptx-sm_100a")
    one = json.loads(r.stdout)
    assert one["kernel"] == "vecadd" and one["threads_per_workgroup"] == 256 and one["vgpr_count"] > 0


def test_run_and_bench_skip_with_77_without_a_device():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    assert cli("run", "--kernel", "vecadd", "--shape", "n=1024").returncode == 77
    assert cli("bench", "--kernel", "vecadd", "--shape", "n=1024").returncode == 77


@pytest.mark.gpu
def test_run_matches_the_oracle_on_bit_exact_kernels(oracle, tmp_path):
    n = 100000
    r = cli("run", "--kernel", "vecadd", "--shape", f"n={n}", "--seed", "0x27ab13", "--dump",
            str(tmp_path / "c.bin"))
    assert r.returncode == 0, r.stderr
    s = oracle.LcgStream(0x27AB13)
    a, b = s.fill(n), s.fill(n)
    ref = oracle.vecadd_ref(a, b)
    got = np.fromfile(tmp_path / "c.bin", np.float32)
    assert oracle.bit_mismatches(got, ref) == 0
    assert f"fnv1a={oracle.fnv1a(ref):016x}" in r.stdout and "run ok" in r.stdout


@pytest.mark.gpu
def test_bench_row_and_results_csv(tmp_path):
    r = cli("bench", "--kernel", "softmax", "--shape", "rows=4096,cols=1024", "--warmup", "2",
            "--iters", "5", "--out", str(tmp_path))
    assert r.returncode == 0, r.stderr
    assert re.search(r"bench: kernelh softmax \[rows=4096,cols=1024\] ms_median=\d+\.\d+ rate=\d+\.\d+ GB/s",
                     r.stdout)
    lines = (tmp_path / "results.csv").read_text().splitlines()
    assert lines[0] == "kernel,shape,backend,ms_median,gflops_or_gbps,timestamp,device"
    assert lines[1].startswith('softmax,"rows=4096,cols=1024",kernelh,') and "B200" in lines[1]


def test_bench_gpus_flag_is_validated_before_any_device_is_opened():
    r = cli("bench", "--kernel", "gemm", "--shape", "m=512,n=256,k=64", "--gpus", "9")
    assert r.returncode == 2 and "--gpus must be between 1 and 8" in r.stderr
    r = cli("bench", "--kernel", "gemm", "--shape", "m=512,n=256,k=64", "--gpus", "0")
    assert r.returncode == 2


@pytest.mark.gpu
def test_bench_on_two_gpus_partitions_gemm_and_attention_and_replicates_the_rest():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    r = cli("bench", "--kernel", "gemm", "--shape", "m=2048,n=1024,k=512", "--gpus", "2", "--warmup", "2", "--iters", "3")
    assert r.returncode == 0, r.stderr
    assert re.search(r"bench: kernelh gemm \[m=2048,n=1024,k=512\] ms_median=\S+ rate=\S+ GFLOPS gpus=2 partitioned", r.stdout)
    r = cli("bench", "--kernel", "attention", "--shape", "batch=2,heads=4,seq=256,head_dim=64", "--gpus", "2",
            "--warmup", "2", "--iters", "3")
    assert r.returncode == 0, r.stderr
    assert "gpus=2 partitioned" in r.stdout
    r = cli("bench", "--kernel", "vecadd", "--shape", "n=1048576", "--gpus", "2", "--warmup", "2", "--iters", "3")
    assert r.returncode == 0, r.stderr
    assert "gpus=2 replicas" in r.stdout
