"""Host logic of the runtime through the C ABI, against the fixtures generated
from the reference's own host code (tests/golden/make_golden.py), plus the
B200 additions. Runs without a GPU."""
import ctypes as C
import os
import re
import subprocess

import pytest

import kernelh_b200 as kh

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "kernelh_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(kh_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 30
    out = subprocess.run(["nm", "-D", "--defined-only", kh.LIB_PATH], capture_output=True, text=True,
                         check=True).stdout
    exported = set(re.findall(r" T (kh_[a-z0-9_]+)", out))
    assert declared <= exported, sorted(declared - exported)
    for name in declared:
        assert hasattr(kh.lib, name)
    assert b"sm_100a" in kh.lib.kh_version()


def test_descriptor_packing_matches_reference(golden):
    for case in golden["host"]["descriptor_slots"]:
        assert kh.pack_memrefs(case["ptrs"], case["shapes"]) == case["slots"]
    # rank-1 / rank-2 / rank-4 descriptors take 5 / 7 / 11 eight-byte slots
    assert len(kh.pack_memrefs([8], [[16]])) == 5
    assert len(kh.pack_memrefs([8], [[4, 4]])) == 7
    assert len(kh.pack_memrefs([8], [[2, 2, 2, 2]])) == 11
    slots = kh.pack_memrefs([0x1000], [[3, 5, 7]])
    assert slots == [0x1000, 0x1000, 0, 3, 5, 7, 35, 7, 1]


def test_device_limits_table(golden):
    ref = golden["host"]["device_limits"]
    for tok in ("gfx1101", "sm_80"):
        got = kh.device_limits(tok)
        assert [got[f] for f in kh.LIMIT_FIELDS[:10]] == ref[tok]["fields"]
        assert got["name"] == ref[tok]["name"]
        assert got["max_dynamic_smem_optin"] == 0  # the reference's targets have no opt-in carve-out
    b200 = kh.device_limits("sm_100a")
    assert b200["lds_bytes_per_workgroup"] == 49152
    assert b200["max_dynamic_smem_optin"] == 232448
    assert b200["smem_per_sm"] == 233472
    assert (b200["wavefront_size"], b200["max_threads_per_workgroup"]) == (32, 1024)
    assert (b200["waves_per_cu"], b200["reg_file_per_cu"], b200["max_blocks_per_sm"]) == (64, 65536, 32)
    assert b200["tmem_columns_per_sm"] == 512
    assert b200["cu_count"] == 0  # runtime query
    assert "sm_100a" in b200["name"]
    with pytest.raises(kh.KernelhError) as e:
        kh.device_limits("sm_999")
    # same text as the reference apart from the longer list of known targets
    assert e.value.message == ref["unknown_message_sm_999"] + ", sm_100a"
    with pytest.raises(kh.KernelhError):
        kh.device_limits("")


def test_cli_target_tokens():
    assert kh.target_token("nvptx-sm_100a") == "sm_100a"
    assert kh.target_token("nvptx-sm_80") == "sm_80"
    assert kh.target_token("amdgcn-gfx1101") == "gfx1101"
    with pytest.raises(kh.KernelhError) as e:
        kh.target_token("nvptx-sm_90")
    assert e.value.code == kh.USAGE_ERROR and "valid --target values" in e.value.message
    assert "nvptx-sm_100a" in e.value.message


def test_launch_verifier_matches_reference_messages(golden):
    for c in golden["host"]["launch_verifier"]:
        msg = kh.verify_launch(c["target"], c["threads"], c["grid"], c["shared"], 0,
                               c["waves_per_cu_override"])
        assert msg == c["message"], c
        assert (msg != "") == (c["rc"] != 0)


def test_launch_verifier_dynamic_shared_memory_rule():
    assert kh.verify_launch("sm_100a", 192, (2048, 1, 1), 48, 197632) == ""
    assert kh.verify_launch("sm_100a", 192, (1, 1, 1), 0, 232448) == ""
    msg = kh.verify_launch("sm_100a", 192, (1, 1, 1), 1024, 232448)
    assert "static + dynamic 233472 bytes exceeds the 232448-byte opt-in limit" in msg
    # a target without opt-in keeps the static limit for the sum
    msg = kh.verify_launch("sm_80", 256, (1, 1, 1), 0, 65536)
    assert "no opt-in carve-out" in msg
    # every rule still reports at once
    msg = kh.verify_launch("sm_100a", 4100, (1, 1, 70000), 50000, 300000)
    assert len(msg.splitlines()) == 6


def test_occupancy_matches_reference(golden):
    for c in golden["host"]["occupancy"]:
        got = kh.occupancy(c["target"], c["vgpr"], c["lds"], c["threads"])
        assert [got["vgpr_limited_waves"], got["lds_limited_blocks"], got["thread_limited_blocks"],
                got["achieved_waves"]] == c["out"][:4]
        assert ("none", "vgpr", "lds", "threads").index(got["limiter"]) == c["out"][4]
        assert got["theoretical_pct"] == pytest.approx(c["pct"])


def test_occupancy_b200_per_sm_view():
    # gemm: 320 threads, ~200 registers, 80 B static + 197632 B dynamic, 512 TMEM columns
    o = kh.occupancy("sm_100a", 200, 80, 320, 197632, 512)
    assert o["sm_resident_blocks"] == 1 and o["sm_limiter"] in ("registers", "shared memory", "tensor memory")
    assert o["sm_occupancy_pct"] == pytest.approx(100.0 * 10 / 64, abs=0.01)
    # a streaming kernel: 256 threads, 40 registers -> 6 blocks by registers, 8 by warps
    o = kh.occupancy("sm_100a", 40, 0, 256)
    assert o["sm_resident_blocks"] == 6 and o["sm_limiter"] == "registers"
    # tensor memory as the limiter
    o = kh.occupancy("sm_100a", 32, 0, 128, 1024, 512)
    assert o["sm_resident_blocks"] == 1 and o["sm_limiter"] == "tensor memory"


def test_metrics_and_rates_match_reference(golden):
    for m in golden["host"]["metrics"]:
        assert kh.metric(m["what"], *m["args"]) == m["value"]
    for r in golden["host"]["rates"]:
        assert kh.rate(bool(r["gflops"]), r["work"], r["ms"]) == r["value"]
    assert kh.metric("vecadd_bytes", 1 << 24) == 201326592.0
    assert kh.metric("nonsense") == -1.0


def test_csv_matches_reference(golden):
    assert kh.csv_header() == golden["host"]["csv"]["header"]
    for c in golden["host"]["csv"]["lines"]:
        assert kh.csv_line(*c["row"]) == c["line"]


def test_shape_text_matches_reference(golden):
    for c in golden["host"]["shape_text"]:
        assert kh.shape_roundtrip(c["text"]) == c["roundtrip"], c


def test_registry_lists_sorted_names_and_rejects_unknown():
    names = kh.registered_kernels()
    assert names == sorted(names)
    assert names == list(kh.REGISTERED)  # the seven templates and the reference's scan_totals
    with pytest.raises(kh.KernelhError) as e:
        kh.plan("nope", "n=4")
    assert e.value.message.startswith("unknown kernel template 'nope'; registered kernels: ")
    assert "attention, fused_gelu, gemm" in e.value.message


@pytest.mark.parametrize("kernel,shape,missing", [
    ("vecadd", "m=4", "'n'"), ("scan", "m=4", "'n'"), ("gemm", "m=4,n=4", "'k'"),
    ("softmax", "rows=4", "'rows' and 'cols'"), ("layernorm", "cols=4", "'rows' and 'cols'"),
    ("fused_gelu", "rows=4", "'n', or 'rows' AND 'cols'"),
    ("attention", "batch=1,heads=1,seq=64", "'head_dim'"),
])
def test_shape_errors_name_the_key(kernel, shape, missing):
    with pytest.raises(kh.KernelhError) as e:
        kh.plan(kernel, shape)
    assert e.value.code == kh.USAGE_ERROR
    assert kernel + " template" in e.value.message and missing in e.value.message


def test_shape_value_rules():
    for kernel, shape in (("vecadd", "n=0"), ("gemm", "m=4,n=-1,k=4"), ("softmax", "rows=0,cols=4"),
                          ("attention", "batch=1,heads=1,seq=0,head_dim=64")):
        with pytest.raises(kh.KernelhError) as e:
            kh.plan(kernel, shape)
        assert "must be positive" in e.value.message
    # seq need not be a multiple of the 64-key tile (the reference's template refuses that,
    # lib/dsl/kernels/attention.cpp:109-120): such shapes take the entry that masks the missing keys
    p = kh.plan("attention", "batch=1,heads=1,seq=100,head_dim=64")
    assert p.entry == b"attention_masked" and p.param_count == 53
    assert p.workspace_bytes == 128 * 64 * 2 * 6 + 2 * 3 * 4  # the splits hold whole tiles: 128 rows
    with pytest.raises(kh.KernelhError) as e:
        kh.plan("attention", "batch=1,heads=1,seq=128,head_dim=32")
    assert "pinned to head_dim = 64" in e.value.message


def test_plans_for_the_benchmark_configurations():
    p = kh.plan("vecadd", "n=16777216")
    assert (p.n_buffers, p.n_launches, p.param_count) == (3, 1, 15)
    assert p.block[0] == 256 and p.grid[0] % 148 == 0 or p.grid[0] <= 148 * 6
    assert p.work == 201326592.0 and not p.work_is_flops
    p = kh.plan("fused_gelu", "n=4194304,bias=1")
    assert p.entry == b"fused_gelu_bias" and p.work == 50331648.0
    assert kh.plan("fused_gelu", "rows=2048,cols=2048").entry == b"fused_gelu"
    p = kh.plan("softmax", "rows=4096,cols=1024")
    assert p.param_count == 14 and p.work == 33554432.0
    assert p.grid[0] * (p.block[0] // 32) >= 4096  # one pass, a warp per row
    assert p.grid[0] <= 148 * 4 and p.block[0] == 7 * 32  # 28 rows per SM as 4 blocks of 7 warps
    p = kh.plan("layernorm", "rows=4096,cols=1024")
    assert p.param_count == 24 and p.work == 33562624.0
    p = kh.plan("softmax", "rows=16384,cols=4096")
    assert p.block[0] == 256 and p.grid[0] == 148 * 8
    p = kh.plan("scan", "n=1000000")
    # 82 tiles of 12288 elements, a block per tile (fewer tiles than SMs), 13 warps, four tile buffers
    assert p.work == 8000000.0 and p.workspace_bytes == (4 + 2 * 82) * 8
    assert p.grid[0] == 82 and p.block[0] == 13 * 32 and p.dynamic_smem == 4 * 12288 * 4 + 1024
    assert p.param_count == 20
    assert kh.verify_launch("sm_100a", p.block[0], tuple(p.grid), 2048, p.dynamic_smem) == ""
    assert kh.plan("scan", "n=67108864").grid[0] == 148
    p = kh.plan("gemm", "m=8192,n=8192,k=8192")
    # split A, B prepared in one pass (sixteen-CTA clusters over 32-column strips), then 74 two-CTA clusters
    assert p.entry == b"gemm" and p.n_launches == 3 and p.grid[0] == 148 and p.block[0] == 320
    assert p.dynamic_smem == 6 * 32768 + 1024 and p.tmem_columns == 512
    assert p.workspace_bytes == 4 * 8192 * 8192 * 2 + 3 * 8192 * 4  # fp16 hi/lo of A and B^T, exponents, maxima
    assert p.work == 1099511627776.0 and p.work_is_flops
    assert kh.verify_launch("sm_100a", p.block[0], tuple(p.grid), 48, p.dynamic_smem) == ""
    p = kh.plan("gemm", "m=1000,n=1000,k=1000")
    # 16 tiles of 256 x 256 would use 16 of the 74 clusters; 32 tiles of 256 x 128 take half the time
    assert p.entry == b"gemm_n128" and p.grid[0] == 2 * 4 * 8
    # large products keep the wide tile: a narrow one costs 0.74 of it, more than the last wave it would fill
    assert kh.plan("gemm", "m=2048,n=8192,k=8192").entry == b"gemm"
    assert kh.plan("gemm", "m=4096,n=8192,k=8192").entry == b"gemm"
    assert kh.plan("gemm", "m=1024,n=8192,k=8192").entry == b"gemm"
    # rows of B that are not 16-byte multiples (or strips too tall for eight SMs) keep the two-pass form
    assert kh.plan("gemm", "m=129,n=257,k=33").n_launches == 4
    assert kh.plan("gemm", "m=64,n=64,k=32768").n_launches == 4
    assert kh.plan("gemm", "m=64,n=64,k=24576").n_launches == 3
    assert p.workspace_bytes == 4 * 1000 * 1024 * 2 + 3 * 4096
    p = kh.plan("attention", "batch=8,heads=16,seq=1024,head_dim=64")
    assert p.grid[0] == 148 and p.param_count == 52 and p.work == 34359738368.0
    assert kh.verify_launch("sm_100a", p.block[0], tuple(p.grid), 80, p.dynamic_smem) == ""


def test_embedded_code_objects_are_sm100_elf():
    for k in kh.KERNELS:
        image = kh.kernel_image(k)
        assert image[:4] == b"\x7fELF" and len(image) > 1000
        assert k.encode() in image  # the entry symbol equals the kernel name
    assert b"tcgen05" not in kh.kernel_image("vecadd")


def test_compute_calls_fail_loudly_without_a_device():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(kh.KernelhError) as e:
        kh.Context(0)
    assert e.value.code == kh.DRIVER_UNAVAILABLE
    assert "cuInit" in e.value.message or "dlopen" in e.value.message


def test_multi_gpu_entry_points_reject_bad_arguments_before_touching_a_device():
    """The sharded entry points validate their arguments on the host: a null
    context is a usage error (2) with a message, not a crash."""
    import ctypes as C

    lib = kh.lib
    reps = (C.c_void_p * 2)(0x1000, 0x2000)
    assert lib.kh_gemm_allgather(None, None, None, None, 2, 0, 256, 256, 64, None) == 2
    assert b"no C replicas" in lib.kh_last_error()
    assert lib.kh_gemm_allgather(None, None, None, reps, 2, 0, 256, 256, 64, None) == 2
    assert b"context" in lib.kh_last_error()
    assert lib.kh_gemm_allgather_multicast(None, None, None, None, None, 2, 0, 256, 256, 64, None) == 2
    assert lib.kh_gemm_allgather_multicast(None, None, None, 0x1000, 0x2000, 2, 0, 256, 256, 64, None) == 2
    assert b"context" in lib.kh_last_error()
    assert lib.kh_attention_allgather(None, None, None, None, reps, None, 2, 0, 4, 64, 64, None) == 2
    assert b"context" in lib.kh_last_error()


def test_kernels_without_a_scalar_path_refuse_misaligned_addresses_on_the_host():
    """attention and the fused all-gathers move 128-bit vectors only: an address
    that is not 16-byte aligned (a contiguous but offset view such as
    t.flatten()[1:]) is a usage error (2) raised before any launch, and the
    message names the buffer. No device is needed to find that out."""
    import ctypes as C

    lib = kh.lib
    ok, off = 0x7000000, 0x7000004
    for q, k, v, o, name in ((off, ok, ok, ok, b"'Q'"), (ok, off, ok, ok, b"'K'"), (ok, ok, off, ok, b"'V'"),
                             (ok, ok, ok, off, b"'O'")):
        assert lib.kh_attention(None, q, k, v, o, 1, 1, 64, 64, None) == 2
        assert b"16-byte aligned" in lib.kh_last_error() and name in lib.kh_last_error()
    assert lib.kh_attention(None, ok, ok, ok, ok, 1, 1, 64, 64, None) == 2
    assert b"context" in lib.kh_last_error()  # aligned: the next check is the context
    reps = (C.c_void_p * 2)(ok, off)
    assert lib.kh_gemm_allgather(None, ok, ok, reps, 2, 0, 256, 256, 64, None) == 2
    assert b"16-byte aligned" in lib.kh_last_error() and b"C replica" in lib.kh_last_error()
    assert lib.kh_gemm_allgather_multicast(None, ok, ok, ok, off, 2, 0, 256, 256, 64, None) == 2
    assert b"multicast" in lib.kh_last_error() and b"16-byte aligned" in lib.kh_last_error()
    assert lib.kh_attention_allgather(None, ok, ok, ok, reps, None, 2, 0, 4, 64, 64, None) == 2
    assert b"O replica" in lib.kh_last_error()
    good = (C.c_void_p * 2)(ok, ok + 64)
    assert lib.kh_attention_allgather(None, ok, off, ok, good, None, 2, 0, 4, 64, 64, None) == 2
    assert b"'K'" in lib.kh_last_error()
    assert lib.kh_attention_allgather(None, ok, ok, ok, good, off, 2, 0, 4, 64, 64, None) == 2
    assert b"multicast" in lib.kh_last_error()


def test_device_wait_codes_have_names():
    """kh_synchronize reports a device-side bounded wait that ran out as code 1001
    and names the wait; the code-to-name table is checked here without a GPU."""
    assert kh.DEVICE_TIMEOUT == 1001
    assert "arrival flag" in kh.wait_name(6)
    assert kh.wait_name(1) == "scan look-back wait"
    assert kh.wait_name(2) == "TMA (full-stage) wait"
    assert kh.wait_name(3) == "MMA (accumulator) wait"
    assert kh.wait_name(4) == "epilogue wait"
    assert kh.wait_name(5) == "empty-stage wait"
    assert kh.wait_name(0) == "ok" and kh.wait_name(77) == "unknown wait"
    # the probe validates its arguments on the host
    assert kh.lib.kh_scan_lookback_probe(None, 0x1000, 0x2000, 1 << 20, 1000, None) == 2
    assert b"context" in kh.lib.kh_last_error()


PTXAS_SAMPLE = """ptxas info    : 0 bytes gmem
ptxas info    : Compiling entry function 'alpha' for 'sm_100a'
ptxas info    : Function properties for alpha
    16 bytes stack frame, 8 bytes spill stores, 12 bytes spill loads
ptxas info    : Used 58 registers, used 1 barriers, 520 bytes cmem[0]
ptxas info    : Compile time = 4.530 ms
ptxas info    : Compiling entry function 'beta' for 'sm_100a'
ptxas info    : Function properties for beta
    0 bytes stack frame, 0 bytes spill stores, 0 bytes spill loads
ptxas info    : Used 168 registers, used 3 barriers, 2048 bytes smem
"""


def test_ptxas_report_parser():
    """resources.json is filled from `ptxas -v` text, as in the reference
    (lib/compiler/resource_reporter.cpp:614-660: "Used N registers", "M bytes smem")."""
    a = kh.parse_ptxas(PTXAS_SAMPLE, "alpha")
    assert a == {"registers": 58, "smem_bytes": 0, "stack_bytes": 16, "spill_store_bytes": 8,
                 "spill_load_bytes": 12, "barriers": 1}
    b = kh.parse_ptxas(PTXAS_SAMPLE, "beta")
    assert (b["registers"], b["smem_bytes"], b["barriers"], b["spill_store_bytes"]) == (168, 2048, 3, 0)
    assert kh.parse_ptxas(PTXAS_SAMPLE) == a  # no name: the first entry
    with pytest.raises(kh.KernelhError) as e:
        kh.parse_ptxas("nothing useful here", None)
    assert "unparseable ptxas output" in e.value.message
    # the reference's own sample of ptxas output, where its tree is present (REF as in oracle/Makefile)
    fixture = os.path.join(os.environ.get("REF", "/root/reference"), "test", "fixtures", "ptxas_gemm_v.txt")
    if os.path.exists(fixture):
        got = kh.parse_ptxas(open(fixture).read(), "gemm")
        assert (got["registers"], got["barriers"], got["smem_bytes"]) == (58, 1, 0)


def test_every_entry_point_has_resource_figures():
    entries = {"vecadd": ["vecadd"], "fused_gelu": ["fused_gelu", "fused_gelu_bias"], "scan": ["scan"],
               "softmax": ["softmax"], "layernorm": ["layernorm"],
               "gemm": ["gemm", "gemm_n128", "gemm_allgather", "gemm_allgather_n128", "gemm_split_a", "gemm_prep_b",
                        "gemm_colmax_b", "gemm_split_bt", "replicate_run"],
               "attention": ["attention", "attention_masked", "attention_allgather", "attention_split"]}
    for kernel, names in entries.items():
        for entry in names:
            fig, text = kh.kernel_resources(kernel, entry)
            assert 8 <= fig["registers"] <= 255, (kernel, entry, fig)
            assert f'"entry": "{entry}"' in text and '"target": "sm_100a"' in text
    assert kh.kernel_resources("gemm")[0]["registers"] >= 128          # the MMA kernel's epilogue holds a tile
    assert kh.kernel_resources("vecadd")[0]["spill_store_bytes"] == 0
    with pytest.raises(kh.KernelhError):
        kh.kernel_resources("gemm", "no_such_entry")
    js, md = kh.occupancy_report("scan", "n=67108864")
    assert '"kernel": "scan"' in js and '"threads_per_workgroup": 416' in js and "| scan |" in md


def test_registry_is_a_plug_in_point():
    """registerKernel(name, fn) adds a template or replaces an existing one
    (include/kernelh/dsl/program.hpp:64-67, lib/dsl/registry.cpp:39-42, pinned by
    test/unit/dsl_test.cpp:153-231): a custom template is added, listed in sorted order beside
    the built-ins, planned through the ordinary operator surface, may replace a built-in, and
    an unknown name lists it among the registered kernels. Here the registered value is a
    finished code object + entry + plan callback instead of an IR-emitting function."""
    image = kh.kernel_image("vecadd")  # any sm_100a code object will do for the host-side checks

    def plan_probe(shape, sm_count):
        if "n" not in shape:
            raise ValueError("shape attribute 'n' is required")
        if shape["n"] <= 0:
            raise ValueError("shape attribute 'n' must be positive")
        n = shape["n"]
        return {"grid": [min((n + 1023) // 1024, sm_count * 2)], "block": [256], "elements": [n, n, n], "outputs": [2],
                "work": 12.0 * n}

    kh.register_kernel("dsl_probe", image, "vecadd", plan_probe)
    try:
        names = kh.registered_kernels()
        assert names == sorted(names) and "dsl_probe" in names and "vecadd" in names
        p = kh.plan("dsl_probe", "n=4096", sm_count=148)
        assert (p.n_buffers, p.n_launches, p.entry, p.grid[0], p.block[0]) == (3, 1, b"vecadd", 4, 256)
        assert p.param_count == 15 and p.work == 12.0 * 4096 and not p.work_is_flops
        assert kh.kernel_image("dsl_probe") == image
        with pytest.raises(kh.KernelhError) as e:  # the callback's refusal comes back as a template error
            kh.plan("dsl_probe", "m=4")
        assert e.value.code == kh.USAGE_ERROR
        assert e.value.message == "dsl_probe template: shape attribute 'n' is required"
        with pytest.raises(kh.KernelhError) as e:
            kh.plan("nope", "n=4")
        assert "unknown kernel template 'nope'" in e.value.message and "dsl_probe" in e.value.message

        # replacing a built-in: the name now plans through the new record ...
        builtin = kh.plan("softmax", "rows=4096,cols=1024")
        kh.register_kernel("softmax", image, "vecadd",
                           lambda shape, sms: {"grid": [7], "block": [64], "elements": [shape["rows"] * shape["cols"]] * 3,
                                               "outputs": [2]})
        replaced = kh.plan("softmax", "rows=4096,cols=1024")
        assert (replaced.grid[0], replaced.block[0], replaced.n_buffers) == (7, 64, 3)
        assert kh.registered_kernels().count("softmax") == 1
        # ... and registering the same name again replaces the replacement
        kh.register_kernel("softmax", image, "vecadd",
                           lambda shape, sms: {"grid": [9], "block": [32], "elements": [4], "outputs": [0]})
        assert kh.plan("softmax", "rows=4,cols=1").grid[0] == 9
        kh.unregister_kernel("softmax")  # the built-in is back
        again = kh.plan("softmax", "rows=4096,cols=1024")
        assert (again.grid[0], again.block[0], again.n_buffers, again.entry) == (builtin.grid[0], builtin.block[0], 2, b"softmax")
    finally:
        kh.unregister_kernel("dsl_probe")
    assert "dsl_probe" not in kh.registered_kernels()
    with pytest.raises(kh.KernelhError):
        kh.unregister_kernel("dsl_probe")      # not registered any more
    with pytest.raises(kh.KernelhError):
        kh.unregister_kernel("vecadd")         # built-ins cannot be taken away
    assert kh.lib.kh_register_kernel(b"x", None, 0, b"e", kh.PLAN_FN(lambda *a: 0), None) == 2


def test_scan_totals_resolves_and_keeps_the_reference_shape_rules():
    p = kh.plan("scan_totals", "n=1000000")
    assert p.n_buffers == 7 and p.n_launches == 0  # the single-pass scan leaves nothing to launch
    with pytest.raises(kh.KernelhError) as e:
        kh.plan("scan_totals", "m=4")
    assert "scan_totals template: shape attribute 'n' is required" in e.value.message
    with pytest.raises(kh.KernelhError) as e:
        kh.plan("scan_totals", "n=0")
    assert "must be positive" in e.value.message


def test_extended_csv_appends_columns_after_the_reference_seven(golden):
    base = golden["host"]["csv"]["header"]
    assert kh.csv_header_ext() == base + ",gpus,roofline_frac,max_rel_err,cpu_ms,cpu_cores"
    row = golden["host"]["csv"]["lines"][0]
    ext = kh.csv_line_ext(*row["row"], gpus=8, roofline_frac=0.75, max_rel_err=2.5e-6, cpu_ms=12.5, cpu_cores=16)
    assert ext == row["line"] + ",8,0.75,2.5e-06,12.5,16"
    # not checked / not timed: empty fields, the first seven untouched
    assert kh.csv_line_ext(*row["row"]) == row["line"] + ",1,0,,,0"


def test_sharded_bench_row_refusals():
    """kh_bench_sharded partitions gemm and attention only (the other kernels are replicas),
    validates the GPU count before touching a device, and answers 77 without a driver."""
    with pytest.raises(kh.KernelhError) as e:
        kh.bench_sharded(2, "softmax", "rows=64,cols=64")
    assert e.value.code == 2 and "only gemm" in e.value.message and "replicas" in e.value.message
    with pytest.raises(kh.KernelhError) as e:
        kh.bench_sharded(9, "gemm", "m=512,n=256,k=64")
    assert e.value.code == 2 and "between 1 and 8" in e.value.message
    with pytest.raises(kh.KernelhError) as e:
        kh.bench_sharded(2, "gemm", "")
    assert e.value.code in (2, 77)


def test_attention_causal_shape_key():
    """`causal` is an optional 0/1 key of the attention template (not one of the reference's)."""
    p = kh.plan("attention", "batch=8,heads=16,seq=1024,head_dim=64,causal=1")
    assert p.entry == b"attention_masked" and p.work == 4.0 * 128 * (1024 * 1025 / 2) * 64
    assert kh.plan("attention", "batch=8,heads=16,seq=1024,head_dim=64,causal=0").work == 34359738368.0
    with pytest.raises(kh.KernelhError) as e:
        kh.plan("attention", "batch=8,heads=16,seq=1024,head_dim=64,causal=2")
    assert e.value.code == 2 and "'causal' must be 0 or 1" in e.value.message
