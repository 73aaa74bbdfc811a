"""Generates ``reference_vectors.json`` from the reference project's OWN code.

Run where the reference tree is mounted (``make -C oracle`` builds
``oracle/_ref/libkernelh_ref.so`` from the reference's sources)::

    python tests/golden/make_golden.py

Every entry records what the reference's input generators, fp64 references and
host-side helpers produce for a fixed case: a 64-bit FNV-1a hash of the raw
bytes, plus a few literal values so a mismatch is readable. The fixture travels
with the repository; the reference tree does not have to.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle_py as O  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.json")


def digest(arr: np.ndarray, nsample: int = 6) -> dict:
    flat = np.ascontiguousarray(arr).reshape(-1)
    idx = np.linspace(0, flat.size - 1, nsample).astype(np.int64)
    return {"fnv1a": f"{O.fnv1a(flat):016x}", "size": int(flat.size), "dtype": str(flat.dtype),
            "sample_index": idx.tolist(),
            "sample": [float.hex(float(flat[i])) for i in idx]}


def ref_lcg(fill, n, seed):
    v = np.empty(n, np.float32)
    s = C.c_uint(seed)
    fill(v, n, C.byref(s))
    return v, s.value


def main() -> None:
    if not O.ref_available():
        raise SystemExit("oracle/_ref/libkernelh_ref.so missing: run `make -C oracle` where the "
                         "reference tree is mounted")
    R = O.ref()
    G: dict = {"generators": {}, "references": {}, "host": {}}

    # ---- generators ----------------------------------------------------------------
    for n in (1024, 65536):
        a = np.empty(n, np.float32)
        b = np.empty(n, np.float32)
        R.khref_vecadd_fill(a, b, n)
        G["generators"][f"vecadd_pattern_n{n}"] = {"a": digest(a), "b": digest(b)}
    for (m, n, k) in ((128, 128, 128), (96, 160, 72)):
        a = np.empty((m, k), np.float32)
        b = np.empty((k, n), np.float32)
        R.khref_gemm_fill(a, b, m, n, k)
        G["generators"][f"gemm_pattern_{m}x{n}x{k}"] = {"a": digest(a), "b": digest(b)}
    for name, fill, seed in (("softmax", R.khref_softmax_fill, 0x27AB13),
                             ("layernorm", R.khref_layernorm_fill, 0x2E2E8A),
                             ("fused_gelu", R.khref_gelu_fill, 0x3A5F91)):
        v, s_after = ref_lcg(fill, 8192, seed)
        G["generators"][f"lcg_{name}_seed{seed:x}_n8192"] = {"v": digest(v), "seed_after": s_after}
    for seed in (0x313A171B, 0x51AC0D3E, 0x29C0FFEE):
        v = np.empty(4096, np.float32)
        R.khref_attention_fill(v, 4096, seed)
        G["generators"][f"lcg_attention_seed{seed:x}_n4096"] = {"v": digest(v)}
    for n, seed in ((1024, 0x29C0FFEE), (1000, 0x29C0FFEE), (1024, 0x51AC0D3E)):
        v = np.empty(n, np.float32)
        R.khref_scan_fill(v, n, seed)
        G["generators"][f"mt19937_scan_seed{seed:x}_n{n}"] = {"v": digest(v)}

    # ---- fp64 references -----------------------------------------------------------
    x, _ = ref_lcg(R.khref_softmax_fill, 16 * 1024, 0x27AB13)
    x = x.reshape(16, 1024)
    out = np.empty((16, 1024), np.float64)
    R.khref_softmax_ref(x, out, 16, 1024)
    G["references"]["softmax_16x1024_seed27ab13"] = digest(out)
    stab = np.tile(np.array([1000, -1000, 0, 0.5, -0.5], np.float32), 1024 * 4 // 5 + 1)[:4096]
    stab = np.ascontiguousarray(stab.reshape(4, 1024))
    out = np.empty((4, 1024), np.float64)
    R.khref_softmax_ref(stab, out, 4, 1024)
    G["references"]["softmax_stability_4x1024"] = digest(out)

    s = C.c_uint(0x2E2E8A)
    x = np.empty(16 * 1024, np.float32)
    g = np.empty(1024, np.float32)
    b = np.empty(1024, np.float32)
    R.khref_layernorm_fill(x, x.size, C.byref(s))
    R.khref_layernorm_fill(g, g.size, C.byref(s))
    R.khref_layernorm_fill(b, b.size, C.byref(s))
    out = np.empty((16, 1024), np.float64)
    R.khref_layernorm_ref(x, g, b, out, 16, 1024, 1e-5)
    G["references"]["layernorm_16x1024_seed2e2e8a"] = digest(out)
    const = np.full(2 * 1024, 3.0, np.float32)
    out2 = np.empty((2, 1024), np.float64)
    R.khref_layernorm_ref(const, g, b, out2, 2, 1024, 1e-5)
    G["references"]["layernorm_constant_rows_2x1024"] = digest(out2)

    x, _ = ref_lcg(R.khref_gelu_fill, 8192, 0x3A5F91)
    out = np.empty(8192, np.float64)
    R.khref_gelu_ref(x, out, 8192, 0)
    G["references"]["fused_gelu_n8192_seed3a5f91"] = digest(out)
    R.khref_gelu_ref(x, out, 8192, 1)
    G["references"]["fused_gelu_no_tanh_control_n8192"] = digest(out)

    seq, hd = 128, 64
    q = np.empty(seq * hd, np.float32)
    k = np.empty(seq * hd, np.float32)
    v = np.empty(seq * hd, np.float32)
    R.khref_attention_fill(q, q.size, 0x313A171B)
    R.khref_attention_fill(k, k.size, 0x51AC0D3E)
    R.khref_attention_fill(v, v.size, 0x29C0FFEE)
    out = np.empty(seq * hd, np.float64)
    R.khref_attention_ref(q, k, v, out, seq, hd, 1)
    G["references"]["attention_seq128_d64_scaled"] = digest(out)
    R.khref_attention_ref(q, k, v, out, seq, hd, 0)
    G["references"]["attention_seq128_d64_unscaled_control"] = digest(out)

    for (m, n, kk) in ((128, 128, 128), (96, 160, 72)):
        a = np.empty((m, kk), np.float32)
        b = np.empty((kk, n), np.float32)
        R.khref_gemm_fill(a, b, m, n, kk)
        c = np.empty((m, n), np.float32)
        R.khref_gemm_ref(a, b, c, m, n, kk)
        G["references"][f"gemm_{m}x{n}x{kk}_pattern"] = digest(c)
    c2 = c.copy()
    c2[3, 5] += 1.0
    G["references"]["gemm_rel_frobenius_one_off"] = float.hex(
        R.khref_gemm_rel_frobenius(c2, c, c.size))

    # ---- host-side helpers ---------------------------------------------------------
    def pack(ptrs, shapes):
        flat = [d for s_ in shapes for d in s_]
        ranks = [len(s_) for s_ in shapes]
        P = (C.c_ulonglong * len(ptrs))(*ptrs)
        S = (C.c_longlong * len(flat))(*flat)
        Rk = (C.c_int * len(ranks))(*ranks)
        slots = (C.c_ulonglong * 128)()
        n = R.khref_pack_memrefs(P, S, Rk, len(ptrs), slots, 128)
        return [int(slots[i]) for i in range(n)]

    G["host"]["descriptor_slots"] = [
        {"ptrs": [0x1000], "shapes": [[1024]], "slots": pack([0x1000], [[1024]])},
        {"ptrs": [0x1000, 0x2000], "shapes": [[4096, 1024], [4096, 1024]],
         "slots": pack([0x1000, 0x2000], [[4096, 1024], [4096, 1024]])},
        {"ptrs": [0xDEADBEEF00], "shapes": [[2, 8, 512, 64]],
         "slots": pack([0xDEADBEEF00], [[2, 8, 512, 64]])},
        {"ptrs": [0x10, 0x20, 0x30], "shapes": [[512, 256], [256, 128], [512, 128]],
         "slots": pack([0x10, 0x20, 0x30], [[512, 256], [256, 128], [512, 128]])},
    ]

    limits = {}
    for tok in ("gfx1101", "sm_80"):
        out10 = (C.c_longlong * 10)()
        name = C.create_string_buffer(256)
        msg = C.create_string_buffer(512)
        assert R.khref_device_limits(tok.encode(), out10, name, 256, msg, 512) == 0
        limits[tok] = {"fields": [int(x_) for x_ in out10], "name": name.value.decode()}
    msg = C.create_string_buffer(512)
    out10 = (C.c_longlong * 10)()
    assert R.khref_device_limits(b"sm_999", out10, None, 0, msg, 512) == 1
    limits["unknown_message_sm_999"] = msg.value.decode()
    G["host"]["device_limits"] = limits

    verifier = []
    for (tok, threads, gx, gy, gz, shared, wov) in (
            ("gfx1101", 256, 1, 1, 1, 70000, 0), ("gfx1101", 2048, 1, 1, 1, 0, 0),
            ("gfx1101", 100, 1, 1, 1, 0, 0), ("gfx1101", 256, 1, 1, 70000, 0, 0),
            ("gfx1101", 256, 1, 1, 1, 0, 4), ("gfx1101", 64, 1, 1, 1, 0, 4),
            ("gfx1101", 256, 40, 1, 1, 0, 0), ("gfx1101", 4100, 1, 1, 70000, 70000, 0),
            ("sm_80", 256, 1, 1, 1, 49153, 0), ("sm_80", 1024, 65535, 65535, 1, 49152, 0)):
        buf = C.create_string_buffer(4096)
        rc = R.khref_verify_launch(tok.encode(), threads, gx, gy, gz, shared, wov, buf, 4096)
        verifier.append({"target": tok, "threads": threads, "grid": [gx, gy, gz], "shared": shared,
                         "waves_per_cu_override": wov, "rc": rc, "message": buf.value.decode()})
    G["host"]["launch_verifier"] = verifier

    occ = []
    for (tok, vgpr, lds, threads) in (("gfx1101", 48, 8192, 512), ("gfx1101", 128, 8192, 128),
                                      ("sm_80", 20, 3072, 256), ("gfx1101", 64, 65536, 256),
                                      ("gfx1101", 0, 16384, 256), ("sm_80", 0, 0, 0),
                                      ("sm_80", 255, 49152, 1024)):
        o = (C.c_int * 5)()
        pct = R.khref_occupancy(tok.encode(), vgpr, lds, threads, o)
        occ.append({"target": tok, "vgpr": vgpr, "lds": lds, "threads": threads,
                    "out": [int(x_) for x_ in o], "pct": pct})
    G["host"]["occupancy"] = occ

    G["host"]["metrics"] = [
        {"what": w, "args": list(a_), "value": R.khref_metric(w.encode(), *a_)}
        for (w, a_) in (("gemm_flops", (512, 512, 512, 0)), ("gemm_bytes", (512, 512, 512, 0)),
                        ("gemm_flops", (8192, 8192, 8192, 0)),
                        ("elementwise_bytes", (4096, 1024, 0, 0)),
                        ("layernorm_bytes", (4096, 1024, 0, 0)), ("scan_bytes", (1000000, 0, 0, 0)),
                        ("fused_gelu_bytes", (4194304, 0, 0, 0)),
                        ("attention_flops", (2, 8, 512, 64)),
                        ("attention_flops", (8, 16, 1024, 64)))]
    G["host"]["rates"] = [
        {"gflops": g_, "work": w_, "ms": ms_, "value": R.khref_rate(g_, w_, ms_)}
        for (g_, w_, ms_) in ((1, 268435456.0, 1.028), (0, 33554432.0, 0.0468), (1, 1.0995e12, 6.5))]

    csv = []
    for row in (("gemm", "m=512,n=512,k=512", "kernelh", 1.028, 261.1234567891,
                 "2026-01-01T00:00:00Z", "NVIDIA B200"),
                ("soft\"max", "rows=1,cols=2", "a,b", 0.5, 1e-7, "t", "line\nbreak")):
        buf = C.create_string_buffer(1024)
        R.khref_csv_line(*[x_.encode() if isinstance(x_, str) else x_ for x_ in row], buf, 1024)
        csv.append({"row": list(row), "line": buf.value.decode()})
    buf = C.create_string_buffer(256)
    R.khref_csv_header(buf, 256)
    G["host"]["csv"] = {"header": buf.value.decode(), "lines": csv}

    shapes = []
    for text in ("m=512,n=512,k=512", "n=16", "rows=4096,cols=1024", "n=", "=4", "n=4x", "a=1,,b=2",
                 "batch=2,heads=8,seq=512,head_dim=64", "", "n=-3", "k=1,m=2,n=3", "n=1,n=2"):
        buf = C.create_string_buffer(512)
        R.khref_shape_roundtrip(text.encode(), buf, 512)
        shapes.append({"text": text, "roundtrip": buf.value.decode()})
    G["host"]["shape_text"] = shapes

    with open(OUT, "w") as f:
        json.dump(G, f, indent=1, sort_keys=True)
        f.write("\n")
    print(f"wrote {OUT} ({os.path.getsize(OUT)} bytes)")


if __name__ == "__main__":
    main()
