"""The CPU oracle against the fixtures generated from the reference's own code
(tests/golden/make_golden.py), and, when the checker library built from the
reference's sources is present, against that code directly on more cases."""
import ctypes as C

import numpy as np
import pytest


def check_digest(oracle, arr, d, exact=True, rtol=1e-13):
    flat = np.ascontiguousarray(arr).reshape(-1)
    assert flat.size == d["size"]
    assert str(flat.dtype) == d["dtype"]
    want = np.array([float.fromhex(s) for s in d["sample"]])
    got = flat[np.array(d["sample_index"])].astype(np.float64)
    if exact:
        assert f"{oracle.fnv1a(flat):016x}" == d["fnv1a"]
        assert np.array_equal(got, want)
    else:
        np.testing.assert_allclose(got, want, rtol=rtol, atol=0)


def test_generators_match_reference(oracle, golden):
    g = golden["generators"]
    for n in (1024, 65536):
        a, b = oracle.vecadd_pattern(n)
        check_digest(oracle, a, g[f"vecadd_pattern_n{n}"]["a"])
        check_digest(oracle, b, g[f"vecadd_pattern_n{n}"]["b"])
    for (m, n, k) in ((128, 128, 128), (96, 160, 72)):
        a, b = oracle.gemm_pattern(m, n, k)
        check_digest(oracle, a, g[f"gemm_pattern_{m}x{n}x{k}"]["a"])
        check_digest(oracle, b, g[f"gemm_pattern_{m}x{n}x{k}"]["b"])
    for name, seed in (("softmax", 0x27AB13), ("layernorm", 0x2E2E8A), ("fused_gelu", 0x3A5F91)):
        s = oracle.LcgStream(seed)
        v = s.fill(8192)
        e = g[f"lcg_{name}_seed{seed:x}_n8192"]
        check_digest(oracle, v, e["v"])
        assert s.seed.value == e["seed_after"]
    for seed in (0x313A171B, 0x51AC0D3E, 0x29C0FFEE):
        check_digest(oracle, oracle.lcg(4096, seed), g[f"lcg_attention_seed{seed:x}_n4096"]["v"])
    for n, seed in ((1024, 0x29C0FFEE), (1000, 0x29C0FFEE), (1024, 0x51AC0D3E)):
        check_digest(oracle, oracle.mt19937_unit(n, seed), g[f"mt19937_scan_seed{seed:x}_n{n}"]["v"])


def test_lcg_values_are_on_the_reference_grid(oracle):
    v = oracle.lcg(100000, 0x27AB13)
    assert v.min() >= -1.0 and v.max() < 1.0
    assert np.array_equal(v * 32768.0, np.round(v * 32768.0))


def test_references_match_reference(oracle, golden):
    r = golden["references"]
    x = oracle.lcg((16, 1024), 0x27AB13)
    check_digest(oracle, oracle.softmax_ref(x), r["softmax_16x1024_seed27ab13"])
    stab = np.tile(np.array([1000, -1000, 0, 0.5, -0.5], np.float32), 1024 * 4 // 5 + 1)[:4096]
    stab = np.ascontiguousarray(stab.reshape(4, 1024))
    out = oracle.softmax_ref(stab)
    assert np.isfinite(out).all()
    check_digest(oracle, out, r["softmax_stability_4x1024"])

    s = oracle.LcgStream(0x2E2E8A)
    x, g, b = s.fill((16, 1024)), s.fill(1024), s.fill(1024)
    check_digest(oracle, oracle.layernorm_ref(x, g, b), r["layernorm_16x1024_seed2e2e8a"])
    const = np.full((2, 1024), 3.0, np.float32)
    y = oracle.layernorm_ref(const, g, b)
    check_digest(oracle, y, r["layernorm_constant_rows_2x1024"])
    assert np.array_equal(y[0], b.astype(np.float64))  # variance-0 rows give exactly beta

    x = oracle.lcg(8192, 0x3A5F91)
    check_digest(oracle, oracle.fused_gelu_ref(x), r["fused_gelu_n8192_seed3a5f91"])
    check_digest(oracle, oracle.fused_gelu_ref(x, no_tanh_control=True),
                 r["fused_gelu_no_tanh_control_n8192"])

    q = oracle.lcg((1, 1, 128, 64), 0x313A171B)
    k = oracle.lcg((1, 1, 128, 64), 0x51AC0D3E)
    v = oracle.lcg((1, 1, 128, 64), 0x29C0FFEE)
    check_digest(oracle, oracle.attention_ref(q, k, v), r["attention_seq128_d64_scaled"])
    check_digest(oracle, oracle.attention_ref(q, k, v, scaled=False),
                 r["attention_seq128_d64_unscaled_control"])

    for (m, n, kk) in ((128, 128, 128), (96, 160, 72)):
        a, bm = oracle.gemm_pattern(m, n, kk)
        check_digest(oracle, oracle.gemm_ref(a, bm), r[f"gemm_{m}x{n}x{kk}_pattern"])
    c = oracle.gemm_ref(a, bm)
    c2 = c.copy()
    c2[3, 5] += 1.0
    assert oracle.compare(c2, c).rel_frobenius == pytest.approx(
        float.fromhex(r["gemm_rel_frobenius_one_off"]), rel=1e-12)


def test_negative_controls_have_teeth(oracle):
    """Each wrong reference the reference's tests use must disagree with the right one."""
    a, b = oracle.vecadd_pattern(1024)
    assert oracle.bit_mismatches(oracle.vecadd_ref(a, b), oracle.vecadd_ref(a, b, subtract=True)) == 1024
    a, b = oracle.gemm_pattern(256, 256, 256)
    assert oracle.compare(oracle.gemm_ref(a, b), oracle.gemm_ref(a, b, b_transposed=True)).rel_frobenius > 1e-5
    x = oracle.lcg((8, 1024), 0x27AB13)
    assert oracle.compare(oracle.softmax_ref(x).astype(np.float32),
                          oracle.softmax_ref(x, uniform_control=True)).max_abs > 1e-4
    x = oracle.mt19937_unit(1024, 0x51AC0D3E)
    assert oracle.compare(oracle.scan_ref(x), oracle.scan_ref(x, exclusive=True)).max_abs > 1e-4
    x = oracle.lcg(4096, 0x9C21A7)
    assert oracle.compare(oracle.fused_gelu_ref(x).astype(np.float32),
                          oracle.fused_gelu_ref(x, no_tanh_control=True)).max_abs > 1e-4
    const = np.full((2, 64), 3.0, np.float32)
    g = np.ones(64, np.float32)
    with np.errstate(all="ignore"):
        y = oracle.layernorm_ref(const, g, g, eps=0.0)
    assert np.isnan(y).all()  # 0 * inf: the eps=0 control


def test_scan_reference_is_exact(oracle):
    """Sums of < 2^20 fp32 values in [0,1) are exact in fp64, so the rounded
    prefix does not depend on association order."""
    x = oracle.mt19937_unit(1 << 16, 0x29C0FFEE)
    want = np.cumsum(x.astype(np.float64)).astype(np.float32)
    assert np.array_equal(oracle.scan_ref(x), want)
    assert oracle.scan_ref(x, exclusive=True)[0] == 0.0


def test_synthetic_generators(oracle):
    u = oracle.uniform(200000, oracle.BASE_SEED, -1.0, 1.0)
    assert u.min() >= -1.0 and u.max() < 1.0 and abs(u.mean()) < 0.01
    assert abs(u.std() - 2 / np.sqrt(12)) < 0.01
    n = oracle.normal(200001, oracle.BASE_SEED + 1, 0.0, 2.0)
    assert abs(n.mean()) < 0.02 and abs(n.std() - 2.0) < 0.02
    assert np.array_equal(u, oracle.uniform(200000, oracle.BASE_SEED, -1.0, 1.0))
    assert not np.array_equal(u, oracle.uniform(200000, oracle.BASE_SEED + 1, -1.0, 1.0))
    # known answer: first splitmix64/xoshiro256** draws for seed 0
    z = oracle.uniform(2, 0, 0.0, 1.0)
    assert 0.0 <= z[0] < 1.0 and z[0] != z[1]


def test_compare_metrics(oracle):
    ref = np.array([1.0, -2.0, 0.0, 4.0])
    got = np.array([1.0, -2.0, 0.0, 4.5], np.float32)
    c = oracle.compare(got, ref, rtol=0.1)
    assert c.max_abs == 0.5
    assert c.rel_frobenius == pytest.approx(0.5 / np.sqrt(21.0))
    assert c.max_violation == pytest.approx(0.5 - 0.4)
    assert c.max_rel_floored == pytest.approx(0.125)
    assert c.max_rel == pytest.approx(0.125)  # |ref| = 4 > rms
    assert c.non_finite == 0
    bad = got.copy()
    bad[1] = np.nan
    c = oracle.compare(bad, ref)
    assert np.isnan(c.max_abs) and c.non_finite == 1
    assert not (c.max_abs <= 1e-4)


def test_live_reference_cross_check(oracle):
    """More cases against the reference's own code when it was compiled here."""
    if not oracle.ref_available():
        pytest.skip("oracle/_ref not built (reference tree absent)")
    R = oracle.ref()
    rng = np.random.default_rng(7)
    x = rng.standard_normal((5, 333)).astype(np.float32) * 3
    out = np.empty((5, 333), np.float64)
    R.khref_softmax_ref(x, out, 5, 333)
    assert np.array_equal(out, oracle.softmax_ref(x))
    g = rng.random(333, dtype=np.float32) + 0.5
    b = rng.standard_normal(333).astype(np.float32)
    R.khref_layernorm_ref(x, g, b, out, 5, 333, 1e-5)
    assert np.array_equal(out, oracle.layernorm_ref(x, g, b))
    q, k, v = (rng.standard_normal((1, 1, 96, 64)).astype(np.float32) for _ in range(3))
    o = np.empty(96 * 64, np.float64)
    R.khref_attention_ref(q.reshape(-1), k.reshape(-1), v.reshape(-1), o, 96, 64, 1)
    assert np.array_equal(o.reshape(1, 1, 96, 64), oracle.attention_ref(q, k, v))
    a = rng.uniform(-1, 1, (70, 50)).astype(np.float32)
    bm = rng.uniform(-1, 1, (50, 90)).astype(np.float32)
    c = np.empty((70, 90), np.float32)
    R.khref_gemm_ref(a, bm, c, 70, 90, 50)
    assert np.array_equal(c, oracle.gemm_ref(a, bm))
    xs = rng.standard_normal(1000).astype(np.float32)
    o = np.empty(1000, np.float64)
    R.khref_gelu_ref(xs, o, 1000, 0)
    assert np.array_equal(o, oracle.fused_gelu_ref(xs))
