"""Parity of the sm_100a kernels with the fp64 CPU oracle, called through the C
ABI on a real B200. Inputs, references, tolerances and negative controls are
those of the reference's end-to-end tests (test/unit/e2e_*_test.cpp), followed
by the benchmark configurations' synthetic inputs with the stricter bounds
stated for them: vecadd bit-exact; max relative error (floored at 1e-3 * rms of
the reference) <= 1e-5 for the elementwise and row kernels and <= 1e-5 * sqrt(K)
for scan (K = n), gemm (K = k) and attention (K = seq)."""
import math
import re

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import kernelh_b200 as kh

pytestmark = pytest.mark.gpu

REL = 1e-5


@pytest.fixture(scope="module")
def ctx():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    torch.zeros(1, device="cuda")
    c = kh.Context(0)
    assert c.device_info().cc_major == 10
    yield c
    c.close()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run(ctx, kernel, shape, inputs, out_shape):
    """Launch through kh_launch on device tensors; returns the output as numpy."""
    out = torch.full(out_shape, float("nan"), dtype=torch.float32, device="cuda")
    bufs = [dev(x) if isinstance(x, np.ndarray) else x for x in inputs] + [out]
    ctx.launch(kernel, shape, bufs, torch.cuda.current_stream().cuda_stream)
    ctx.synchronize(torch.cuda.current_stream().cuda_stream)
    return out.cpu().numpy()


# --------------------------------------------------------------------------- vecadd
@pytest.mark.parametrize("n", [1024, 65536, 1 << 20, 1, 3, 1025, 4097, 1000003])
def test_vecadd_reference_pattern_bit_exact(ctx, oracle, n):
    a, b = oracle.vecadd_pattern(n)
    c = run(ctx, "vecadd", f"n={n}", [a, b], (n,))
    ref = oracle.vecadd_ref(a, b)
    assert oracle.compare(c, ref).max_abs <= 1e-6  # the reference's bound
    assert oracle.bit_mismatches(c, ref) == 0      # the bound asked of this build
    # negative control: a - b must disagree everywhere
    assert oracle.bit_mismatches(c, oracle.vecadd_ref(a, b, subtract=True)) == n


def test_vecadd_benchmark_config_bit_exact(ctx, oracle):
    n = 1 << 24
    a = oracle.uniform(n, oracle.BASE_SEED, -1, 1)
    b = oracle.uniform(n, oracle.BASE_SEED + 1, -1, 1)
    c = run(ctx, "vecadd", f"n={n}", [a, b], (n,))
    assert oracle.bit_mismatches(c, oracle.vecadd_ref(a, b)) == 0


def test_vecadd_misaligned_pointers_and_typed_entry(ctx, oracle):
    n = 10007
    a, b = oracle.vecadd_pattern(n + 1)
    da, db = dev(a), dev(b)
    out = torch.zeros(n + 1, device="cuda")
    ctx.vecadd(da[1:], db[1:], out[1:], n, torch.cuda.current_stream().cuda_stream)
    ctx.synchronize()
    assert oracle.bit_mismatches(out[1:].cpu().numpy(), oracle.vecadd_ref(a[1:].copy(), b[1:].copy())) == 0
    assert out[0].item() == 0.0


def test_run_host_path(ctx, oracle):
    n = 100000
    a, b = oracle.vecadd_pattern(n)
    c = np.zeros(n, np.float32)
    ctx.run_host("vecadd", f"n={n}", [a, b, c])
    assert oracle.bit_mismatches(c, oracle.vecadd_ref(a, b)) == 0


# --------------------------------------------------------------------------- fused_gelu
@pytest.mark.parametrize("n", [4194304, 1048576, 1000, 7])
def test_fused_gelu_reference_inputs(ctx, oracle, n):
    x = oracle.lcg(n, 0x3A5F91)
    y = run(ctx, "fused_gelu", f"n={n}", [x, None], (n,))
    cmp_ = oracle.compare(y, oracle.fused_gelu_ref(x))
    assert cmp_.non_finite == 0 and cmp_.max_abs <= 1e-4  # the reference's bound
    assert cmp_.max_rel <= REL
    xs = oracle.lcg(n, 0x9C21A7)
    ys = run(ctx, "fused_gelu", f"n={n}", [xs, None], (n,))
    if n >= 1000:  # negative control: GELU without tanh must fail the same check
        assert oracle.compare(ys, oracle.fused_gelu_ref(xs, no_tanh_control=True)).max_abs > 1e-4


def test_fused_gelu_rows_cols_shape_and_bias_form(ctx, oracle):
    x = oracle.lcg(64 * 96, 0x3A5F91)
    y = run(ctx, "fused_gelu", "rows=64,cols=96", [x, None], (64 * 96,))
    assert oracle.compare(y, oracle.fused_gelu_ref(x)).max_rel <= REL
    n = 1 << 22
    x = oracle.normal(n, oracle.BASE_SEED, 0, 1)
    bias = oracle.normal(n, oracle.BASE_SEED + 1, 0, 1)
    y = run(ctx, "fused_gelu", f"n={n},bias=1", [x, bias], (n,))
    cmp_ = oracle.compare(y, oracle.bias_gelu_ref(x, bias))
    assert cmp_.non_finite == 0 and cmp_.max_rel <= REL and cmp_.max_abs <= 1e-4
    wide = oracle.normal(4096, 5, 0, 30)  # saturating arguments stay finite
    y = run(ctx, "fused_gelu", "n=4096,bias=1", [wide, np.zeros(4096, np.float32)], (4096,))
    assert oracle.compare(y, oracle.bias_gelu_ref(wide, np.zeros(4096, np.float32))).max_rel <= REL


# --------------------------------------------------------------------------- softmax
@pytest.mark.parametrize("rows,cols", [(4096, 1024), (16384, 4096), (1, 8192), (37, 1000), (5, 333),
                                       (3, 10000), (2, 4), (9, 12288)])
def test_softmax_reference_inputs(ctx, oracle, rows, cols):
    x = oracle.lcg((rows, cols), 0x27AB13)
    y = run(ctx, "softmax", f"rows={rows},cols={cols}", [x], (rows, cols))
    ref = oracle.softmax_ref(x)
    cmp_ = oracle.compare(y, ref)
    assert cmp_.non_finite == 0 and cmp_.max_abs <= 1e-4
    assert cmp_.max_rel <= REL
    np.testing.assert_allclose(y.sum(axis=1), 1.0, atol=1e-5)
    assert oracle.compare(y, oracle.softmax_ref(x, uniform_control=True)).max_abs > (1e-4 if cols <= 4096 else 0)


def test_softmax_stability_rows(ctx, oracle):
    pat = np.array([1000, -1000, 0, 0.5, -0.5], np.float32)
    x = np.ascontiguousarray(np.tile(pat, 1024 * 1024 // 5 + 1)[:1024 * 1024].reshape(1024, 1024))
    y = run(ctx, "softmax", "rows=1024,cols=1024", [x], (1024, 1024))
    cmp_ = oracle.compare(y, oracle.softmax_ref(x))
    assert cmp_.non_finite == 0 and cmp_.max_abs <= 1e-4


def test_softmax_benchmark_config(ctx, oracle):
    x = oracle.normal((4096, 1024), oracle.BASE_SEED, 0, 2.0)  # N(0, 4) read as variance 4
    y = run(ctx, "softmax", "rows=4096,cols=1024", [x], (4096, 1024))
    cmp_ = oracle.compare(y, oracle.softmax_ref(x))
    assert cmp_.non_finite == 0 and cmp_.max_rel <= REL


# --------------------------------------------------------------------------- layernorm
@pytest.mark.parametrize("rows,cols", [(4096, 1024), (16384, 4096), (37, 1000), (5, 333), (3, 10000),
                                       (2, 4)])
def test_layernorm_reference_inputs(ctx, oracle, rows, cols):
    s = oracle.LcgStream(0x2E2E8A)
    x, g, b = s.fill((rows, cols)), s.fill(cols), s.fill(cols)
    y = run(ctx, "layernorm", f"rows={rows},cols={cols}", [x, g, b], (rows, cols))
    cmp_ = oracle.compare(y, oracle.layernorm_ref(x, g, b))
    assert cmp_.non_finite == 0 and cmp_.max_abs <= 1e-4
    assert cmp_.max_rel <= REL


def test_layernorm_constant_rows_give_beta(ctx, oracle):
    s = oracle.LcgStream(0xC0578A)
    g, b = s.fill(1024), s.fill(1024)
    x = np.full((64, 1024), 3.0, np.float32)
    y = run(ctx, "layernorm", "rows=64,cols=1024", [x, g, b], (64, 1024))
    assert np.isfinite(y).all()
    assert oracle.compare(y, oracle.layernorm_ref(x, g, b)).max_abs <= 1e-4
    assert np.array_equal(y[0], b)
    with np.errstate(all="ignore"):  # negative control: eps = 0 turns these rows into NaN
        assert not (oracle.compare(y, oracle.layernorm_ref(x, g, b, eps=0.0)).max_abs <= 1e-4)


def test_layernorm_benchmark_config(ctx, oracle):
    x = oracle.normal((4096, 1024), oracle.BASE_SEED, 0, 1)
    g = oracle.uniform(1024, oracle.BASE_SEED + 1, 0.5, 1.5)
    b = oracle.normal(1024, oracle.BASE_SEED + 2, 0, 0.1)  # N(0, 0.1) read as sigma 0.1
    y = run(ctx, "layernorm", "rows=4096,cols=1024", [x, g, b], (4096, 1024))
    cmp_ = oracle.compare(y, oracle.layernorm_ref(x, g, b))
    assert cmp_.non_finite == 0 and cmp_.max_rel <= REL


# --------------------------------------------------------------------------- scan
@pytest.mark.parametrize("n,atol", [(1024, 1e-4), (65536, 1e-3), (1 << 20, 5e-3), (1000, 1e-4),
                                    (1, 1e-4), (4096, 1e-4), (4097, 1e-4)])
def test_scan_reference_inputs(ctx, oracle, n, atol):
    x = oracle.mt19937_unit(n, 0x29C0FFEE)
    y = run(ctx, "scan", f"n={n}", [x], (n,))
    ref = oracle.scan_ref(x)
    assert oracle.compare(y, ref).max_abs <= atol  # the reference's per-size bound
    assert oracle.bit_mismatches(y, ref) == 0      # exact sums: every association order agrees
    if n >= 1024:
        xc = oracle.mt19937_unit(1024, 0x51AC0D3E)
        yc = run(ctx, "scan", "n=1024", [xc], (1024,))
        assert oracle.compare(yc, oracle.scan_ref(xc, exclusive=True)).max_abs > 1e-4


def test_scan_benchmark_config_and_repeated_launches(ctx, oracle):
    n = 1000000
    x = oracle.uniform(n, oracle.BASE_SEED, 0, 1)
    ref = oracle.scan_ref(x)
    for _ in range(4):  # the look-back state is reused across launches (epochs)
        y = run(ctx, "scan", f"n={n}", [x], (n,))
        cmp_ = oracle.compare(y, ref)
        assert cmp_.max_rel <= REL * math.sqrt(n)
        assert oracle.bit_mismatches(y, ref) == 0
    assert np.all(np.diff(y.astype(np.float64)) >= 0)  # non-negative input: non-decreasing


def test_scan_large_and_signed(ctx, oracle):
    n = (1 << 24) + 5
    x = oracle.uniform(n, 99, -1, 1)
    y = run(ctx, "scan", f"n={n}", [x], (n,))
    ref = oracle.scan_ref(x)
    assert oracle.compare(y, ref).max_abs <= 1e-3
    assert oracle.bit_mismatches(y, ref) <= n // 1000  # fp64 sums of general data: last-bit ties only


def test_scan_misaligned_strided_and_ragged_sizes(ctx, oracle):
    """Buffers the tensor-map copies cannot take (not 16-byte aligned) go through the plain
    load / store path of the same kernel, sizes that end inside a 32-element row use the
    partial-row code, and sizes around the 12288-element tile and the 1024-element warp part
    cross every boundary of the pipeline; all must give the oracle's bits."""
    for n in (31, 32, 33, 1023, 1025, 12287, 12288, 12289, 24576 + 17, 36864, 49152 + 1, 200000, 12288 * 148 + 5):
        x = oracle.mt19937_unit(n, 0x29C0FFEE + n)
        ref = oracle.scan_ref(x)
        assert oracle.bit_mismatches(run(ctx, "scan", f"n={n}", [x], (n,)), ref) == 0, n
    n = 100003
    x = oracle.mt19937_unit(n + 1, 0x51AC0D3E)
    dx, out = dev(x), torch.full((n + 2,), float("nan"), device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    ctx.scan(dx[1:], out[1:], n, stream)  # both sides misaligned
    ctx.synchronize(stream)
    ref = oracle.scan_ref(x[1:].copy())
    assert oracle.bit_mismatches(out[1:n + 1].cpu().numpy(), ref) == 0
    assert torch.isnan(out[0]).item() and torch.isnan(out[n + 1]).item()
    out.fill_(float("nan"))
    ctx.scan(dx[1:], out, n, stream)      # input misaligned, output through the tensor map
    ctx.synchronize(stream)
    assert oracle.bit_mismatches(out[:n].cpu().numpy(), ref) == 0 and torch.isnan(out[n]).item()


def test_scan_lookback_that_runs_out_is_reported_and_survivable(ctx, oracle):
    """A bounded device-side wait that gives up, shown without any fault: the scan is
    launched so that tile 0 is never produced (every ticket shifted by one), the look-back
    of tile 1 polls its missing predecessor a few thousand times (about a millisecond),
    records the scan look-back code in the status word, every role of the kernel stops and
    the kernel returns. kh_synchronize then reports 1001 and names the wait, and the next
    ordinary scan on the same context gives the oracle's bits."""
    n = 3 * 12288 + 100
    x = oracle.mt19937_unit(n, 0x29C0FFEE)
    dx, dy = dev(x), torch.zeros(n, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    ctx.scan_lookback_probe(dx, dy, n, 3000, stream)
    with pytest.raises(kh.KernelhError) as e:
        ctx.synchronize(stream)
    assert e.value.code == kh.DEVICE_TIMEOUT == 1001
    # detail = the tile whose look-back gave up first (whichever of the shifted tickets 1..4 that was)
    assert "scan look-back wait" in e.value.message and re.search(r"code 1, detail [1-4]\b", e.value.message)
    assert "output is incomplete" in e.value.message
    ctx.synchronize(stream)  # the status was cleared: a second wait is clean
    for _ in range(2):
        y = run(ctx, "scan", f"n={n}", [x], (n,))
        assert oracle.bit_mismatches(y, oracle.scan_ref(x)) == 0
    with pytest.raises(kh.KernelhError) as e:  # argument checks happen on the host
        ctx.scan_lookback_probe(dx, dy, 1000, 3000, stream)
    assert e.value.code == kh.USAGE_ERROR and "two tiles" in e.value.message
    with pytest.raises(kh.KernelhError):
        ctx.scan_lookback_probe(dx, dy, n, 0, stream)


# --------------------------------------------------------------------------- gemm
@pytest.mark.parametrize("size", [128, 512, 1024, 1000, 2048])
def test_gemm_reference_pattern(ctx, oracle, size):
    a, b = oracle.gemm_pattern(size, size, size)
    c = run(ctx, "gemm", f"m={size},n={size},k={size}", [a, b], (size, size))
    ref = oracle.gemm_ref(a, b)
    assert oracle.compare(c, ref).rel_frobenius <= 1e-5  # the reference's bound
    assert oracle.bit_mismatches(c, ref) == 0            # exact integers survive the scaled fp16 hi/lo split


def test_gemm_negative_control(ctx, oracle):
    a, b = oracle.gemm_pattern(256, 256, 256)
    c = run(ctx, "gemm", "m=256,n=256,k=256", [a, b], (256, 256))
    assert oracle.compare(c, oracle.gemm_ref(a, b)).rel_frobenius <= 1e-5
    assert oracle.compare(c, oracle.gemm_ref(a, b, b_transposed=True)).rel_frobenius > 1e-5


@pytest.mark.parametrize("m,n,k", [(512, 512, 512), (100, 200, 72), (129, 257, 33), (1, 1, 1),
                                   (300, 40, 1000), (1024, 768, 4096)])
def test_gemm_uniform_inputs_keep_fp32_accuracy(ctx, oracle, m, n, k):
    a = oracle.uniform((m, k), oracle.BASE_SEED, -1, 1)
    b = oracle.uniform((k, n), oracle.BASE_SEED + 1, -1, 1)
    c = run(ctx, "gemm", f"m={m},n={n},k={k}", [a, b], (m, n))
    cmp_ = oracle.compare(c, oracle.gemm_ref(a, b))
    assert cmp_.non_finite == 0
    assert cmp_.rel_frobenius <= 1e-5
    assert cmp_.max_rel <= REL * math.sqrt(k)


@pytest.mark.parametrize("kind", ["rows_and_columns", "inside_rows", "tiny_times_huge"])
def test_gemm_is_insensitive_to_operand_scaling(ctx, oracle, kind):
    """The fp16 splits see every row of A and column of B scaled into one fixed
    range, so magnitudes from 1e-38 to 1e+15 must not cost accuracy: the error
    stays a small multiple of fp32 epsilon of (|A| |B|) element by element."""
    m, n, k = 512, 768, 1000
    a = oracle.normal((m, k), oracle.BASE_SEED + 7, 0, 1)
    b = oracle.normal((k, n), oracle.BASE_SEED + 8, 0, 1)
    rng = np.random.default_rng(5)
    if kind == "rows_and_columns":
        a *= (10.0 ** rng.integers(-15, 16, (m, 1))).astype(np.float32)
        b *= (10.0 ** rng.integers(-15, 16, (1, n))).astype(np.float32)
        a[3] = 0
        b[:, 5] = 0
    elif kind == "inside_rows":
        a *= (2.0 ** rng.integers(-30, 1, (m, k))).astype(np.float32)
        b *= (2.0 ** rng.integers(-30, 1, (k, n))).astype(np.float32)
    else:
        a *= np.float32(1e-38)
        b *= np.float32(1e30)
    c = run(ctx, "gemm", f"m={m},n={n},k={k}", [a, b], (m, n)).astype(np.float64)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    bound = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
    assert np.all(np.isfinite(c))
    assert np.max(np.abs(c - ref) / np.maximum(bound, 1e-300)) <= 4e-6
    if kind == "rows_and_columns":
        assert not c[3].any() and not c[:, 5].any()


def test_gemm_reference_pattern_4096(ctx, oracle):
    """The largest size of the reference's pattern list (test/unit/e2e_gemm_test.cpp:277),
    checked bit for bit on sampled rows (the fp64 routine over all of C would take minutes)."""
    size = 4096
    a, b = oracle.gemm_pattern(size, size, size)
    c = run(ctx, "gemm", f"m={size},n={size},k={size}", [a, b], (size, size))
    rows = np.sort(np.random.default_rng(2).choice(size, 96, replace=False))
    ref = oracle.gemm_ref_pick_rows(a, b, rows)
    assert oracle.compare(c[rows], ref).rel_frobenius <= 1e-5
    assert oracle.bit_mismatches(np.ascontiguousarray(c[rows]), ref) == 0
    assert np.isfinite(c).all()


def test_gemm_propagates_inf_and_nan_like_fp32(ctx, oracle):
    """The scaled fp16 hi/lo split must not turn one non-finite input into a
    non-finite C anywhere an fp32 product would be finite, and must keep C
    non-finite wherever fp32 gives Inf or NaN (Inf and NaN are not told apart:
    the split of Inf has a NaN low part)."""
    m, n, k = 300, 520, 264
    a = oracle.normal((m, k), oracle.BASE_SEED + 21, 0, 1)
    b = oracle.normal((k, n), oracle.BASE_SEED + 22, 0, 1)
    a[7, 100] = np.inf        # row 7 of C: +-Inf everywhere (NaN where B[100, c] == 0)
    a[130, 5] = np.nan        # row 130 of C: NaN
    b[17, 260] = -np.inf      # column 260 of C: non-finite
    b[200, 3] = np.nan        # column 3 of C: NaN
    b[:, 400] = 0             # a zero column: Inf * 0 = NaN in row 7, exact zeros elsewhere
    c = run(ctx, "gemm", f"m={m},n={n},k={k}", [a, b], (m, n))
    with np.errstate(all="ignore"):
        ref32 = a.astype(np.float64) @ b.astype(np.float64)
    expect_bad = ~np.isfinite(ref32)
    assert expect_bad[7].all() and expect_bad[130].all() and expect_bad[:, 260].all() and expect_bad[:, 3].all()
    assert expect_bad.sum() == 2 * n + 2 * m - 4
    assert np.array_equal(~np.isfinite(c), expect_bad)
    assert np.isnan(c[7, 400]) and np.isnan(c[130]).all() and np.isnan(c[:, 3]).all()
    good = ~expect_bad
    bound = np.abs(np.nan_to_num(a, nan=0, posinf=0, neginf=0)).astype(np.float64) @ \
        np.abs(np.nan_to_num(b, nan=0, posinf=0, neginf=0)).astype(np.float64)
    assert np.max(np.abs(c.astype(np.float64) - ref32)[good] / np.maximum(bound[good], 1e-300)) <= 4e-6
    assert not c[np.arange(m) != 7][:, 400][np.arange(m - 1) != 129].any()  # zero column stays exactly zero


def test_gemm_subnormal_rows_and_columns(ctx, oracle):
    """Rows of A (columns of B) that hold only subnormal fp32 values are scaled up
    exactly before the split, so they keep their significant bits; the product is
    compared with fp64 to a few fp32 roundings of |A||B| plus one subnormal step
    (the final power-of-two un-scaling rounds once into the subnormal range)."""
    m, n, k = 256, 384, 200
    a = oracle.uniform((m, k), oracle.BASE_SEED + 31, -1, 1)
    b = oracle.uniform((k, n), oracle.BASE_SEED + 32, -1, 1)
    a[10] *= np.float32(1e-39)            # subnormal-only row
    a[11] = a[11] * np.float32(1e-30)
    a[11] = a[11] * np.float32(1e-9)      # 1e-39 again, reached in two steps
    b[:, 20] *= np.float32(3e-40)         # subnormal-only column
    assert np.all(np.abs(a[10]) < 1.1754944e-38) and np.all(np.abs(b[:, 20]) < 1.1754944e-38)
    c = run(ctx, "gemm", f"m={m},n={n},k={k}", [a, b], (m, n)).astype(np.float64)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    bound = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
    assert np.all(np.isfinite(c))
    assert np.all(np.abs(c - ref) <= 4e-6 * bound + 1.5e-45)
    assert np.count_nonzero(c[10]) > n // 2      # the subnormal row was not flushed to zero
    assert np.count_nonzero(c[:, 20]) > m // 2


@pytest.mark.parametrize("m,n,k", [(2500, 384, 200), (256, 256, 64), (100, 40, 33), (8192, 256, 64)])
def test_gemm_host_path_is_pipelined_and_identical(ctx, oracle, m, n, k):
    """kh_run_host for gemm uploads A in row blocks and multiplies them while the
    next block is on the wire; the result equals the device path bit for bit. m = 8192 has the
    benchmark's block list: 1024-row blocks with the first and the last cut into 256, 256 and 512 rows."""
    a = oracle.uniform((m, k), oracle.BASE_SEED + 11, -1, 1)
    b = oracle.uniform((k, n), oracle.BASE_SEED + 12, -1, 1)
    c_dev = run(ctx, "gemm", f"m={m},n={n},k={k}", [a, b], (m, n))
    c_host = np.full((m, n), np.nan, np.float32)
    ctx.run_host("gemm", f"m={m},n={n},k={k}", [a, b, c_host])
    assert np.array_equal(c_host, c_dev)
    assert oracle.compare(c_host, oracle.gemm_ref(a, b)).rel_frobenius <= 1e-5


def test_gemm_8192_sampled_rows_and_scaling_property(ctx, oracle):
    size = 8192
    a = oracle.uniform((size, size), oracle.BASE_SEED, -1, 1)
    b = oracle.uniform((size, size), oracle.BASE_SEED + 1, -1, 1)
    da, db = dev(a), dev(b)
    c = run(ctx, "gemm", f"m={size},n={size},k={size}", [da, db], (size, size))
    rows = np.sort(np.random.default_rng(1).choice(size, 48, replace=False))
    ref = oracle.gemm_ref_pick_rows(a, b, rows)
    cmp_ = oracle.compare(c[rows], ref)
    assert cmp_.rel_frobenius <= 1e-5
    assert cmp_.max_rel <= REL * math.sqrt(size)
    # scaling A by a power of two scales every hi/lo part exactly: C doubles bit for bit
    c2 = run(ctx, "gemm", f"m={size},n={size},k={size}", [da * 2, db], (size, size))
    assert np.array_equal(c2, c * 2)


def test_gemm_last_wave_split_over_k(ctx, oracle):
    """80 tiles on 74 clusters: the six tiles of the last wave are each done by two clusters,
    half of K each, which meet through a scratch of partial sums. Same bound against fp64 as any
    gemm; the rows of the split tiles are the last ones in rasterised order, so all of C is
    compared. Three times in a row (the meeting flags start from zero again), then through the fused
    all-gather with two ranks played one after the other, where the split tiles are also pushed."""
    m, n, k = 2560, 2048, 512
    a = oracle.uniform((m, k), oracle.BASE_SEED + 81, -1, 1)
    b = oracle.uniform((k, n), oracle.BASE_SEED + 82, -1, 1)
    ref = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
    da, db = dev(a), dev(b)
    runs = []
    for _ in range(3):
        c = run(ctx, "gemm", f"m={m},n={n},k={k}", [da, db], (m, n))
        cmp_ = oracle.compare(c, ref)
        assert cmp_.non_finite == 0 and cmp_.max_rel <= REL * math.sqrt(k) and cmp_.rel_frobenius <= 1e-5
        runs.append(c)
    # whichever unit comes last adds the same two numbers: the bits do not depend on timing
    assert np.array_equal(runs[0], runs[1]) and np.array_equal(runs[0], runs[2])
    replicas = [torch.full((2 * m, n), float("nan"), device="cuda") for _ in range(2)]
    stream = torch.cuda.current_stream().cuda_stream
    a2 = np.concatenate([a, a[::-1]])
    da2 = dev(a2)
    for rank in range(2):
        ctx.gemm_allgather(da2[rank * m:(rank + 1) * m], db, replicas, rank, m, n, k, stream)
    ctx.synchronize(stream)
    ref2 = np.concatenate([ref, ref[::-1]])
    for r in replicas:
        cmp_ = oracle.compare(r.cpu().numpy(), ref2)
        assert cmp_.non_finite == 0 and cmp_.max_rel <= REL * math.sqrt(k)
    assert torch.equal(replicas[0], replicas[1])


def test_gemm_allgather_short_shard_splits_its_first_tiles_too(ctx, oracle, monkeypatch):
    """A shard of 128 tiles (1024 x 8192, what a rank has at 8 GPUs) in the fused all-gather: the
    first 37 tiles AND the 17 of the last wave are each done by two clusters over half of K, so
    that the first pushes leave after half a tile's time. Two ranks played one after the other;
    every element of both replicas against fp64."""
    m, n, k = 1024, 8192, 512
    monkeypatch.setenv("KERNELH_GEMM_SPLIT_HEAD", "1")  # two ranks would not be bound by NVLink ingress: ask for it
    a = oracle.uniform((2 * m, k), oracle.BASE_SEED + 91, -1, 1)
    b = oracle.uniform((k, n), oracle.BASE_SEED + 92, -1, 1)
    ref = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
    da, db = dev(a), dev(b)
    replicas = [torch.full((2 * m, n), float("nan"), device="cuda") for _ in range(2)]
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        for rank in range(2):
            ctx.gemm_allgather(da[rank * m:(rank + 1) * m], db, replicas, rank, m, n, k, stream)
        ctx.synchronize(stream)
        for r in replicas:
            cmp_ = oracle.compare(r.cpu().numpy(), ref)
            assert cmp_.non_finite == 0 and cmp_.max_rel <= REL * math.sqrt(k) and cmp_.rel_frobenius <= 1e-5
        assert torch.equal(replicas[0], replicas[1])
        for r in replicas:
            r.fill_(float("nan"))


def test_gemm_scaled_store_alpha_beta(ctx, oracle):
    """C = alpha * A.B + beta * C (the first generalisation of the reference's plain store,
    lib/dsl/kernels/gemm.cpp:47-53): alpha = 1, beta = 0 is the plain gemm bit for bit and never
    reads C (NaN in, numbers out); general alpha, beta meet the gemm's bound against fp64, on an
    aligned shape, a ragged one (scalar store path) and a small one (narrow tiles)."""
    for (m, n, k) in [(512, 768, 320), (300, 250, 100), (1000, 1000, 64)]:
        a = oracle.uniform((m, k), oracle.BASE_SEED + 71, -1, 1)
        b = oracle.uniform((k, n), oracle.BASE_SEED + 72, -1, 1)
        c0 = oracle.uniform((m, n), oracle.BASE_SEED + 73, -4, 4)
        da, db = dev(a), dev(b)
        stream = torch.cuda.current_stream().cuda_stream
        plain = run(ctx, "gemm", f"m={m},n={n},k={k}", [da, db], (m, n))
        c = torch.full((m, n), float("nan"), device="cuda")
        ctx.gemm_scaled(da, db, c, m, n, k, 1.0, 0.0, stream)
        ctx.synchronize(stream)
        assert np.array_equal(c.cpu().numpy(), plain)
        for alpha, beta in [(2.5, 0.0), (1.0, 1.0), (-0.75, 0.5)]:
            c = dev(c0)
            ctx.gemm_scaled(da, db, c, m, n, k, alpha, beta, stream)
            ctx.synchronize(stream)
            ref = alpha * (a.astype(np.float64) @ b.astype(np.float64)) + beta * c0.astype(np.float64)
            cmp_ = oracle.compare(c.cpu().numpy(), ref.astype(np.float32))
            assert cmp_.non_finite == 0 and cmp_.max_rel <= REL * math.sqrt(k), (m, n, k, alpha, beta, cmp_.max_rel)


def test_gemm_allgather_two_shards_fill_every_replica(ctx, oracle):
    """The fused gemm + all-gather on one GPU: the two ranks' launches run one
    after the other and each stores its row shard into both replicas of C."""
    m, n, k = 512, 768, 320
    a = oracle.uniform((m, k), oracle.BASE_SEED, -1, 1)
    b = oracle.uniform((k, n), oracle.BASE_SEED + 1, -1, 1)
    da, db = dev(a), dev(b)
    replicas = [torch.full((m, n), float("nan"), device="cuda") for _ in range(2)]
    stream = torch.cuda.current_stream().cuda_stream
    for rank in range(2):
        ctx.gemm_allgather(da[rank * 256:(rank + 1) * 256], db, replicas, rank, 256, n, k, stream)
    ctx.synchronize(stream)
    plain = run(ctx, "gemm", f"m={m},n={n},k={k}", [da, db], (m, n))
    for r in replicas:
        assert np.array_equal(r.cpu().numpy(), plain)  # same tiles, same arithmetic
    assert oracle.compare(plain, oracle.gemm_ref(a, b)).rel_frobenius <= 1e-5
    with pytest.raises(kh.KernelhError):
        ctx.gemm_allgather(da, db, replicas, 2, 256, n, k, stream)


def test_gemm_allgather_arrival_flags_signal_and_bounded_wait(ctx, oracle):
    """The barrier inside the fused gemm + all-gather. One GPU plays rank 0 of two: (1) with the
    peer's arrival word already at the epoch (written by the host, standing in for the peer), the
    kernel signals - word 0 of the peer's array becomes the epoch - finds the peer arrived and
    returns cleanly, twice in a row (the finished-CTA counter went back to zero); (2) with a peer
    word that nothing sets, the kernel's last CTA waits its two seconds, records the peer-arrival
    code with the missing rank as detail and returns: kh_synchronize gives 1001, and the context
    still computes the right product afterwards. A wait that gives up, not a fault."""
    m, n, k = 512, 256, 128
    a = oracle.uniform((m, k), oracle.BASE_SEED + 61, -1, 1)
    b = oracle.uniform((k, n), oracle.BASE_SEED + 62, -1, 1)
    da, db = dev(a), dev(b)
    plain = run(ctx, "gemm", f"m={m},n={n},k={k}", [da, db], (m, n))
    replicas = [torch.full((m, n), float("nan"), device="cuda") for _ in range(2)]
    flags = [torch.zeros(8, dtype=torch.int64, device="cuda") for _ in range(2)]  # [mine, the peer's]
    stream = torch.cuda.current_stream().cuda_stream
    for epoch in (1, 2):
        flags[0][1] = epoch  # "rank 1 has arrived"
        ctx.arm_arrival_flags([f.data_ptr() for f in flags], epoch)
        ctx.gemm_allgather(da[:256], db, replicas, 0, 256, n, k, stream)
        ctx.synchronize(stream)
        assert flags[1][0].item() == epoch and flags[1][1:].abs().sum().item() == 0
    for r in replicas:
        assert np.array_equal(r[:256].cpu().numpy(), plain[:256])
    # the flags are for ONE launch: an unarmed launch neither signals nor waits
    ctx.gemm_allgather(da[:256], db, replicas, 0, 256, n, k, stream)
    ctx.synchronize(stream)
    assert flags[1][0].item() == 2
    # nobody sets epoch 3 in my array: the wait runs out after two seconds and is reported
    ctx.arm_arrival_flags([f.data_ptr() for f in flags], 3)
    ctx.gemm_allgather(da[:256], db, replicas, 0, 256, n, k, stream)
    with pytest.raises(kh.KernelhError) as e:
        ctx.synchronize(stream)
    assert e.value.code == kh.DEVICE_TIMEOUT
    assert "another GPU's arrival flag" in e.value.message and "code 6, detail 1" in e.value.message
    assert flags[1][0].item() == 3  # it had signalled before it waited
    again = run(ctx, "gemm", f"m={m},n={n},k={k}", [da, db], (m, n))
    assert np.array_equal(again, plain)
    # the overlapped form: the kernel only signals, a one-thread launch on the context's second stream
    # waits; the next fused launch, join_arrivals and synchronize are ordered behind it
    for epoch in (4, 5):
        flags[0][1] = epoch
        torch.cuda.current_stream().synchronize()
        ctx.arm_arrival_flags([f.data_ptr() for f in flags], epoch, overlapped=True)
        ctx.gemm_allgather(da[:256], db, replicas, 0, 256, n, k, stream)
    ctx.join_arrivals(stream)
    ctx.synchronize(stream)
    assert flags[1][0].item() == 5
    ctx.arm_arrival_flags([f.data_ptr() for f in flags], 6, overlapped=True)  # nobody sets 6 in my array
    ctx.gemm_allgather(da[:256], db, replicas, 0, 256, n, k, stream)
    with pytest.raises(kh.KernelhError) as e:
        ctx.synchronize(stream)  # waits for the second stream too: its wait gave up after two seconds
    assert e.value.code == kh.DEVICE_TIMEOUT and "code 6, detail 1" in e.value.message
    assert flags[1][0].item() == 6
    assert np.array_equal(run(ctx, "gemm", f"m={m},n={n},k={k}", [da, db], (m, n)), plain)
    with pytest.raises(kh.KernelhError):
        ctx.arm_arrival_flags([flags[0].data_ptr()], 1)  # one array: not a world
    with pytest.raises(kh.KernelhError):
        ctx.arm_arrival_flags([f.data_ptr() for f in flags], 0)  # epochs are positive


def test_gemm_host_sharded_uploads_each_slice_of_b_once(ctx, oracle):
    """The sharded product on host buffers: every rank uploads only its rows of B, the slices
    are sent on to every replica of B, and after the ranks have met each one multiplies its
    rows of A. Two ranks are played here by two contexts on one GPU (plain replica pointers,
    no multicast address); the rows of C equal the device path bit for bit."""
    m, n, k = 640, 384, 256
    a = oracle.uniform((m, k), oracle.BASE_SEED + 51, -1, 1)
    b = oracle.uniform((k, n), oracle.BASE_SEED + 52, -1, 1)
    plain = run(ctx, "gemm", f"m={m},n={n},k={k}", [a, b], (m, n))
    ranks = [ctx, kh.Context(0)]
    try:
        replicas = [torch.full((k, n), float("nan"), device="cuda") for _ in range(2)]
        c_host = [np.full((m // 2, n), np.nan, np.float32) for _ in range(2)]
        for r in range(2):
            ranks[r].gemm_host_sharded_begin(np.ascontiguousarray(a[r * m // 2:(r + 1) * m // 2]),
                                             np.ascontiguousarray(b[r * k // 2:(r + 1) * k // 2]),
                                             replicas, 0, r, m // 2, n, k)
        torch.cuda.synchronize()  # stands in for the barrier across ranks
        for rep in replicas:
            assert np.array_equal(rep.cpu().numpy(), b)  # both slices reached both replicas
        for r in range(2):
            ranks[r].gemm_host_sharded_finish(c_host[r])
        assert np.array_equal(np.concatenate(c_host), plain)
        with pytest.raises(kh.KernelhError) as e:  # finish without begin
            ranks[0].gemm_host_sharded_finish(c_host[0])
        assert e.value.code == kh.USAGE_ERROR and "without a begin" in e.value.message
        with pytest.raises(kh.KernelhError):  # k does not split over three ranks
            ranks[0].gemm_host_sharded_begin(a, b, replicas + [replicas[0]], 0, 0, m, n, k)
    finally:
        ranks[1].close()


# --------------------------------------------------------------------------- attention
def attention_inputs(oracle, b, h, s):
    return (oracle.lcg((b, h, s, 64), 0x313A171B), oracle.lcg((b, h, s, 64), 0x51AC0D3E),
            oracle.lcg((b, h, s, 64), 0x29C0FFEE))


@pytest.mark.parametrize("s", [192, 512])
def test_attention_allgather_two_shards_fill_every_replica(ctx, oracle, s):
    """The fused attention + all-gather on one GPU: the two ranks' launches run one
    after the other and each stores its (batch, head) slices into both replicas of O."""
    b, h = 2, 3
    q, k, v = attention_inputs(oracle, b, h, s)
    plain = run(ctx, "attention", f"batch={b},heads={h},seq={s},head_dim=64", [q, k, v], (b, h, s, 64))
    dq, dk, dv = (dev(t).reshape(b * h, s, 64) for t in (q, k, v))
    replicas = [torch.full((b * h, s, 64), float("nan"), device="cuda") for _ in range(2)]
    stream = torch.cuda.current_stream().cuda_stream
    slices = b * h // 2
    for rank in range(2):
        lo, hi = rank * slices, (rank + 1) * slices
        ctx.attention_allgather(dq[lo:hi], dk[lo:hi], dv[lo:hi], replicas, 0, rank, slices, s, 64, stream)
    ctx.synchronize(stream)
    for r in replicas:
        assert np.array_equal(r.cpu().numpy().reshape(b, h, s, 64), plain)  # same tiles, same arithmetic
    with pytest.raises(kh.KernelhError):
        ctx.attention_allgather(dq, dk, dv, replicas, 0, 2, slices, s, 64, stream)


@pytest.mark.parametrize("b,h,s", [(2, 8, 512), (2, 8, 1024), (1, 1, 64), (1, 3, 192)])
def test_attention_reference_inputs(ctx, oracle, b, h, s):
    q, k, v = attention_inputs(oracle, b, h, s)
    o = run(ctx, "attention", f"batch={b},heads={h},seq={s},head_dim=64", [q, k, v], (b, h, s, 64))
    cmp_ = oracle.compare(o, oracle.attention_ref(q, k, v), rtol=2e-3)
    assert cmp_.non_finite == 0
    assert cmp_.max_violation <= 2e-3  # |gpu-ref| <= 2e-3 + 2e-3 |ref| on every element
    assert cmp_.max_rel <= REL * math.sqrt(s)


@pytest.mark.parametrize("b,h,s", [(5, 31, 192), (1, 300, 64), (2, 80, 320)])
def test_attention_more_work_items_than_sms(ctx, oracle, b, h, s):
    """The attention grid is persistent (a CTA per SM walks the 128-query work
    items): more items than SMs, an odd number of key tiles (the groups end an
    item on different sides), a single key tile (one softmax group idle), and a
    second launch that must give the same bits."""
    q, k, v = attention_inputs(oracle, b, h, s)
    name = f"batch={b},heads={h},seq={s},head_dim=64"
    o = run(ctx, "attention", name, [q, k, v], (b, h, s, 64))
    cmp_ = oracle.compare(o, oracle.attention_ref(q, k, v), rtol=2e-3)
    assert cmp_.non_finite == 0 and cmp_.max_violation <= 2e-3
    assert cmp_.max_rel <= REL * math.sqrt(s)
    assert np.array_equal(o, run(ctx, "attention", name, [q, k, v], (b, h, s, 64)))


@pytest.mark.parametrize("kind", ["rows_inside_tiles", "large_scores"])
def test_attention_wide_range_inside_tiles(ctx, oracle, kind):
    """What the 3xFP16 arithmetic could lose against fp32: Q, K and V are scaled by
    ONE power of two per 64-row tile before the fp16 hi/lo split, so a row far below
    its tile's largest keeps fewer bits, and the scores carry 22 significand bits,
    not 24. The error is measured against sum_j p_ij |v_jd| (the size of the terms
    the output is made of). Bounds are what the kernel meets on a B200, with margin:
    rows with e^N(0, 1.5^2) scale factors inside the tiles stay within 1e-4 (an fp32
    evaluation of the same inputs: 2e-5 to 4e-5); Q * 6, whose scores reach several
    hundred in exp2 units, within 5e-4 (fp32: 1e-5 to 2e-5; the missing two bits
    of the scores are multiplied by their size)."""
    b, h, s = (1, 300, 64) if kind == "rows_inside_tiles" else (2, 40, 320)
    rng = np.random.default_rng(77)
    q, k, v = (oracle.normal((b, h, s, 64), oracle.BASE_SEED + 40 + i, 0, 1) for i in range(3))
    if kind == "rows_inside_tiles":
        q *= np.exp(rng.normal(0, 1.0, (b, h, 1, 1))).astype(np.float32)
        k *= np.exp(rng.normal(0, 0.5, (b, h, s, 1))).astype(np.float32)
        v *= np.exp(rng.normal(0, 1.5, (b, h, s, 1))).astype(np.float32)
    else:
        q *= np.float32(6.0)
    o = run(ctx, "attention", f"batch={b},heads={h},seq={s},head_dim=64", [q, k, v], (b, h, s, 64))
    assert np.isfinite(o).all()
    q64, k64, v64 = (t.astype(np.float64) for t in (q, k, v))
    scores = q64 @ np.swapaxes(k64, -1, -2) / 8.0
    p = np.exp(scores - scores.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    ref = p @ v64
    assert np.allclose(ref, oracle.attention_ref(q, k, v), rtol=1e-9, atol=1e-12)  # the oracle agrees with this fp64 form
    err = np.max(np.abs(o - ref) / np.maximum(p @ np.abs(v64), 1e-300))
    assert err <= (1e-4 if kind == "rows_inside_tiles" else 5e-4), err
    cmp_ = oracle.compare(o, ref.astype(np.float32), rtol=2e-3)
    assert cmp_.max_violation <= 2e-3  # the reference's own tolerance still holds


def test_attention_negative_control(ctx, oracle):
    q, k, v = attention_inputs(oracle, 2, 8, 256)
    o = run(ctx, "attention", "batch=2,heads=8,seq=256,head_dim=64", [q, k, v], (2, 8, 256, 64))
    assert oracle.compare(o, oracle.attention_ref(q, k, v)).max_abs <= 2e-3
    assert oracle.compare(o, oracle.attention_ref(q, k, v, scaled=False)).max_abs > 2e-3


def test_attention_benchmark_parity_config(ctx, oracle):
    shape = (1, 1, 1024, 64)
    q, k, v = (oracle.normal(shape, oracle.BASE_SEED + i, 0, 1) for i in range(3))
    o = run(ctx, "attention", "batch=1,heads=1,seq=1024,head_dim=64", [q, k, v], shape)
    cmp_ = oracle.compare(o, oracle.attention_ref(q, k, v), rtol=2e-3)
    assert cmp_.non_finite == 0 and cmp_.max_violation <= 2e-3
    assert cmp_.max_rel <= REL * math.sqrt(1024)
    assert o.min() >= v.min() - 1e-4 and o.max() <= v.max() + 1e-4  # rows are convex combinations of V


def test_attention_batched_config_sampled(ctx, oracle):
    shape = (8, 16, 1024, 64)
    q, k, v = (oracle.normal(shape, oracle.BASE_SEED + i, 0, 1) for i in range(3))
    o = run(ctx, "attention", "batch=8,heads=16,seq=1024,head_dim=64", [q, k, v], shape)
    for lo in (0, 63, 127):  # three of the 128 (batch, head) problems in fp64
        ref = oracle.attention_ref(q, k, v, bh_begin=lo, bh_end=lo + 1).reshape(128, 1024, 64)[lo]
        cmp_ = oracle.compare(o.reshape(128, 1024, 64)[lo], ref, rtol=2e-3)
        assert cmp_.non_finite == 0 and cmp_.max_violation <= 2e-3
        assert cmp_.max_rel <= REL * math.sqrt(1024)


# --------------------------------------------------------------------------- the reference's launch sequence
def test_reference_launch_geometry_through_kernel_launch(ctx, oracle):
    """GpuModule::load + KernelLaunch with the geometry the reference's callers
    choose (bench/harness/kernelh_backend.cpp:223-427): the streaming and row
    kernels stride over whatever grid they are given."""
    n = 100003
    a, b = oracle.vecadd_pattern(n)
    da, db, dc = dev(a), dev(b), torch.zeros(n, device="cuda")
    ctx.module_launch(kh.kernel_image("vecadd"), "vecadd", ((n + 255) // 256, 1, 1), (256, 1, 1),
                      [da, db, dc], [[n], [n], [n]])
    assert oracle.bit_mismatches(dc.cpu().numpy(), oracle.vecadd_ref(a, b)) == 0
    rows, cols = 300, 1024
    x = oracle.lcg((rows, cols), 0x27AB13)
    dx, dy = dev(x), torch.zeros(rows, cols, device="cuda")
    ctx.module_launch(kh.kernel_image("softmax"), "softmax", (rows, 1, 1), (min(cols, 256), 1, 1),
                      [dx, dy], [[rows, cols], [rows, cols]])
    assert oracle.compare(dy.cpu().numpy(), oracle.softmax_ref(x)).max_abs <= 1e-4
    s = oracle.LcgStream(0x2E2E8A)
    x, g, be = s.fill((rows, cols)), s.fill(cols), s.fill(cols)
    dy.zero_()
    ctx.module_launch(kh.kernel_image("layernorm"), "layernorm", (rows, 1, 1), (256, 1, 1),
                      [dev(x), dev(g), dev(be), dy], [[rows, cols], [cols], [cols], [rows, cols]])
    assert oracle.compare(dy.cpu().numpy(), oracle.layernorm_ref(x, g, be)).max_abs <= 1e-4


def test_kernel_launch_refuses_what_the_device_cannot_run(ctx):
    x = torch.zeros(1024, device="cuda")
    image = kh.kernel_image("vecadd")
    with pytest.raises(kh.KernelhError) as e:  # 2048 threads: over the block limit, and occupancy 0
        ctx.module_launch(image, "vecadd", (1, 1, 1), (2048, 1, 1), [x, x, x], [[1024]] * 3)
    assert e.value.code == 1 and e.value.message.startswith("KernelLaunch::launch refused: ")
    assert "threads per workgroup 2048 exceeds the max 1024" in e.value.message
    with pytest.raises(kh.KernelhError) as e:  # more dynamic shared memory than the opt-in limit
        ctx.module_launch(image, "vecadd", (1, 1, 1), (256, 1, 1), [x, x, x], [[1024]] * 3,
                          dynamic_smem=300000)
    assert "opt-in limit" in e.value.message
    with pytest.raises(kh.KernelhError) as e:
        ctx.module_launch(image, "no_such_entry", (1, 1, 1), (256, 1, 1), [x, x, x], [[1024]] * 3)
    assert e.value.code != 0 and "cuModuleGetFunction(no_such_entry)" in e.value.message
    with pytest.raises(kh.KernelhError) as e:  # a corrupted code object is a typed error, not a crash
        ctx.module_launch(b"\x7fELF" + b"garbage" * 64, "vecadd", (1, 1, 1), (256, 1, 1), [x, x, x],
                          [[1024]] * 3)
    assert e.value.code != 0 and "cuModuleLoadData" in e.value.message
    ctx.vecadd(x, x, x, 1024)  # the context is still usable
    ctx.synchronize()


# --------------------------------------------------------------------------- surface
def test_launch_errors_are_reported(ctx):
    x = torch.zeros(16, device="cuda")
    with pytest.raises(kh.KernelhError) as e:
        ctx.launch("vecadd", "n=16", [x, x])
    assert e.value.code == kh.USAGE_ERROR and "takes 3 buffers, got 2" in e.value.message
    with pytest.raises(kh.KernelhError) as e:
        ctx.launch("nope", "n=16", [x])
    assert "unknown kernel template 'nope'" in e.value.message
    with pytest.raises(kh.KernelhError) as e:
        ctx.launch("vecadd", "n=abc", [x, x, x])
    assert "malformed --shape" in e.value.message


def test_bench_row_reports_reference_metrics(ctx):
    ms, rate, is_gflops = ctx.bench_row("vecadd", "n=16777216", 2, 5)
    assert ms > 0 and not is_gflops
    assert rate == pytest.approx(kh.rate(False, kh.metric("vecadd_bytes", 1 << 24), ms))
    ms, rate, is_gflops = ctx.bench_row("gemm", "m=512,n=512,k=512", 2, 5)
    assert is_gflops and rate == pytest.approx(kh.rate(True, 268435456.0, ms))


def test_registered_kernel_runs_through_the_operator_surface(ctx, oracle):
    """The plug-in point on the device: a code object registered under a new name is planned
    by its callback and launched by kh_launch like a built-in (here the vecadd code object
    under another name and with another geometry: its kernel strides over any grid), and a
    record registered over a built-in takes its place until it is unregistered."""
    image = kh.kernel_image("vecadd")
    n = 123457
    a, b = oracle.vecadd_pattern(n)
    kh.register_kernel("user_add", image, "vecadd",
                       lambda shape, sms: {"grid": [37], "block": [128], "elements": [shape["n"]] * 3, "outputs": [2],
                                           "work": 12.0 * shape["n"]})
    try:
        c = run(ctx, "user_add", f"n={n}", [a, b], (n,))
        assert oracle.bit_mismatches(c, oracle.vecadd_ref(a, b)) == 0
        ms, rate, is_gflops = ctx.bench_row("user_add", f"n={n}", 1, 3)
        assert ms > 0 and not is_gflops and rate == pytest.approx(kh.rate(False, 12.0 * n, ms))
        # over a built-in: fused_gelu now adds, until the record is taken away again
        x = oracle.lcg(n, 0x3A5F91)
        want = run(ctx, "fused_gelu", f"n={n}", [x, None], (n,))
        kh.register_kernel("fused_gelu", image, "vecadd",
                           lambda shape, sms: {"grid": [64], "block": [256], "elements": [shape["n"]] * 3, "outputs": [2]})
        assert oracle.bit_mismatches(run(ctx, "fused_gelu", f"n={n}", [a, b], (n,)), oracle.vecadd_ref(a, b)) == 0
        kh.unregister_kernel("fused_gelu")
        assert np.array_equal(run(ctx, "fused_gelu", f"n={n}", [x, None], (n,)), want)
    finally:
        kh.unregister_kernel("user_add")
    with pytest.raises(kh.KernelhError) as e:
        ctx.launch("user_add", f"n={n}", [dev(a), dev(b), dev(a)])
    assert "unknown kernel template 'user_add'" in e.value.message


@pytest.mark.parametrize("batch,heads,seq", [(1, 2, 128), (2, 3, 256), (1, 1, 1024), (1, 150, 320)])
def test_attention_causal_mask(ctx, oracle, batch, heads, seq):
    """`causal=1`: query i attends to keys 0..i. Reference: an fp64 softmax over the allowed keys
    (the oracle's routine has no mask: the reference's template has none), on the reference test's
    kind of inputs; same bound as the unmasked kernel. Row 0 of every slice must equal V's row 0
    (one key), and the unmasked result must differ (negative control). seq = 128 makes one item of
    two diagonal tiles, where the upper 64 queries of the second tile see nothing at all;
    150 slices x 3 query tiles gives the persistent CTAs items of different lengths."""
    q = oracle.lcg((batch, heads, seq, 64), 0xA77E17)
    k = oracle.lcg((batch, heads, seq, 64), 0xA77E18)
    v = oracle.lcg((batch, heads, seq, 64), 0xA77E19)
    shape = f"batch={batch},heads={heads},seq={seq},head_dim=64"
    o = run(ctx, "attention", shape + ",causal=1", [q, k, v], (batch, heads, seq, 64))
    s = np.einsum("bhqd,bhkd->bhqk", q.astype(np.float64), k.astype(np.float64)) / 8.0
    s = np.where(np.tril(np.ones((seq, seq), bool)), s, -np.inf)
    p = np.exp(s - s.max(axis=-1, keepdims=True))
    ref = np.einsum("bhqk,bhkd->bhqd", p / p.sum(axis=-1, keepdims=True), v.astype(np.float64))
    cmp_ = oracle.compare(o, ref, rtol=2e-3)
    assert cmp_.non_finite == 0 and cmp_.max_violation <= 2e-3
    assert cmp_.max_rel <= REL * math.sqrt(seq)
    assert np.allclose(o[:, :, 0, :], v[:, :, 0, :], rtol=0, atol=1e-6)
    plain = run(ctx, "attention", shape, [q, k, v], (batch, heads, seq, 64))
    assert oracle.compare(plain, ref).max_abs > 1e-3
    assert oracle.compare(plain, oracle.attention_ref(q, k, v), rtol=2e-3).max_violation <= 2e-3  # unmasked path intact


@pytest.mark.parametrize("batch,heads,seq,causal", [(1, 2, 100, 0), (2, 2, 333, 0), (1, 1, 1000, 0), (1, 3, 65, 0),
                                                     (1, 1, 40, 0), (2, 2, 200, 1), (1, 2, 1000, 1)])
def test_attention_ragged_seq(ctx, oracle, batch, heads, seq, causal):
    """seq that is not a multiple of the 64-key tile (the reference refuses it): the last tile's
    missing keys are masked and its missing queries are not stored. Against an fp64 softmax on the
    reference test's kind of inputs, with and without the causal mask; the rows after the output
    (a canary slice) stay untouched."""
    q = oracle.lcg((batch, heads, seq, 64), 0xA77E27)
    k = oracle.lcg((batch, heads, seq, 64), 0xA77E28)
    v = oracle.lcg((batch, heads, seq, 64), 0xA77E29)
    shape = f"batch={batch},heads={heads},seq={seq},head_dim=64" + (",causal=1" if causal else "")
    out = torch.full((batch * heads * seq * 64 + 4096,), float("nan"), device="cuda")
    bufs = [dev(q), dev(k), dev(v), out]
    ctx.launch("attention", shape, bufs, torch.cuda.current_stream().cuda_stream)
    ctx.synchronize(torch.cuda.current_stream().cuda_stream)
    got = out.cpu().numpy()
    assert np.isnan(got[batch * heads * seq * 64:]).all()  # nothing written past the last real query
    o = got[:batch * heads * seq * 64].reshape(batch, heads, seq, 64)
    s = np.einsum("bhqd,bhkd->bhqk", q.astype(np.float64), k.astype(np.float64)) / 8.0
    if causal:
        s = np.where(np.tril(np.ones((seq, seq), bool)), s, -np.inf)
    p = np.exp(s - s.max(axis=-1, keepdims=True))
    ref = np.einsum("bhqk,bhkd->bhqd", p / p.sum(axis=-1, keepdims=True), v.astype(np.float64))
    cmp_ = oracle.compare(o, ref, rtol=2e-3)
    assert cmp_.non_finite == 0 and cmp_.max_violation <= 2e-3
    assert cmp_.max_rel <= REL * math.sqrt(seq)
