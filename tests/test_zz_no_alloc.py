"""The allocation-free scan entry point (kh_scan_noalloc) against the ordinary
one (kh_scan), through the C ABI on a B200.

kh_scan_noalloc exists for callers that may not allocate device memory: hosts
whose memory pool owns the whole device, plugin callbacks that must not enter an
allocator, deployments with a fixed, audited memory budget. Its look-back
scratch is a fixed array inside the library, shared by every call on a device,
so this file checks exactly what that sharing could break: two calls in a row
of different sizes (the second sees whatever the first left in the array), the
size limit, and agreement with the allocating entry point bit for bit (both run
the same fp64-accumulating kernel source, so equality is the right bound).

This file sorts last on purpose: if it fails, `pytest -x` has already run every
other test."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
import kernelh_b200 as kh

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    torch.zeros(1, device="cuda")
    c = kh.Context(0)
    yield c
    c.close()


def both(ctx, x):
    n = x.numel()
    stream = torch.cuda.current_stream().cuda_stream
    want = torch.full_like(x, float("nan"))
    ctx.scan(x, want, n, stream)
    ctx.synchronize(stream)
    got = torch.full_like(x, float("nan"))
    kh.scan_noalloc(x, got, n, stream)
    torch.cuda.synchronize()
    return got, want


def test_no_alloc_scan_matches_scan_on_consecutive_calls(ctx, oracle):
    torch.manual_seed(7)
    # first call: many tiles; second call: fewer tiles on the now-dirty array;
    # third: back to the large size; fourth: a ragged single tile
    for n in (1_000_000, 12_345, 1_000_000, 1000):
        x = torch.rand(n, device="cuda")
        got, want = both(ctx, x)
        assert torch.equal(got, want), n
        ref = oracle.scan_ref(x.cpu().numpy())
        assert oracle.bit_mismatches(got.cpu().numpy(), ref) == 0
        kh.scan_noalloc_status(torch.cuda.current_stream().cuda_stream)  # no wait ran out


def test_no_alloc_scan_allocates_nothing(ctx):
    n = 1 << 20
    x = torch.rand(n, device="cuda")
    y = torch.empty_like(x)
    kh.scan_noalloc(x, y, n, torch.cuda.current_stream().cuda_stream)  # set-up call
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        kh.scan_noalloc(x, y, n, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before


def test_no_alloc_scan_size_limit(ctx):
    limit = kh.scan_noalloc_max_elements()
    assert limit == 1 << 24
    x = torch.rand(limit, device="cuda")
    got, want = both(ctx, x)
    assert torch.equal(got, want)
    big = torch.empty(limit + 1, device="cuda")
    with pytest.raises(kh.KernelhError) as e:
        kh.scan_noalloc(big, big, limit + 1, None)
    assert e.value.code == kh.USAGE_ERROR
    assert "exceeds the fixed scratch" in e.value.message and "kh_scan" in e.value.message
    with pytest.raises(kh.KernelhError):
        kh.scan_noalloc(big, big, 0, None)
