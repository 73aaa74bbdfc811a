"""The multi-GPU partitioning and gather logic on CPU: two gloo ranks, with a
plain CPU matmul / attention standing in for the kernels (only the host-side
sharding and the collective are under test here)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kernelh_b200 import sharding


def test_unit_range_rules():
    assert sharding.unit_range(8192, 8, 3) == (3072, 4096)
    assert [sharding.unit_range(128, 4, r) for r in range(4)] == [(0, 32), (32, 64), (64, 96), (96, 128)]
    with pytest.raises(ValueError):
        sharding.unit_range(10, 4, 0)
    with pytest.raises(ValueError):
        sharding.unit_range(8, 2, 2)
    assert sharding.gemm_shard_shape(8192, 8192, 8192, 8, 7) == {"rows": (7168, 8192), "shape": "m=1024,n=8192,k=8192"}
    assert sharding.attention_shard_shape(8, 16, 1024, 64, 8, 1) == {
        "units": (16, 32), "shape": "batch=16,heads=1,seq=1024,head_dim=64"}


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)  # identical inputs on every rank
        m, n, k = 64, 48, 32
        a, b = torch.randn(m, k), torch.randn(k, n)
        c = torch.zeros(m, n)
        lo, hi = sharding.gemm_shard_shape(m, n, k, world, rank)["rows"]
        c[lo:hi] = a[lo:hi] @ b                      # this rank's row block, written in place
        sharding.gather_output(c, c[lo:hi], dist)    # one all-gather of the C shards
        ok_gemm = torch.allclose(c, a @ b)

        bsz, heads, seq, d = 2, 4, 16, 8
        q, kk, v = (torch.randn(bsz, heads, seq, d) for _ in range(3))
        o = torch.zeros(bsz * heads, seq, d)
        ulo, uhi = sharding.attention_shard_shape(bsz, heads, seq, d, world, rank)["units"]
        flat = lambda t: t.reshape(bsz * heads, seq, d)
        att = lambda qq, k2, vv: torch.softmax(qq @ k2.transpose(-1, -2) / d ** 0.5, -1) @ vv
        o[ulo:uhi] = att(flat(q)[ulo:uhi], flat(kk)[ulo:uhi], flat(v)[ulo:uhi])
        sharding.gather_output(o, o[ulo:uhi], dist)
        ok_att = torch.allclose(o, att(flat(q), flat(kk), flat(v)), atol=1e-6)

        # timing convention: the job time is the max over ranks
        t = torch.tensor([1.0 + rank])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        results[rank] = (ok_gemm, ok_att, t.item())
    finally:
        dist.destroy_process_group()


def test_two_rank_shard_and_gather_over_gloo():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert dict(results) == {0: (True, True, 2.0), 1: (True, True, 2.0)}
