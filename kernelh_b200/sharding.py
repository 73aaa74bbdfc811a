"""Partitioning of the two kernels that run on several GPUs of one box: gemm by
M-row blocks (B replicated), attention by flattened (batch, head) problems. The
units are independent, so the only exchange is one all-gather of the output
shards. One process per GPU; `torch.distributed` (NCCL on GPUs, gloo in the CPU
tests) is the plumbing. No kernel reads another GPU's memory."""
from __future__ import annotations


def unit_range(units: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, equal shares of `units` (C rows, or (batch, head) problems)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is outside a world of {world}")
    if units % world != 0:
        raise ValueError(f"{units} units do not split evenly over {world} ranks "
                         "(the all-gather needs equal shards)")
    per = units // world
    return rank * per, (rank + 1) * per


def gemm_shard_shape(m: int, n: int, k: int, world: int, rank: int) -> dict:
    lo, hi = unit_range(m, world, rank)
    return {"rows": (lo, hi), "shape": f"m={hi - lo},n={n},k={k}"}


def attention_shard_shape(batch: int, heads: int, seq: int, head_dim: int, world: int,
                          rank: int) -> dict:
    lo, hi = unit_range(batch * heads, world, rank)
    # a shard is `hi - lo` independent (batch, head) problems: present it as batch=hi-lo, heads=1
    return {"units": (lo, hi), "shape": f"batch={hi - lo},heads=1,seq={seq},head_dim={head_dim}"}


def gather_output(full, shard, dist, group=None):
    """All-gather equal row shards into `full` (in place when `shard` is a view of it)."""
    dist.all_gather_into_tensor(full.view(-1), shard.reshape(-1), group=group)
    return full
