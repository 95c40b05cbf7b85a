"""Splitting the hot path over the GPUs of one box: one process per GPU, independent shards.

The reference has no multi-GPU code at all.  The GEMM shards along M (rows of A and D, B
replicated), the weight-bound decode GEMM along N (rows of W, columns of Y, X replicated) and
the copy along row blocks; no shard needs another shard's data, so the timed path has no
collective.  `all_gather_*` reassemble a result over NCCL (or gloo) when a caller wants the
whole matrix on every rank.
"""
import torch

__all__ = ["shard_range", "shard_rows", "all_gather_rows", "all_gather_cols", "max_over_ranks"]


def shard_range(extent, world, rank, align=1):
    """[begin, end) of rank's contiguous block of `extent` items, blocks being multiples of
    `align` (the last block takes the ragged remainder); every item belongs to exactly one rank."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank / world size")
    units = -(-extent // align)
    lo = (units * rank // world) * align
    hi = (units * (rank + 1) // world) * align
    return min(lo, extent), min(hi, extent)


def shard_rows(t, world, rank, align=1):
    """Rows [begin, end) of a 2-D tensor as a view (no copy)."""
    lo, hi = shard_range(t.shape[0], world, rank, align)
    return t[lo:hi]


def all_gather_rows(shard, extent, world, align=1, group=None):
    """Gather row-block shards (dim 0) of a matrix with `extent` rows onto every rank."""
    import torch.distributed as dist
    sizes = [hi - lo for lo, hi in (shard_range(extent, world, r, align) for r in range(world))]
    biggest = max(sizes)
    # collectives want equal-sized pieces: pad the ragged last shard, trim after the gather
    padded = torch.zeros((biggest,) + tuple(shard.shape[1:]), dtype=shard.dtype, device=shard.device)
    padded[:shard.shape[0]] = shard
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:n] for p, n in zip(parts, sizes)], dim=0)


def all_gather_cols(shard, extent, world, align=1, group=None):
    """Gather column-block shards (dim 1), e.g. the N-sharded Y of the decode GEMM."""
    return all_gather_rows(shard.t().contiguous(), extent, world, align, group).t()


def max_over_ranks(value, device, group=None):
    """The slowest rank's time: what a multi-GPU measurement reports."""
    import torch.distributed as dist
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
