"""Splitting the hot path over the GPUs of one box: one process per GPU, independent shards.

The reference has no multi-GPU code at all.  The GEMM shards along M (rows of A and D, B
replicated), the weight-bound decode GEMM along N (rows of W, columns of Y, X replicated) and
the copy along row blocks; no shard needs another shard's data, so the timed path has no
collective.  `all_gather_*` reassemble a result over NCCL (or gloo) when a caller wants the
whole matrix on every rank.
"""
import ctypes

import torch

__all__ = ["shard_range", "shard_rows", "all_gather_rows", "all_gather_cols", "max_over_ranks", "Communicator"]


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
    if min(sizes) == biggest and shard.is_contiguous():
        # equal blocks: one collective straight into the assembled matrix, no staging copies
        full = torch.empty((extent,) + tuple(shard.shape[1:]), dtype=shard.dtype, device=shard.device)
        dist.all_gather_into_tensor(full, shard, group=group)
        return full
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


class Communicator:
    """This rank's NCCL communicator behind the C ABI (`moye_b200_comm_init`, `moye_b200_allgather`,
    `moye_b200_bcast`): what a Julia or C caller of the library uses to put an M- or N-sharded result back
    together, driven here from Python.  The 128-byte id made by rank 0 has to reach the other ranks over some host
    channel; this class sends it through an already initialised `torch.distributed` group (any backend), a C
    caller would use MPI, a file or a socket.  One communicator per handle, i.e. per (thread, device)."""

    def __init__(self, rank, world, device, group=None):
        import torch.distributed as dist
        from . import _lib
        self._lib, self.rank, self.world = _lib, rank, world
        self.device = torch.device(device)
        lib = _lib.load()
        buf = ctypes.create_string_buffer(128)
        if rank == 0:
            _lib.check(lib.moye_b200_comm_unique_id(buf))
        box = [buf.raw]
        dist.broadcast_object_list(box, src=0, group=group)
        self._h = _lib.handle(self.device.index)
        with torch.cuda.device(self.device):
            _lib.check(lib.moye_b200_comm_init(self._h, rank, world, box[0]))

    def _stream(self, stream):
        return stream if stream is not None else ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _tensor(self, t):
        from .algorithm import _tensor_arg
        from .array import MoYeArray
        return _tensor_arg(t if isinstance(t, MoYeArray) else MoYeArray(t), "tensor")

    def allgather(self, shard, full, mode=0, align=1, stream=None):
        """Every rank's block of `full` along `mode` (cut by `shard_range`) ends up in every rank's `full`."""
        with torch.cuda.device(self.device):
            self._lib.check(self._lib.load().moye_b200_allgather(
                self._h, ctypes.byref(self._tensor(shard)), ctypes.byref(self._tensor(full)), mode, align,
                self._stream(stream)))
        return full

    def bcast(self, t, root=0, stream=None):
        """`t` of rank `root` into `t` of every rank (the replicated operand: B of the M-sharded GEMM)."""
        with torch.cuda.device(self.device):
            self._lib.check(self._lib.load().moye_b200_bcast(self._h, ctypes.byref(self._tensor(t)), root,
                                                             self._stream(stream)))
        return t

    def destroy(self):
        if self._h is not None:
            self._lib.check(self._lib.load().moye_b200_comm_destroy(self._h))
            self._h = None
