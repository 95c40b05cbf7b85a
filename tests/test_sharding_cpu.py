"""The multi-GPU path on CPU: two gloo ranks shard a GEMM along M (and a decode GEMM along N),
each computes its shard with the oracle, and the gathered result equals the unsharded one."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_ranges_partition_everything(mb):
    for extent, world, align in [(8192, 8, 128), (8192, 4, 128), (1000, 3, 128), (28672, 8, 128), (5, 8, 1), (130, 2, 128)]:
        seen = []
        for r in range(world):
            lo, hi = mb.shard_range(extent, world, r, align)
            assert 0 <= lo <= hi <= extent
            assert lo % align == 0 or lo == extent
            seen += list(range(lo, hi))
        assert seen == list(range(extent))
    with pytest.raises(ValueError):
        mb.shard_range(10, 2, 2)


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import __graft_entry__ as ge
    import host_oracle as ho
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mb = ge.load_package()
    M, N, K = 200, 96, 64
    a, b = ho.uniform_pm1_f16_bits(3, (M * K,)), ho.uniform_pm1_f16_bits(4, (N * K,))
    full = ho.gemm_samples(a, b, ho.F16, M, N, K, np.arange(M, dtype=np.int32))
    # M-sharded GEMM: rank owns rows [lo, hi) of A and C, B replicated
    lo, hi = mb.shard_range(M, world, rank, align=8)
    mine = ho.gemm_samples(a[lo * K:hi * K], b, ho.F16, hi - lo, N, K, np.arange(hi - lo, dtype=np.int32))
    gathered = mb.all_gather_rows(torch.from_numpy(mine), M, world, align=8)
    ok_rows = np.array_equal(gathered.numpy(), full)
    # N-sharded decode GEMM: rank owns rows [lo, hi) of W = columns of Y
    lo, hi = mb.shard_range(N, world, rank, align=16)
    cols = ho.gemm_samples(a, b[lo * K:hi * K], ho.F16, M, hi - lo, K, np.arange(M, dtype=np.int32))
    gathered_c = mb.all_gather_cols(torch.from_numpy(cols), N, world, align=16)
    ok_cols = np.array_equal(gathered_c.numpy(), full)
    slowest = mb.max_over_ranks(10.0 + rank, torch.device("cpu"))
    dist.barrier()
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(f"{int(ok_rows)} {int(ok_cols)} {slowest}")
    dist.destroy_process_group()


def test_two_gloo_ranks_shard_and_gather(tmp_path):
    world = 2
    port = 29600 + os.getpid() % 300
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        ok_rows, ok_cols, slowest = open(tmp_path / f"rank{r}.txt").read().split()
        assert ok_rows == "1" and ok_cols == "1"
        assert float(slowest) == 11.0


def test_stream_k_schedule_covers_every_unit_once():
    """The arithmetic of the decode kernel's schedule (`plan_runs` and the `locate` / `segment_end` lambdas of
    csrc/gemm_skinny.cu), restated here line for line: for T row-blocks of k K-blocks on up to 148 CTAs, every
    (row-block, K-block) unit is processed exactly once, and no CTA produces more than the two partial pieces its
    workspace slots hold.  (The kernel itself is checked against the oracle on the same shapes in the GPU tests.)"""
    def plan(T, kb, sms=148, k_min=8):
        total = T * kb
        grid = min(sms, total // k_min) if total // k_min > 0 else 1
        if grid == sms and T < sms and 2 * T >= sms and (sms - T) * kb <= 3000:
            grid = T                                         # one whole row-block per CTA, the other SMs idle
        q, r = T // grid, T % grid
        whole, split = (q, r) if q >= 1 else (0, T)
        return grid, whole, split, split * kb

    for T, kb in [(224, 128), (64, 128), (112, 64), (1, 8), (8, 16), (148, 128), (296, 4), (300, 1), (149, 128), (185, 64),
                  (185, 8), (221, 32), (4096, 8), (33, 100), (7, 1), (296, 8), (17, 2), (5, 3), (150, 2), (223, 16), (112, 32), (140, 128), (128, 96),
                  (147, 1000), (74, 8), (150, 128), (160, 32), (149, 64), (149, 148), (149, 147)]:
        grid, whole, split, units = plan(T, kb)
        seen = set()
        for c in range(grid):
            run_start = lambda cc: cc * units // grid if units >= grid else min(cc, units)
            ub, ue = run_start(c), run_start(c + 1)
            ns = ue - ub
            # the partial-sum exchange of a cut row-block counts on EVERY CTA between its first and its last owner
            # arriving: no CTA before the last one with units may have an empty run
            assert ns >= 1 or ub == units, (T, kb, c)
            nv = ns + whole * kb
            v, partial_pieces = 0, 0
            while v < nv:
                if v < ns:
                    u = ub + v
                    tile = u // kb
                    k = u - tile * kb
                    seg_end = min((tile + 1) * kb - ub, ns)
                else:
                    j = (v - ns) // kb
                    tile = split + c + j * grid
                    k = (v - ns) - j * kb
                    seg_end = ns + (j + 1) * kb
                if not (k == 0 and seg_end - v == kb):
                    partial_pieces += 1
                for i in range(seg_end - v):
                    assert (tile, k + i) not in seen
                    seen.add((tile, k + i))
                v = seg_end
            assert partial_pieces <= 2, (T, kb, c)
        assert seen == {(t, k) for t in range(T) for k in range(kb)}, (T, kb)
