"""The double-buffered `matmul_kernel` of the reference manual (docs/src/manual/pipeline.md:89-202) on B200.

The manual's kernel overlaps three things by hand: the gmem -> smem copy of K tile k+1 (`copyto!(copy_A, tAsA[:, :, :,
smem_write], tAgA[:, :, :, k_tile + 1])`), the smem -> register copy of K block k+1 and the `gemm!` of K block k,
with two shared-memory buffers and register prefetch.  `host_side()` builds exactly the objects the manual builds
(the padded `(bM, bK, 2)` shared-memory layouts, the `CPOP_ASYNC_CACHEALWAYS` tiled copies, the 32 x 8 thread MMA)
and evaluates every partition the kernel takes, so the shapes in the manual's comments can be checked.

On sm_100a the same pipeline is part of the library's GEMM kernel: the two buffers become a ring of 4 stages filled
by TMA and handed over with mbarriers (producer warp), the register prefetch disappears because tcgen05.mma reads
its operands from shared memory, and `gemm!` is one `tcgen05.mma` per 32 bytes of K issued by one thread.  `matmul`
is therefore the manual's `matmul(A, B, C)` with the launch replaced by one device-level `gemm!`.

    python examples/pipeline.py        # needs an sm_100 GPU
"""
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import __graft_entry__ as entry  # noqa: E402

mb = entry.load_package()
F32 = mb._lib.F32


def host_side(M=2048, N=2048, K=256):
    """Everything `matmul` and `matmul_kernel` of pipeline.md:89-191 compute before the first byte moves, for thread 1
    of CTA (1, 1).  Returns the shapes the manual writes in its comments."""
    bM, bN, bK = 128, 128, 8
    sA_layout = mb.make_layout((bM, bK, 2), (1, bM + 2, (bM + 2) * bK))       # pipeline.md:171
    sB_layout = mb.make_layout((bN, bK, 2), (1, bN + 2, (bN + 2) * bK))
    copy_A = mb.make_tiled_copy(mb.CopyAtom(mb.CPOP_ASYNC_CACHEALWAYS(64), F32), mb.make_layout((32, 8)), mb.make_layout((2, 1)))
    copy_B = mb.make_tiled_copy(mb.CopyAtom(mb.CPOP_ASYNC_CACHEALWAYS(64), F32), mb.make_layout((32, 8)), mb.make_layout((2, 1)))
    mma_C = mb.make_tiled_mma(mb.UniversalFMA(F32), mb.make_layout((32, 8)))  # pipeline.md:185-186
    buf = torch.zeros(1)                                                       # a pointer stand-in: only layouts matter here
    mA = mb.MoYeArray(buf, mb.make_layout((M, K)))
    mB = mb.MoYeArray(buf, mb.make_layout((N, K)))
    mC = mb.MoYeArray(buf, mb.make_layout((M, N)))
    sA, sB = mb.MoYeArray(buf, sA_layout), mb.MoYeArray(buf, sB_layout)
    gA = mb.local_tile(mA, (bM, bK), (1, mb.COLON))                            # @tile mA (bM, bK) (blockIdx().x, :)
    gB = mb.local_tile(mB, (bN, bK), (1, mb.COLON))
    gC = mb.local_tile(mC, (bM, bN), (1, 1))
    thr_copy_a, thr_copy_b = copy_A.get_slice(1), copy_B.get_slice(1)
    tAgA, tAsA = thr_copy_a.partition_S(gA), thr_copy_a.partition_D(sA)        # (CPY, CPY_M, CPY_K, k), (CPY, CPY_M, CPY_K, 2)
    tBgB, tBsB = thr_copy_b.partition_S(gB), thr_copy_b.partition_D(sB)
    thr_mma = mma_C.get_slice(1)
    tCsA, tCsB, tCgC = thr_mma.partition_A(sA), thr_mma.partition_B(sB), thr_mma.partition_C(gC)
    tCrA = mb.make_fragment_like(tCsA.layout(mb.COLON, mb.COLON, mb.COLON, 1))  # make_fragment_A(thr_mma, tCsA[:, :, :, _1])
    tCrC = mb.make_fragment_like(tCgC.layout)
    return {
        "threads": len(mma_C), "blocks": (-(-M // bM), -(-N // bN)),
        "copy_tiler": copy_A.tiler_mn, "mma_tile": mma_C.tile_shape(),
        "gA": gA.layout.shape, "gC": gC.layout.shape,
        "tAgA": tAgA.layout.shape, "tAsA": tAsA.layout.shape, "tBgB": tBgB.layout.shape, "tBsB": tBsB.layout.shape,
        "tCsA": tCsA.layout.shape, "tCsB": tCsB.layout.shape, "tCgC": tCgC.layout.shape,
        "tCrA": tCrA.shape, "tCrC": tCrC.shape,
        "k_tile_max": mb.size(tAgA.layout, 3), "k_block_max": mb.size(tCrA, 2),
        "smem_floats": int(mb.cosize(sA_layout)) + int(mb.cosize(sB_layout)),
    }


def matmul(A, B, C):
    """pipeline.md:165-191: C = A * B' for column-major Float32 MoYeArrays.  The manual multiplies Float32 with FMAs
    (`UniversalFMA`); the device call keeps Float32 accuracy (three tf32 tensor-core products of high and low parts)."""
    return mb.gemm_(mb.make_tiled_mma(mb.sm100_mma_op("TF32", 256)), C, A, B, None)


def test():
    """pipeline.md:193-202: A (2048, 256), B (2048, 256), C (2048, 2048), `C == A * B'` up to Float32 rounding."""
    dev = torch.device("cuda", 0)
    M, N, K = 2048, 2048, 256
    a, b = torch.randn(M * K, device=dev), torch.randn(N * K, device=dev)
    c = torch.zeros(M * N, device=dev)
    A = mb.MoYeArray(a, mb.make_layout((M, K)))
    B = mb.MoYeArray(b, mb.make_layout((N, K)))
    C = mb.MoYeArray(c, mb.make_layout((M, N)))
    matmul(A, B, C)
    mb.synchronize_status(dev)
    want = a.view(K, M).t().double() @ b.view(K, N).double()
    err = ((c.view(N, M).t().double() - want).abs().max() / want.abs().max()).item()
    print(f"C = A * B'  ({M} x {N} x {K}, Float32): max |err| / max |C| = {err:.2e}")
    assert err < 1e-5
    return err


if __name__ == "__main__":
    for k, v in host_side().items():
        print(f"{k:12s} {v}")
    test()
