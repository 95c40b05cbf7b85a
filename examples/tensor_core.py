"""The TF32 tensor-core `matmul_kernel` of the reference manual (docs/src/manual/tensor_core.md:265-391) on B200.

The manual's kernel feeds `mma.sync.m16n8k8` (TF32) from shared memory: 128-bit `cp.async` tiled copies gmem ->
smem, then smem -> register copies retiled for the MMA -- a `UniversalCopy` for the M-major A and `ldmatrix`
(`LDSM_U32x4_N`) for the K-major B, built with `make_tiled_copy_A / _B` -- double-buffered like the pipeline example.
`host_side()` builds those objects as the manual does and evaluates them.

On sm_100a the smem -> register step does not exist: `tcgen05.mma` reads both operands from shared memory through
descriptors (M-major and K-major alike), TMA writes them there in the 128-byte swizzle, and the accumulator lives in
tensor memory.  `matmul` is the manual's `matmul(A, B, C)` with one device-level `gemm!` on the `kind::tf32` atom; like
the manual's kernel it is a tf32 product (operands read with a 10-bit mantissa, fp32 accumulation), which is what
`allow_tf32=True` asks for.

    python examples/tensor_core.py     # needs an sm_100 GPU
"""
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import __graft_entry__ as entry  # noqa: E402

mb = entry.load_package()
F32 = mb._lib.F32


def host_side():
    """tensor_core.md:352-381 for thread 1: the tiled MMA, the four tiled copies and the shared-memory layouts."""
    mma = mb.make_tiled_mma(mb.mma_op("MMAOP_16x8x8_F32TF32TF32F32_TN"), mb.make_layout((2, 2, 1), (2, 1, 1)), (32, 32, 8))
    gmem_copy_A = mb.make_tiled_copy(mb.CopyAtom(mb.CPOP_ASYNC_CACHEALWAYS(128), F32), mb.make_layout((16, 8)),
                                     mb.make_layout((4, 1)))
    gmem_copy_B = mb.make_tiled_copy(mb.CopyAtom(mb.CPOP_ASYNC_CACHEALWAYS(128), F32), mb.make_layout((32, 4), (4, 1)),
                                     mb.make_layout((1, 4)))
    # "A is M-major, so we cannot use LDSM_U32x4_N" (tensor_core.md:369)
    smem_copy_A = mb.make_tiled_copy_A(mb.CopyAtom(mb.UniversalCopy(32), F32), mma)
    smem_copy_B = mb.make_tiled_copy_B(mb.CopyAtom(mb.ldsm_op("LDSM_U32x4_N"), F32), mma)
    sA_layout = mb.make_layout((128, 16, 2), (1, 128, 2048))
    sB_layout = mb.make_layout((128, 16, 2), (16, 1, 2048))
    buf = torch.zeros(1)
    sA, sB = mb.MoYeArray(buf, sA_layout), mb.MoYeArray(buf, sB_layout)
    thr_mma = mma.get_slice(1)
    tCsA, tCsB = thr_mma.partition_A(sA), thr_mma.partition_B(sB)                  # (MMA, MMA_M, MMA_K, 2)
    tCsA_retiled = smem_copy_A.get_slice(1).partition_S(sA)
    tCsB_retiled = smem_copy_B.get_slice(1).partition_S(sB)
    return {
        "threads": len(mma), "mma_tile": mma.tile_shape(),
        "gmem_copy_A_tiler": gmem_copy_A.tiler_mn, "gmem_copy_B_tiler": gmem_copy_B.tiler_mn,
        "smem_copy_A_tiler": smem_copy_A.tiler_mn, "smem_copy_B_tiler": smem_copy_B.tiler_mn,
        "smem_copy_threads": (len(smem_copy_A), len(smem_copy_B)),
        "tCsA": tCsA.layout.shape, "tCsB": tCsB.layout.shape,
        "tCsA_retiled": tCsA_retiled.layout.shape, "tCsB_retiled": tCsB_retiled.layout.shape,
        "values_per_thread_A": mb.size(tCsA.layout) // 2, "values_per_thread_B": mb.size(tCsB.layout) // 2,
    }


def matmul(A, B, C):
    """tensor_core.md:352-391 with the launch replaced by the library call: the tile of one CTA is one tcgen05 atom of
    128 x 256 x 8 (the manual tiles 128 x 128 x 16 out of sixteen m16n8k8 atoms per K block)."""
    mma = mb.make_tiled_mma(mb.sm100_mma_op("TF32", 256))
    return mb.gemm_(mma, C, A, B, None, allow_tf32=True)


def test():
    """tensor_core.md:393-404: A (2048, 256) M-major, B (2048, 256) stored K-major, C (2048, 2048) column-major."""
    dev = torch.device("cuda", 0)
    M, N, K = 2048, 2048, 256
    a = torch.randn(M * K, device=dev)                      # A is M-major: (M, K):(1, M)
    bt = torch.randn(N * K, device=dev)                     # B is K-major: (N, K):(K, 1)
    c = torch.zeros(M * N, device=dev)
    A = mb.MoYeArray(a, mb.make_layout((M, K)))
    B = mb.MoYeArray(bt, mb.make_layout((N, K), (K, 1)))
    C = mb.MoYeArray(c, mb.make_layout((M, N)))
    matmul(A, B, C)
    mb.synchronize_status(dev)
    trunc = lambda t: (t.view(torch.int32) & -8192).view(torch.float32)   # what the tf32 kind reads: low 13 bits dropped
    want = trunc(a).view(K, M).t().double() @ trunc(bt).view(N, K).t().double()
    got = c.view(N, M).t().double()
    err = ((got - want).abs().max() / want.abs().max()).item()
    exact = a.view(K, M).t().double() @ bt.view(N, K).t().double()
    err_exact = ((got - exact).abs().max() / exact.abs().max()).item()
    print(f"C = A * B'  ({M} x {N} x {K}, tf32 tensor cores): vs tf32-read operands {err:.2e}, vs exact product {err_exact:.2e}")
    assert err < 1e-5 and err_exact < 2e-3
    return err


if __name__ == "__main__":
    for k, v in host_side().items():
        print(f"{k:22s} {v}")
    test()
