"""The reference's examples/gemm.jl on the tcgen05 atoms: C = A * B' for column-major Float32 arrays.

The reference's `matmul_kernel` (examples/gemm.jl:4-64) tiles A, B, C with `@tile`, stages the tiles in shared
memory with `copyto!`, partitions them over 256 threads with `@parallelize` and runs the `gemm!` tower.  Here the
same call, `matmul(A, B, C)` (examples/gemm.jl:66-89), hands the whole product to one device-level
`gemm!(tiled_mma, C, A, B)` whose atom is a tcgen05 instruction: the kernel stages the same tiles by TMA and
accumulates in tensor memory.  Float32 operands keep Float32 accuracy: three tf32 tensor-core products of their high
and low parts (pass `allow_tf32=True` for a single product with 10-bit mantissas).

    python examples/gemm.py            # needs an sm_100 GPU
"""
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import __graft_entry__ as entry  # noqa: E402

mb = entry.load_package()


def matmul(A, B, C):
    """examples/gemm.jl:66-89 with the launch replaced by the library call."""
    M, K = A.layout.shape
    N = B.layout.shape[0]
    # the CTA tile the reference spells as blocklayout_A/B/C = (128,8) / (128,8) / (128,128):
    # one tcgen05 atom of 128 x 256 x 8 per CTA, K walked in 32-element blocks by the kernel
    mma = mb.make_tiled_mma(mb.sm100_mma_op("TF32", 256))
    assert mma.tile_size(0) == 128 and mma.tile_size(1) == 256 and mma.tile_size(2) == 8
    # what one CTA sees, in the reference's own vocabulary (host-evaluated layout algebra, no data moved)
    gA = mb.local_tile(A, (128, 32), (1, mb.COLON))      # (128, 32, K/32)
    gC = mb.local_tile(C, (128, 256), (1, 1))            # (128, 256)
    assert gA.layout.shape[:2] == (128, 32) and gC.layout.shape == (128, 256)
    return mb.gemm_(mma, C, A, B, None)


def test():
    """examples/gemm.jl:91-100: A (2048, 256), B (2048, 256), C (2048, 2048), all column-major Float32."""
    dev = torch.device("cuda", 0)
    M, N, K = 2048, 2048, 256
    a, b = torch.randn(M * K, device=dev), torch.randn(N * K, device=dev)
    c = torch.randn(M * N, device=dev)
    A = mb.MoYeArray(a, mb.make_layout((M, K)))          # column-major like a Julia CuArray
    B = mb.MoYeArray(b, mb.make_layout((N, K)))
    C = mb.MoYeArray(c, mb.make_layout((M, N)))
    matmul(A, B, C)
    mb.synchronize_status(dev)
    want = a.view(K, M).t().double() @ b.view(K, N).double()   # torch views are row-major: a.view(K, M).t() is A
    got = c.view(N, M).t().double()
    err = ((got - want).abs().max() / want.abs().max()).item()
    print(f"C = A * B'  ({M} x {N} x {K}, Float32): max |err| / max |C| = {err:.2e}")
    assert err < 1e-5
    return err


if __name__ == "__main__":
    test()
