"""The reference's transpose test (test/host/copy_async.jl:51-95) as one library call.

`transpose_kernel` tiles both arrays, copies a tile to a padded shared-memory array, views it through
`MoYe.transpose` and copies it out.  Here `copyto!(a, transpose(b))` on global-memory arrays runs the transposing
TMA kernel; the copy kernel of the same file (`copy_kernel`, :3-25) is `copyto!(tiled_copy, dst, src)`.

    python examples/transpose.py       # needs an sm_100 GPU
"""
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import __graft_entry__ as entry  # noqa: E402

mb = entry.load_package()


def test_transpose(M, N):
    dev = torch.device("cuda", 0)
    a = torch.rand(M * N, device=dev)                    # a: (M, N) column-major
    b = torch.rand(N * M, device=dev)                    # b: (N, M) column-major
    A = mb.MoYeArray(a, mb.make_layout((M, N)))
    B = mb.MoYeArray(b, mb.make_layout((N, M)))
    mb.copyto_(A, mb.transpose(B))
    mb.synchronize_status(dev)
    assert torch.equal(a.view(N, M), b.view(M, N).t())   # a == transpose(b)
    print(f"a == transpose(b) for {M} x {N} Float32")


def test_copy_async(M, N):
    """copy_kernel with 128-bit atoms: thread layout (16, 16), 8 fp16 values per thread."""
    dev = torch.device("cuda", 0)
    src = torch.rand(M * N, device=dev).half()
    dst = torch.zeros_like(src)
    atom = mb.CopyAtom(mb.UniversalCopy(128), mb._lib.F16)
    tiled_copy = mb.make_tiled_copy(atom, mb.make_layout((16, 16)), mb.make_layout((8, 1)))
    lay = mb.make_layout((M, N))
    mb.copyto_(tiled_copy, mb.MoYeArray(dst, lay), mb.MoYeArray(src, lay))
    mb.synchronize_status(dev)
    assert torch.equal(dst, src)
    print(f"copyto!(tiled_copy, dst, src) for {M} x {N} Float16")


if __name__ == "__main__":
    test_copy_async(2048, 2048)
    test_transpose(2048, 2048)
