"""The allocation-free decode GEMM entry point (`moye_b200_gemm_skinny_static`).

Some users of the library cannot allocate device memory while they run (a serving loop with
a fixed memory budget, a plugin under a no-allocation rule, code that never made a handle).
For them the stream-K scratch lives in a static device array inside the library.  This file
checks, through the C ABI, that the entry point gives the same result as the handle-based
one on two calls in a row (the array keeps the first call's contents), also when the shape
changes between calls, and that it refuses problems larger than the array.  It is named so
that pytest collects it last.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _operands(ho, M, N, K, dev, dtype=torch.bfloat16):
    x = ho.normal_bf16_bits(9, (M * K,), 0.02)
    w = ho.normal_bf16_bits(10, (N * K,), 0.02)
    X = torch.from_numpy(x.view(np.int16)).to(dev).view(torch.bfloat16).view(M, K)
    W = torch.from_numpy(w.view(np.int16)).to(dev).view(torch.bfloat16).view(N, K)
    if dtype != torch.bfloat16:
        X, W = X.to(dtype), W.to(dtype)
    return X, W


def _static_call(mb, D, A, B, alpha, status, dev):
    """Straight through the C ABI: no handle is passed, nothing is allocated by the call."""
    lib = mb._lib.load()
    T = lambda t: mb._lib.make_tensor(t.data_ptr(), mb.TORCH_TO_MOYE[t.dtype], list(t.shape), list(t.stride()))
    return lib.moye_b200_gemm_skinny_static(ctypes.byref(T(D)), ctypes.byref(T(A)), ctypes.byref(T(B)),
                                            ctypes.c_float(alpha), ctypes.c_void_p(status.data_ptr()),
                                            mb.current_stream_ptr(dev))


@pytest.mark.parametrize("M,N,K,out_dtype", [(16, 4096, 2048, torch.bfloat16), (7, 1000, 1024, torch.float32),
                                             (32, 2048, 4096, torch.bfloat16)])
def test_static_entry_point_matches_handle_entry_point_twice(mb, ho, dev, M, N, K, out_dtype):
    X, W = _operands(ho, M, N, K, dev)
    want = torch.zeros(M, N, dtype=out_dtype, device=dev)
    mb.matmul(X, W, want, path=2, alpha=1.25)          # the existing, handle-based entry point
    mb.synchronize_status(dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    outs = []
    for _ in range(2):                                   # two calls in a row share the static array
        got = torch.full((M, N), float("nan"), dtype=out_dtype, device=dev)
        rc = _static_call(mb, got, X, W, 1.25, status, dev)
        assert rc == 0, mb._lib.load().moye_b200_last_error()
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert ho.max_rel_err(got.float().cpu().numpy(), want.float().cpu().numpy()) <= 1e-2
        outs.append(got)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], want)
    # and against the oracle itself
    ref = ho.gemm_samples(ho.normal_bf16_bits(9, (M * K,), 0.02), ho.normal_bf16_bits(10, (N * K,), 0.02), ho.BF16,
                          M, N, K, np.arange(M, dtype=np.int32), threads=4)
    assert ho.max_rel_err(outs[1].float().cpu().numpy(), 1.25 * ref) <= 1e-2


def test_static_entry_point_with_changing_shapes_and_wrapper(mb, ho, dev):
    """Back-to-back calls with different row-block counts: whatever the previous call left in
    the array must not leak into the next result."""
    for M, N, K in [(16, 8192, 512), (3, 129, 520), (16, 8192, 512), (32, 640, 8192)]:
        X, W = _operands(ho, M, N, K, dev)
        want = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        mb.matmul(X, W, want, path=2)
        got = torch.zeros_like(want)
        mb.gemm_skinny_static_(got, X, W)                # same entry point through the Python wrapper
        torch.cuda.synchronize()
        mb.synchronize_status(dev)
        assert torch.equal(got, want)
    Xh, Wh = _operands(ho, 16, 1024, 1024, dev, torch.float16)
    want = torch.zeros(16, 1024, dtype=torch.float16, device=dev)
    mb.matmul(Xh, Wh, want, path=2)
    got = torch.zeros_like(want)
    mb.gemm_skinny_static_(got, Xh, Wh)
    torch.cuda.synchronize()
    assert torch.equal(got, want)


def test_static_entry_point_rejects_what_does_not_fit(mb, dev):
    lib = mb._lib.load()
    T = mb._lib.make_tensor
    buf = torch.zeros(1 << 20, dtype=torch.bfloat16, device=dev)
    st = mb.current_stream_ptr(dev)
    BF16, F32 = mb._lib.BF16, mb._lib.F32

    def call(M, N, K, a_dt=BF16, d_dt=BF16, a_stride=None):
        A = T(buf.data_ptr(), a_dt, [M, K], a_stride or [K, 1])
        B = T(buf.data_ptr(), a_dt, [N, K], [K, 1])
        D = T(buf.data_ptr(), d_dt, [M, N], [N, 1])
        return lib.moye_b200_gemm_skinny_static(ctypes.byref(D), ctypes.byref(A), ctypes.byref(B), ctypes.c_float(1.0),
                                                None, st)

    assert call(33, 256, 64) == -9 and b"32 rows" in lib.moye_b200_last_error()       # more rows than the scratch holds
    assert call(16, 524288 + 128, 64) == -9 and b"row blocks" in lib.moye_b200_last_error()
    assert call(16, 256, 64, a_dt=F32) == -2                                            # operand type
    assert call(16, 256, 64, d_dt=mb._lib.S32) == -2                                    # output type
    assert call(16, 256, 64, a_stride=[1, 16]) == -3                                    # not K-major
    assert lib.moye_b200_gemm_skinny_static(None, None, None, ctypes.c_float(1.0), None, st) == -1
    torch.cuda.synchronize()
