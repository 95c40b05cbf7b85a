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


def test_static_entry_point_allocates_nothing(mb, ho, dev):
    """The contract in its name: device memory before and after a call is the same to the byte (operands, output
    and the first-call set-up are done beforehand)."""
    M, N, K = 16, 4096, 2048
    X, W = _operands(ho, M, N, K, dev)
    got = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    assert _static_call(mb, got, X, W, 1.0, status, dev) == 0     # warm-up: the once-per-device set-up happens here
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info(dev)
    for _ in range(3):
        assert _static_call(mb, got, X, W, 1.0, status, dev) == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info(dev)
    assert free1 == free0
    # the status word kept inside the array (device_status == NULL) can be read back without allocating either
    lib = mb._lib.load()
    T = lambda t: mb._lib.make_tensor(t.data_ptr(), mb.TORCH_TO_MOYE[t.dtype], list(t.shape), list(t.stride()))
    assert lib.moye_b200_gemm_skinny_static(ctypes.byref(T(got)), ctypes.byref(T(X)), ctypes.byref(T(W)),
                                            ctypes.c_float(1.0), None, mb.current_stream_ptr(dev)) == 0
    site = ctypes.c_int32(-1)
    assert lib.moye_b200_gemm_skinny_static_status(mb.current_stream_ptr(dev), ctypes.byref(site)) == 0 and site.value == 0
    mb.gemm_skinny_static_status(dev)
    free2, _ = torch.cuda.mem_get_info(dev)
    assert free2 == free0


_NO_HANDLE_SCRIPT = r"""
import ctypes, sys
import numpy as np
import torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/oracle")
import __graft_entry__ as ge
import host_oracle as ho
mb = ge.load_package()
lib = mb._lib.load()
dev = torch.device("cuda", 0)
torch.cuda.set_device(dev)
M, N, K = 16, 1024, 1024
x, w = ho.normal_bf16_bits(9, (M * K,), 0.02), ho.normal_bf16_bits(10, (N * K,), 0.02)
X = torch.from_numpy(x.view(np.int16)).to(dev).view(torch.bfloat16).view(M, K)
W = torch.from_numpy(w.view(np.int16)).to(dev).view(torch.bfloat16).view(N, K)
Y = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
T = lambda t: mb._lib.make_tensor(t.data_ptr(), mb.TORCH_TO_MOYE[t.dtype], list(t.shape), list(t.stride()))
st = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
for _ in range(2):
    rc = lib.moye_b200_gemm_skinny_static(ctypes.byref(T(Y)), ctypes.byref(T(X)), ctypes.byref(T(W)), ctypes.c_float(1.0), None, st)
    assert rc == 0, lib.moye_b200_last_error()
site = ctypes.c_int32(-1)
assert lib.moye_b200_gemm_skinny_static_status(st, ctypes.byref(site)) == 0 and site.value == 0
assert not mb._lib._handles, "a handle was created"
ref = ho.gemm_samples(x, w, ho.BF16, M, N, K, np.arange(M, dtype=np.int32), threads=4)
err = ho.max_rel_err(Y.float().cpu().numpy(), ref)
assert err <= 1e-2, err
print("NO_HANDLE_OK")
"""


def test_static_entry_point_needs_no_handle(dev):
    """A fresh process that loads the library and calls only the static entry point -- `moye_b200_create` never
    runs -- gets the oracle's result."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-c", _NO_HANDLE_SCRIPT, root], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "NO_HANDLE_OK" in res.stdout, res.stdout + res.stderr
