"""GPU parity of the stand-alone `axpby!` and of the NCCL entry points in a world of one rank, through the C ABI."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1000,), (256, 384), (130, 72), (4096, 2048)])
def test_axpby_bit_exact(mb, ho, dev, dtype, shape):
    """Y = a*X + b*Y against the oracle's restatement of reference src/algorithm/blas.jl:1-9, bit for bit: both
    products rounded to Float32, one add, one rounding to the element type; b == 0 never reads Y (NaNs in it
    must not leak)."""
    n = int(np.prod(shape))
    x32 = ho.uniform_pm1(21, (n,))
    y32 = ho.uniform_pm1(22, (n,))
    X = torch.from_numpy(x32).to(dev).to(dtype).view(*shape)
    Y0 = torch.from_numpy(y32).to(dev).to(dtype).view(*shape)
    xw, yw = X.float().cpu().numpy().ravel(), Y0.float().cpu().numpy().ravel()   # what the device holds, widened (exact)
    for a, b in ((0.75, -1.5), (2.0, 0.0), (1.0, 1.0)):
        Y = Y0.clone() if b != 0.0 else torch.full_like(Y0, float("nan"))
        mb.axpby_(a, X, b, Y)
        mb.synchronize_status(dev)
        want = torch.from_numpy(ho.axpby(a, xw, b, yw)).to(dtype).view(*shape)   # torch's CPU cast rounds to nearest even
        assert torch.equal(Y.cpu(), want), (a, b)


def test_axpby_pitched_views_and_in_place(mb, ho, dev):
    base_x = torch.from_numpy(ho.uniform_pm1(23, (300 * 512,))).to(dev).view(300, 512)
    base_y = torch.from_numpy(ho.uniform_pm1(24, (300 * 640,))).to(dev).view(300, 640)
    X, Y = base_x[:, 8:392], base_y[:, 16:400]                 # pitched rows, 16-byte aligned: the vector kernel
    keep = base_y.clone()
    want = ho.axpby(0.5, X.cpu().numpy(), 2.0, Y.cpu().numpy())
    mb.axpby_(0.5, mb.MoYeArray(X), 2.0, mb.MoYeArray(Y))
    mb.synchronize_status(dev)
    assert np.array_equal(Y.cpu().numpy(), want)
    assert torch.equal(base_y[:, :16], keep[:, :16]) and torch.equal(base_y[:, 400:], keep[:, 400:])   # padding untouched
    X2, Y2 = base_x[:, 3:100], base_y[:, 5:102]                # odd offsets: element by element
    want = ho.axpby(-1.0, X2.cpu().numpy(), 0.25, Y2.cpu().numpy())
    mb.axpby_(-1.0, mb.MoYeArray(X2), 0.25, mb.MoYeArray(Y2))
    mb.synchronize_status(dev)
    assert np.array_equal(Y2.cpu().numpy(), want)
    Z = torch.from_numpy(ho.uniform_pm1(25, (4096,))).to(dev)   # axpby!(a, Z, b, Z) scales in place
    want = ho.axpby(3.0, Z.cpu().numpy(), -1.0, Z.cpu().numpy())
    mb.axpby_(3.0, Z, -1.0, Z)
    mb.synchronize_status(dev)
    assert np.array_equal(Z.cpu().numpy(), want)
    with pytest.raises(mb.MoyeError):
        mb.axpby_(1.0, torch.zeros(8, 4, device=dev), 1.0, torch.zeros(8, 4, device=dev).t().contiguous().t())
    with pytest.raises(mb.MoyeError):
        mb.axpby_(1.0, torch.zeros(8, device=dev), 1.0, torch.zeros(8, device=dev, dtype=torch.float16))


def test_comm_entry_points_in_a_world_of_one(mb, ho, dev):
    """`moye_b200_comm_*`, `moye_b200_allgather`, `moye_b200_bcast` through the C ABI with one rank: the argument
    checks, the block arithmetic and the NCCL calls all run (NCCL copies the single block); the multi-rank
    behaviour of the same arithmetic is covered by the gloo tests and by the benchmark on 2-8 GPUs."""
    lib, h = mb._lib.load(), mb._lib.handle(dev.index)
    st = mb.current_stream_ptr(dev)
    T = lambda t: mb._lib.make_tensor(t.data_ptr(), mb.TORCH_TO_MOYE[t.dtype], list(t.shape), list(t.stride()))
    shard = torch.from_numpy(ho.uniform_pm1(26, (96 * 256,))).to(dev).view(96, 256)
    full = torch.zeros_like(shard)
    assert lib.moye_b200_allgather(h, ctypes.byref(T(shard)), ctypes.byref(T(full)), 0, 1, st) == -1   # no communicator yet
    ident = ctypes.create_string_buffer(128)
    rc = lib.moye_b200_comm_unique_id(ident)
    assert rc == 0, lib.moye_b200_last_error()
    for bad_rank, bad_world in ((1, 1), (-1, 1), (0, 0)):                                       # a rank outside its world
        assert lib.moye_b200_comm_init(h, bad_rank, bad_world, ident.raw) == -1 and b"bad rank" in lib.moye_b200_last_error()
    assert lib.moye_b200_comm_init(None, 0, 1, ident.raw) == -1
    assert lib.moye_b200_comm_init(h, 0, 1, ident.raw) == 0, lib.moye_b200_last_error()
    try:
        assert lib.moye_b200_comm_init(h, 0, 1, ident.raw) == -1                                   # one communicator per handle
        assert lib.moye_b200_allgather(h, ctypes.byref(T(shard)), ctypes.byref(T(full)), 0, 1, st) == 0
        torch.cuda.synchronize()
        assert torch.equal(full, shard)
        cm = shard.t().contiguous().t()                                                            # column-major: split the columns
        fullc = torch.zeros(256, 96, device=dev).t()
        assert lib.moye_b200_allgather(h, ctypes.byref(T(cm)), ctypes.byref(T(fullc)), 1, 1, st) == 0
        torch.cuda.synchronize()
        assert torch.equal(fullc, cm)
        assert lib.moye_b200_allgather(h, ctypes.byref(T(cm)), ctypes.byref(T(fullc)), 0, 1, st) == -3  # rows of a column-major matrix
        assert b"outermost" in lib.moye_b200_last_error()
        assert lib.moye_b200_allgather(h, ctypes.byref(T(shard[:50])), ctypes.byref(T(full)), 0, 1, st) == -4
        assert lib.moye_b200_bcast(h, ctypes.byref(T(full)), 0, st) == 0
        assert lib.moye_b200_bcast(h, ctypes.byref(T(full)), 1, st) == -1
        assert lib.moye_b200_bcast(h, ctypes.byref(T(full[:, :100])), 0, st) == -3
        torch.cuda.synchronize()
        assert torch.equal(full, shard)
    finally:
        assert lib.moye_b200_comm_destroy(h) == 0
    assert lib.moye_b200_comm_destroy(h) == 0
