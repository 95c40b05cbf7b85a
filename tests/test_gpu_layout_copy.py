"""GPU parity, layout function and copies: the device results must be bit-identical to the
oracle (and to the committed fixtures), through the C ABI."""
import ctypes
import json
import os

import numpy as np
import pytest
import torch

import layout_oracle as lo

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def tt(x):
    return tuple(tt(e) for e in x) if isinstance(x, (list, tuple)) else int(x)


def test_layout_eval_config1_fixture(mb, ho, dev):
    with open(os.path.join(GOLD, "cfg1_layouts.json")) as f:
        cases = json.load(f)["cases"]
    for c in cases:
        L = mb.make_layout(tt(c["shape"]), tt(c["stride"]))
        got = mb.layout_eval(L, device=dev).cpu().numpy()
        assert got.tolist() == c["values"]
        for name, lay in (("coalesce", mb.coalesce(L)), ("logical_divide", mb.logical_divide(
                L, (mb.make_layout(2), mb.make_layout(4), mb.make_layout(4))))):
            vals = mb.layout_eval(lay, device=dev).cpu().numpy().tolist()
            assert vals == (c["values"] if name == "coalesce" else c["logical_divide"]["values"])
        comp = mb.composition(L, mb.make_layout((32, 2), (2, 64)))
        assert mb.layout_eval(comp, device=dev).cpu().numpy().tolist() == c["composition"]["values"]
    mb.synchronize_status(dev)


def test_layout_eval_wraps_like_the_reference(mb, ho, dev):
    # indices past size(layout) wrap in every mode; a single-mode layout does not wrap
    L = mb.make_layout((2, 3), (5, 7))
    got = mb.layout_eval(L, n=18, device=dev).cpu().numpy()
    O = lo.SL((2, 3), (5, 7))
    assert got.tolist() == [int(O(i)) for i in range(1, 19)]
    L1 = mb.make_layout(4, 3)
    assert mb.layout_eval(L1, n=9, first=3, device=dev).cpu().numpy().tolist() == [1 + (i - 1) * 3 for i in range(3, 12)]
    assert ho.layout_eval([4], [3], 3, 9).tolist() == [1 + (i - 1) * 3 for i in range(3, 12)]
    big = mb.make_layout((1 << 20, 1 << 12), (1 << 12, 1))  # 2^32 elements: 64-bit arithmetic
    first = (1 << 32) - 1000
    got = mb.layout_eval(big, n=1000, first=first, device=dev).cpu().numpy()
    assert np.array_equal(got, ho.layout_eval([1 << 20, 1 << 12], [1 << 12, 1], first, 1000))


@pytest.mark.parametrize("elem", [torch.uint8, torch.int16, torch.float32, torch.int64])
def test_layout_copy_matches_oracle(mb, ho, dev, elem):
    """copyto!(dst, src) through two different hierarchical layouts (reference
    src/algorithm/copy.jl:4-16)."""
    src_l = mb.make_layout((8, (4, 2), 16), (1, (16, 8), 64))
    dst_l = mb.make_ordered_layout(((4, 2), 8, 16), ((1, 0), 3, 2))  # a bijection onto 0..1023
    assert sorted(dst_l(i) for i in range(1, 1025)) == list(range(1, 1025))
    n = 1024
    host = torch.from_numpy(ho.rng(5).integers(0, 127, size=n, dtype=np.int64)).to(elem)
    src = host.to(dev)
    dst = torch.zeros(n, dtype=elem, device=dev)
    mb.copyto_(mb.MoYeArray(dst, dst_l), mb.MoYeArray(src, src_l))
    mb.synchronize_status(dev)
    want = np.zeros(n, dtype=host.numpy().dtype)
    ss, sd = src_l.flat()
    ds, dd = dst_l.flat()
    ho.copy_layout(want, ds, dd, host.numpy(), ss, sd)
    assert np.array_equal(dst.cpu().numpy(), want)


def _roundtrip(mb, dev, m, n, mode, dtype=torch.float16, ld_src=None, ld_dst=None, tile=(0, 0), seed=2):
    g = torch.Generator(device="cpu").manual_seed(seed)
    ld_src, ld_dst = ld_src or m, ld_dst or m
    src_host = (torch.rand(n * ld_src, generator=g) * 2 - 1).to(dtype) if dtype.is_floating_point else \
        torch.randint(-100, 100, (n * ld_src,), generator=g).to(dtype)
    src = src_host.to(dev)
    dst = torch.full((n * ld_dst,), 7, dtype=dtype, device=dev)
    lib, h = mb._lib.load(), mb._lib.handle(dev.index)
    ts = mb._lib.make_tensor(src.data_ptr(), mb.TORCH_TO_MOYE[dtype], [m, n], [1, ld_src])
    td = mb._lib.make_tensor(dst.data_ptr(), mb.TORCH_TO_MOYE[dtype], [m, n], [1, ld_dst])
    p = mb._lib.CopyParams(mode, tile[0], tile[1], 0)
    rc = lib.moye_b200_copy(h, ctypes.byref(td), ctypes.byref(ts), ctypes.byref(p), mb.current_stream_ptr(dev))
    return rc, src, dst


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("m,n", [(8192, 8192), (8000, 777), (128, 64), (8, 1), (136, 3), (4096, 1)])
def test_tiled_copy_bit_exact(mb, dev, mode, m, n):
    rc, src, dst = _roundtrip(mb, dev, m, n, mode)
    assert rc == 0, mb._lib.load().moye_b200_last_error()
    mb.synchronize_status(dev)
    assert torch.equal(src, dst)


@pytest.mark.parametrize("mode", [1, 2])
def test_tiled_copy_pitched_views_leave_padding_alone(mb, dev, mode):
    m, n, lds, ldd = 1000 * 8, 65, 8200, 8064
    rc, src, dst = _roundtrip(mb, dev, m, n, mode, ld_src=lds, ld_dst=ldd)
    assert rc == 0
    mb.synchronize_status(dev)
    s = src.view(n, lds)[:, :m]
    d = dst.view(n, ldd)
    assert torch.equal(s, d[:, :m])
    assert bool((d[:, m:] == 7).all()), "the copy wrote outside the destination view"


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("dtype", [torch.int8, torch.float32, torch.int64])
def test_tiled_copy_other_element_sizes(mb, dev, mode, dtype):
    rc, src, dst = _roundtrip(mb, dev, 1024, 96, mode, dtype=dtype)
    assert rc == 0
    mb.synchronize_status(dev)
    assert torch.equal(src, dst)


def test_tiled_copy_matches_reference_copy_kernel(mb, ho, dev):
    """The oracle's emulation of copy_kernel (reference test/host/copy_async.jl:3-25) and the
    device kernels give the same bytes, via the MoYe-level API with a TiledCopy."""
    m, n = 512, 256
    bits = ho.uniform_pm1_f16_bits(2, (m * n,))
    want = np.zeros_like(bits)
    ho.copy_kernel(want, bits, m, n, bm=128, bn=64, tm=16, tn=16)
    src = torch.from_numpy(bits.view(np.int16)).to(dev).view(torch.float16)
    copies = [mb.make_tiled_copy(mb.CopyAtom(op, mb._lib.F16), mb.make_layout((16, 16)), mb.make_layout((8, 1)))
              for op in (mb.UniversalCopy(128), mb.CPOP_ASYNC_CACHEALWAYS(128))]
    copies += [mb.make_tma_tiled_copy(mb._lib.F16, (128, 64)), mb.make_tma_tiled_copy(mb._lib.F16, (64, 32))]
    for tc in copies:
        dst = torch.zeros_like(src)
        mb.copyto_(tc, mb.MoYeArray(dst, mb.make_layout((m, n))), mb.MoYeArray(src, mb.make_layout((m, n))))
        mb.synchronize_status(dev)
        assert np.array_equal(dst.view(torch.int16).cpu().numpy().view(np.uint16), want)
    narrow = mb.make_tiled_copy(mb.CopyAtom(mb.UniversalCopy(16), mb._lib.F16), mb.make_layout((32, 8)))
    with pytest.raises(mb.MoyeError):
        mb.copyto_(narrow, mb.MoYeArray(dst, mb.make_layout((m, n))), mb.MoYeArray(src, mb.make_layout((m, n))))


def test_tma_copy_tiles_of_growing_size_on_one_handle(mb, dev):
    """The kernel's shared-memory limit is raised once per handle: it has to admit every legal tile, whatever tile the
    first call used (a small first tile used to lock later, larger ones out)."""
    for tile in ((64, 16), (128, 32), (128, 64), (256, 16)):
        rc, src, dst = _roundtrip(mb, dev, 1024, 256, 2, tile=tile)
        assert rc == 0, (tile, mb._lib.load().moye_b200_last_error())
        mb.synchronize_status(dev)
        assert torch.equal(src, dst), tile


def _rand(dtype, numel, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    if dtype.is_floating_point:
        return (torch.rand(numel, generator=g) * 2 - 1).to(dtype)
    return torch.randint(-120, 120, (numel,), generator=g).to(dtype)


@pytest.mark.parametrize("dtype", [torch.int8, torch.float16, torch.float32, torch.int64])
@pytest.mark.parametrize("m,n", [(2048, 2048), (1008, 528), (16, 16), (16, 4096), (4096, 16), (8192, 3008)])
def test_transposing_copy_bit_exact(mb, ho, dev, dtype, m, n):
    """`copyto!(dest, transpose(src))` (reference test/host/copy_async.jl:51-74 and :77-95): operands contiguous
    along different modes go through the transposing kernel; bytes must match the oracle's copy through the two
    layouts (checked in full on the small shapes) and torch's transpose."""
    b = _rand(dtype, n * m, 11).to(dev)                  # b: (n, m) column-major, like the reference's `b`
    a = torch.zeros(m * n, dtype=dtype, device=dev)      # a: (m, n) column-major
    A = mb.MoYeArray(a, mb.make_layout((m, n)))
    B = mb.MoYeArray(b, mb.make_layout((n, m)))
    mb.copyto_(A, mb.transpose(B))                       # a == transpose(b)
    mb.synchronize_status(dev)
    assert torch.equal(a.view(n, m), b.view(m, n).t())   # torch views are row-major: a[j][i] = A(i, j)
    if m * n <= 1 << 20:
        want = np.zeros(m * n, dtype=a.cpu().numpy().dtype)
        ho.copy_layout(want, (m, n), (1, m), b.cpu().numpy(), (m, n), (n, 1))
        assert np.array_equal(a.cpu().numpy(), want)
    # the mirrored pair: source column-major, destination row-major
    c = torch.zeros(m * n, dtype=dtype, device=dev)
    mb.copyto_(mb.MoYeArray(c, mb.make_layout((m, n), (n, 1))), A)
    mb.synchronize_status(dev)
    assert torch.equal(c.view(m, n), a.view(n, m).t())
    # both row-major: the plain tiled copy with the modes swapped
    d = torch.zeros(m * n, dtype=dtype, device=dev)
    mb.copyto_(mb.MoYeArray(d, mb.make_layout((m, n), (n, 1))), mb.MoYeArray(c, mb.make_layout((m, n), (n, 1))))
    mb.synchronize_status(dev)
    assert torch.equal(d, c)


def test_transposing_copy_pitched_views_leave_padding_alone(mb, dev):
    m, n, lds, ldd = 1000, 264, 272, 1008              # src rows of 272 elements hold 264; dst columns of 1008 hold 1000
    src = _rand(torch.float32, m * lds, 12).to(dev)
    dst = torch.full((n * ldd,), 7.0, dtype=torch.float32, device=dev)
    S = mb.MoYeArray(src, mb.make_layout((m, n), (lds, 1)))
    D = mb.MoYeArray(dst, mb.make_layout((m, n), (1, ldd)))
    mb.copyto_(D, S)
    mb.synchronize_status(dev)
    d = dst.view(n, ldd)
    assert torch.equal(d[:, :m], src.view(m, lds)[:, :n].t())
    assert bool((d[:, m:] == 7).all()), "the copy wrote outside the destination view"


def test_transposing_copy_errors(mb, dev):
    lib, h = mb._lib.load(), mb._lib.handle(dev.index)
    st = mb.current_stream_ptr(dev)
    buf = torch.zeros(1 << 16, dtype=torch.float16, device=dev)
    T = lambda off, shape, stride: mb._lib.make_tensor(buf.data_ptr() + off, mb._lib.F16, shape, stride)
    p = mb._lib.CopyParams(mb._lib.COPY_TRANSPOSE, 0, 0, 0)
    same = lib.moye_b200_copy(h, ctypes.byref(T(0, [64, 64], [1, 64])), ctypes.byref(T(32768, [64, 64], [1, 64])),
                              ctypes.byref(p), st)
    assert same == -3                                   # both contiguous along the same mode: not a transpose
    odd = lib.moye_b200_copy(h, ctypes.byref(T(0, [64, 60], [1, 64])), ctypes.byref(T(32768, [64, 60], [60, 1])),
                             None, st)
    assert odd == -5                                    # 120-byte source rows
    tiled = mb._lib.CopyParams(mb._lib.COPY_TRANSPOSE, 32, 32, 0)
    assert lib.moye_b200_copy(h, ctypes.byref(T(0, [64, 64], [1, 64])), ctypes.byref(T(32768, [64, 64], [64, 1])),
                              ctypes.byref(tiled), st) == -1
    mb.synchronize_status(dev)


def test_empty_and_invalid_copies(mb, dev):
    lib, h = mb._lib.load(), mb._lib.handle(dev.index)
    st = mb.current_stream_ptr(dev)
    buf = torch.zeros(4096, dtype=torch.float16, device=dev)
    T = lambda ptr, shape, stride, dt=mb._lib.F16: mb._lib.make_tensor(ptr, dt, shape, stride)
    p = mb._lib.CopyParams(0, 0, 0, 0)
    # empty: nothing to do, success
    assert lib.moye_b200_copy(h, ctypes.byref(T(buf.data_ptr(), [0, 8], [1, 64])),
                              ctypes.byref(T(buf.data_ptr(), [0, 8], [1, 64])), ctypes.byref(p), st) == 0
    a, b = T(buf.data_ptr(), [64, 8], [1, 64]), T(buf.data_ptr() + 4096, [64, 8], [1, 64])
    cases = [
        (T(buf.data_ptr() + 2, [64, 8], [1, 64]), a, -5),            # misaligned base
        (T(buf.data_ptr(), [64, 8], [2, 128]), a, -3),              # no unit stride
        (T(buf.data_ptr(), [64, 4], [1, 64]), a, -4),               # shape mismatch
        (T(buf.data_ptr(), [64, 8], [1, 64], mb._lib.BF16), a, -2),  # dtype mismatch
        (T(buf.data_ptr(), [60, 8], [1, 60]), T(buf.data_ptr() + 4096, [60, 8], [1, 60]), -5),  # 120-byte columns
    ]
    for d, s, want in cases:
        assert lib.moye_b200_copy(h, ctypes.byref(d), ctypes.byref(s), ctypes.byref(p), st) == want
        assert lib.moye_b200_last_error()
    bad = mb._lib.CopyParams(1, 24, 0, 0)  # tile_m * 2 bytes = 48 is not 16 * 2^k
    assert lib.moye_b200_copy(h, ctypes.byref(b), ctypes.byref(a), ctypes.byref(bad), st) == -1
    mb.synchronize_status(dev)


@pytest.mark.parametrize("op", ["LDSM_U32x1_N", "LDSM_U32x2_N", "LDSM_U32x4_N"])
def test_ldmatrix_tiled_copy_reference_device_test(mb, dev, op):
    """The reference's own device test of its ldmatrix atoms (test/device/tiled_copy.jl:58-97): iota tiles of UInt16
    through shared memory, `ldmatrix` per thread, registers to global memory; `g_out == g_in`."""
    U16 = mb._lib.U16
    cases = [(mb.make_layout((32, 32), (1, 32)), mb.make_layout((16, 2)), mb.make_layout((2, 4)), 32 * 32),
             (mb.make_layout((32, (2, 4)), (2, (1, 64))), mb.make_layout((32, 1)), mb.make_layout((1, 8)), 32 * 8)]
    for smem_layout, thr, val, n in cases:
        tiled_copy = mb.make_tiled_copy(mb.CopyAtom(mb.ldsm_op(op), U16), thr, val)
        g_in = torch.arange(1, n + 1, dtype=torch.int16, device=dev)
        g_out = torch.zeros(n, dtype=torch.int16, device=dev)
        mb.copyto_(tiled_copy, mb.MoYeArray(g_out, smem_layout), mb.MoYeArray(g_in, smem_layout))
        mb.synchronize_status(dev)
        assert torch.equal(g_out, g_in), (op, smem_layout)
    # fp16 values and four warps: the smem -> register copy of B in the manual's tensor-core kernel
    # (docs/src/manual/tensor_core.md:369-371), 128 threads over one (128, 16) K-major buffer
    if op == "LDSM_U32x4_N":
        mma = mb.make_tiled_mma(mb.mma_op("MMAOP_16x8x16_F32F16F16F32_TN"), mb.make_layout((2, 2, 1), (2, 1, 1)), (32, 32, 16))
        smem_copy_B = mb.make_tiled_copy_B(mb.CopyAtom(mb.ldsm_op(op), mb._lib.F16), mma)
        sB = mb.make_layout((128, 16), (16, 1))
        src = torch.randn(128 * 16, device=dev).half()
        dst = torch.zeros_like(src)
        mb.copyto_(smem_copy_B, mb.MoYeArray(dst, sB), mb.MoYeArray(src, sB))
        mb.synchronize_status(dev)
        assert torch.equal(dst, src)


def test_ldmatrix_tiled_copy_refuses_what_the_instruction_cannot_do(mb, dev):
    U16 = mb._lib.U16
    tiled_copy = mb.make_tiled_copy(mb.CopyAtom(mb.ldsm_op("LDSM_U32x1_N"), U16), mb.make_layout((16, 2)), mb.make_layout((2, 4)))
    buf = torch.zeros(4096, dtype=torch.int16, device=dev)
    with pytest.raises(mb.MoyeError):    # rows of the tile are 2 elements long: no fragment of 8 contiguous values
        mb.copyto_(tiled_copy, mb.MoYeArray(buf, mb.make_layout((32, 32), (32, 1))), mb.MoYeArray(buf, mb.make_layout((32, 32), (32, 1))))
    with pytest.raises(mb.MoyeError):    # different layouts on the two sides
        mb.copyto_(tiled_copy, mb.MoYeArray(buf, mb.make_layout((32, 32), (1, 32))), mb.MoYeArray(buf, mb.make_layout((32, 32), (1, 64))))
    f32 = torch.zeros(1024, device=dev)
    with pytest.raises(mb.MoyeError):    # 32-bit elements
        mb.copyto_(tiled_copy, mb.MoYeArray(f32, mb.make_layout((32, 32))), mb.MoYeArray(f32, mb.make_layout((32, 32))))
