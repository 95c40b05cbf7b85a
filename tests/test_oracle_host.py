"""Pins the C oracle (oracle/moye_host.c): scalar codecs against torch's CPU conversions,
the literal UniversalFMA known answers, the reference's bit-exact copy goldens
(test/copy.jl), agreement of the three host GEMM forms, and the committed fixtures."""
import json
import os

import numpy as np
import pytest
import torch

import layout_oracle as lo

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def bits16(t):
    return t.view(torch.int16).numpy().view(np.uint16)


def test_half_and_bf16_codecs_match_torch(ho):
    x = np.concatenate([ho.uniform_pm1(0, (20000,)) * s for s in (1.0, 500.0, 7e4, 1e-4, 6e-8)]).astype(np.float32)
    x = np.concatenate([x, np.array([0.0, -0.0, 65504.0, 65520.0, 65519.9, np.inf, -np.inf], dtype=np.float32)])
    assert np.array_equal(ho.float_to_half(x), bits16(torch.from_numpy(x).half()))
    assert np.array_equal(ho.float_to_bf16(x), bits16(torch.from_numpy(x).bfloat16()))
    allh = np.arange(65536, dtype=np.uint16)
    ref = torch.from_numpy(allh.view(np.int16)).view(torch.float16).float().numpy()
    got = ho.half_to_float(allh)
    ok = ~np.isnan(ref)
    assert np.array_equal(got[ok], ref[ok]) and np.isnan(got[~ok]).all()
    refb = torch.from_numpy(allh.view(np.int16)).view(torch.bfloat16).float().numpy()
    gotb = ho.bf16_to_float(allh)
    ok = ~np.isnan(refb)
    assert np.array_equal(gotb[ok], refb[ok])


@pytest.mark.skipif(not hasattr(torch, "float8_e4m3fn"), reason="torch without fp8")
def test_e4m3_codec_matches_torch(ho):
    allb = np.arange(256, dtype=np.uint8)
    ref = torch.from_numpy(allb).view(torch.float8_e4m3fn).float().numpy()
    got = ho.e4m3_to_float(allb)
    ok = ~np.isnan(ref)
    assert np.array_equal(got[ok], ref[ok]) and np.isnan(got[~ok]).all()
    x = np.concatenate([ho.uniform_pm1(1, (50000,)) * s for s in (1.0, 0.05, 448.0, 2e-3)]).astype(np.float32)
    x = np.clip(x, -448, 448)
    assert np.array_equal(ho.float_to_e4m3(x), torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    # saturation instead of NaN/inf ("satfinite")
    big = np.array([1e6, -1e6, 449.0, 464.0, 480.0], dtype=np.float32)
    assert np.array_equal(ho.float_to_e4m3(big), np.array([0x7e, 0xfe, 0x7e, 0x7e, 0x7e], dtype=np.uint8))
    # every representable value round-trips
    finite = allb[ok]
    assert np.array_equal(ho.float_to_e4m3(ho.e4m3_to_float(finite)) & 0x7f, finite & 0x7f)


def test_universal_fma_literal_semantics(ho):
    # Int8(100)*Int8(100) wraps to 16 before widening (reference src/arch/mma/mma.jl:64 with
    # Julia's promote_type(Int8,Int8) == Int8); the widened form gives 10000
    assert ho.fma_literal_s8(100, 100, 0) == 16
    assert ho.fma_literal_s8(-128, -128, 5) == 5  # 16384 mod 256 == 0
    a = np.array([100], dtype=np.int8)
    assert ho.gemm_samples(a, a, ho.S8, 1, 1, 1, np.array([0]))[0, 0] == 10000
    # Float16 product rounds to Float16 first: 0.1h * 0.1h
    h = ho.float_to_half(np.array([0.1], dtype=np.float32))
    lit = ho.fma_literal_f16(int(h[0]), int(h[0]), 0.0)
    wide = float(ho.half_to_float(h)[0]) ** 2
    assert lit != np.float32(wide)
    assert lit == float(ho.half_to_float(ho.float_to_half(np.array([wide], dtype=np.float32)))[0])


def test_copy_goldens_sequential_and_parallelized(ho):
    # test/copy.jl:8-19 and :55-66: y == x after copyto!(y, x) on (4,2) Int32 arrays
    a = np.arange(1, 9, dtype=np.int32)
    b = np.arange(9, 17, dtype=np.int32)
    ho.copy_layout(b, [4, 2], [1, 4], a, [4, 2], [1, 4])
    assert np.array_equal(a, b)
    # test/copy.jl:23-49 and :71-98: 6x6 Int32, thread layout (2,3), each thread copies its partition
    a_data = np.arange(1, 37, dtype=np.int32)
    b_data = np.arange(37, 73, dtype=np.int32)
    thread_layout = lo.SL((2, 3))
    for static_layout in (False, True):
        layout = lo.SL((6, 6)) if static_layout else lo.make_layout((6, 6))
        b_work = b_data.copy()
        va, vb = lo.make_view(a_data, layout), lo.make_view(b_work, layout)
        for i in range(1, 7):
            ta = lo.local_partition(va, thread_layout, i)
            tb = lo.local_partition(vb, thread_layout, i)
            assert int(lo.size(ta.layout)) == 6
            lo.copyto(tb, ta)
        assert np.array_equal(b_work, a_data)


def test_copy_kernel_emulation_is_exact(ho):
    # test/host/copy_async.jl:27-48 at reduced size: (32,32) block tile, (32,8) threads
    m, n = 256, 128
    src = ho.rng(3).integers(0, 2 ** 31 - 1, size=m * n, dtype=np.int32)
    dst = np.zeros_like(src)
    ho.copy_kernel(dst, src, m, n, bm=32, bn=32, tm=32, tn=8)
    assert np.array_equal(src, dst)
    with pytest.raises(ValueError):
        ho.copy_kernel(dst, src, m, n, bm=48, bn=32, tm=32, tn=8)


def test_host_gemm_forms_agree_at_config1(ho):
    # tower (test/device/matmul.jl), explicit loop nest (examples/gemm.jl), plain triple loop and
    # the threaded host GEMM (test/host/tiling_matmul.jl) give bit-identical C
    M = N = K = 256
    A, B = ho.uniform_pm1(0, (M * K,)), ho.uniform_pm1(1, (N * K,))
    seq = ho.gemm_f32(A, (1, M), B, (1, N), M, N, K)
    tower = ho.matmul_kernel_f32(A, B, M, N, K, tA=(32, 8), tC=(16, 16), use_tower=True)
    loops = ho.matmul_kernel_f32(A, B, M, N, K, tA=(32, 8), tC=(32, 8), use_tower=False)
    threads = ho.matmul_threads_f32(A, B, M, N, K, thread_layout=(4, 4))
    assert np.array_equal(seq, tower) and np.array_equal(seq, loops) and np.array_equal(seq, threads)
    f64 = ho.gemm_f64(A.astype(np.float64), (1, M), B.astype(np.float64), (1, N), M, N, K)
    assert ho.max_rel_err(seq, f64) < 1e-3  # "C ≈ A*B'" of test/host/tiling_matmul.jl:41
    gold = np.load(os.path.join(GOLD, "cfg1_host_gemm_f32_256.npz"))["C"]
    assert np.array_equal(seq.reshape(N, M).T, gold)


def test_widened_samples_match_float_forms(ho):
    g = np.load(os.path.join(GOLD, "small_gemm_goldens.npz"))
    m, n, k = 64, 48, 128
    a = ho.half_to_float(g["f16_a"])
    b = ho.half_to_float(g["f16_b"])
    seq = ho.gemm_f32(a, (k, 1), b, (k, 1), m, n, k, c_strides=(n, 1)).reshape(m, n)
    assert np.array_equal(seq, g["f16_c"])
    rows = ho.gemm_samples(g["f16_a"], g["f16_b"], ho.F16, m, n, k, np.arange(m, dtype=np.int32), threads=3)
    cols = ho.gemm_samples(g["f16_a"], g["f16_b"], ho.F16, m, n, k, np.arange(n, dtype=np.int32), by_rows=False)
    assert np.array_equal(rows, g["f16_c"]) and np.array_equal(cols.T, g["f16_c"])
    ai, bi = g["s8_a"].astype(np.int32), g["s8_b"].astype(np.int32)
    assert np.array_equal(ho.gemm_s32(ai, (k, 1), bi, (k, 1), m, n, k, c_strides=(n, 1)).reshape(m, n), g["s8_c"])
    assert np.array_equal((ai.reshape(m, k).astype(np.int64) @ bi.reshape(n, k).astype(np.int64).T), g["s8_c"])
    for key, dt in (("e4m3", ho.E4M3), ("bf16", ho.BF16)):
        mm = 16 if key == "bf16" else m
        got = ho.gemm_samples(g[key + "_a"], g[key + "_b"], dt, mm, n, k, np.arange(mm, dtype=np.int32))
        assert np.array_equal(got, g[key + "_c"])


def test_layout_fixture_matches_oracle(ho):
    with open(os.path.join(GOLD, "cfg1_layouts.json")) as f:
        cases = json.load(f)["cases"]

    def tt(x):
        return tuple(tt(e) for e in x) if isinstance(x, list) else x

    for c in cases:
        L = lo.SL(tt(c["shape"]), tt(c["stride"]))
        vals = [int(L(i)) for i in range(1, 1025)]
        assert vals == c["values"]
        fs, fd = lo.flatten(L.shape), lo.flatten(L.stride)
        assert ho.layout_eval(fs, fd, 1, 1024).tolist() == vals  # the C evaluator agrees with the Python one
        co = lo.coalesce(L)
        assert [int(co(i)) for i in range(1, 1025)] == vals
        comp = lo.composition(L, lo.SL((32, 2), (2, 64)))
        assert [int(comp(i)) for i in range(1, 65)] == c["composition"]["values"]
        rhs = lo.SL((32, 2), (2, 64))
        assert all(int(comp(i)) == int(L(rhs(i))) for i in range(1, 65))
        div = lo.logical_divide(L, (lo.SL(2), lo.SL(4), lo.SL(4)))
        assert [int(div(i)) for i in range(1, 1025)] == c["logical_divide"]["values"]
