"""GPU parity of the tcgen05 GEMMs against the widened-input host gemm! of the oracle,
through the C ABI.  Tolerances are the ones the configurations state: int8 bit-exact;
fp16/bf16 max relative error <= 1e-2; e4m3 <= 3e-2 (metric: host_oracle.max_rel_err)."""
import ctypes
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
NTHREADS = max(1, min(64, os.cpu_count() or 1))
TOL = {"f16": 1e-2, "bf16": 1e-2, "e4m3": 3e-2, "f32": 1e-2}  # "f32" here: ONE tf32 product (allow_tf32), 10-bit mantissas


def f32_as_accurate_as_host(ho, got, host32, exact64):
    """Float32 operands without allow_tf32 (three tf32 products of high and low parts).  No device product can equal
    the host's sequential-k Float32 `gemm!` bit for bit (a different summation order alone moves the test metric by
    3e-4 at K = 1024: that is the host's own distance from the exact product), so the bar is accuracy.  Largest
    absolute error over largest |C|, against the exact (float64) product: within 4x of what the host's Float32
    `gemm!` achieves.  And in the metric of every GEMM test the device agrees with the host to 2e-3, where ONE tf32
    product is off by 1e-1 and more."""
    got, host32, exact64 = (np.asarray(x, dtype=np.float64) for x in (got, host32, exact64))
    scale = np.abs(exact64).max()
    e_dev, e_host = np.abs(got - exact64).max() / scale, np.abs(host32 - exact64).max() / scale
    assert e_dev <= 4.0 * e_host + 1e-7, (e_dev, e_host)
    assert ho.max_rel_err(got, host32) <= 2e-3


def kw_of(kind):
    """Float32 operands are compared with the oracle on tf32-truncated operands: ask for the single tf32 product."""
    return {"allow_tf32": True} if kind == "f32" else {}


def dev_bits(bits, dtype, shape, dev):
    t = torch.from_numpy(bits.view(np.int16) if bits.dtype == np.uint16 else bits).to(dev)
    return t.view(dtype).view(*shape)


def operands(ho, kind, M, N, K, dev, seeds):
    if kind == "f16":
        a, b = ho.uniform_pm1_f16_bits(seeds[0], (M * K,)), ho.uniform_pm1_f16_bits(seeds[1], (N * K,))
        return a, b, dev_bits(a, torch.float16, (M, K), dev), dev_bits(b, torch.float16, (N, K), dev), ho.F16
    if kind == "bf16":
        a, b = ho.normal_bf16_bits(seeds[0], (M * K,), 0.02), ho.normal_bf16_bits(seeds[1], (N * K,), 0.02)
        return a, b, dev_bits(a, torch.bfloat16, (M, K), dev), dev_bits(b, torch.bfloat16, (N, K), dev), ho.BF16
    if kind == "f32":
        # the device gets the raw Float32 values; the oracle gets them as the tf32 kind reads them (low 13 bits dropped)
        a, b = ho.uniform_pm1(seeds[0], (M * K,)), ho.uniform_pm1(seeds[1], (N * K,))
        return (ho.tf32_trunc(a), ho.tf32_trunc(b), torch.from_numpy(a).to(dev).view(M, K),
                torch.from_numpy(b).to(dev).view(N, K), ho.F32)
    if kind == "s8":
        a, b = ho.uniform_s8(seeds[0], (M * K,)), ho.uniform_s8(seeds[1], (N * K,))
        return a, b, torch.from_numpy(a).to(dev).view(M, K), torch.from_numpy(b).to(dev).view(N, K), ho.S8
    a, b = ho.normal_e4m3_bits(seeds[0], (M * K,)), ho.normal_e4m3_bits(seeds[1], (N * K,))
    return (a, b, torch.from_numpy(a).to(dev).view(torch.float8_e4m3fn).view(M, K),
            torch.from_numpy(b).to(dev).view(torch.float8_e4m3fn).view(N, K), ho.E4M3)


def out_tensor(M, N, dtype, dev, m_major):
    return torch.zeros(N, M, dtype=dtype, device=dev).t() if m_major else torch.zeros(M, N, dtype=dtype, device=dev)


def test_small_goldens_all_dtypes(mb, ho, dev):
    """The committed fixtures: raw operand bits -> widened host gemm! result."""
    g = np.load(os.path.join(GOLD, "small_gemm_goldens.npz"))
    m, n, k = 64, 48, 128
    A = dev_bits(g["f16_a"], torch.float16, (m, k), dev)
    B = dev_bits(g["f16_b"], torch.float16, (n, k), dev)
    for m_major in (False, True):
        C = out_tensor(m, n, torch.float32, dev, m_major)
        mb.matmul(A, B, C)
        mb.synchronize_status(dev)
        assert ho.max_rel_err(C.cpu().numpy(), g["f16_c"]) <= 1e-2
    A8 = torch.from_numpy(g["s8_a"]).to(dev).view(m, k)
    B8 = torch.from_numpy(g["s8_b"]).to(dev).view(n, k)
    for m_major in (False, True):
        C8 = out_tensor(m, n, torch.int32, dev, m_major)
        mb.matmul(A8, B8, C8)
        mb.synchronize_status(dev)
        assert np.array_equal(C8.cpu().numpy(), g["s8_c"])
    Ae = torch.from_numpy(g["e4m3_a"]).to(dev).view(torch.float8_e4m3fn).view(m, k)
    Be = torch.from_numpy(g["e4m3_b"]).to(dev).view(torch.float8_e4m3fn).view(n, k)
    Ce = torch.zeros(m, n, dtype=torch.bfloat16, device=dev)
    mb.matmul(Ae, Be, Ce, scale_a=0.05, scale_b=0.02)
    mb.synchronize_status(dev)
    assert ho.max_rel_err(Ce.float().cpu().numpy(), g["e4m3_c"] * np.float32(0.05 * 0.02)) <= 3e-2
    Ab = dev_bits(g["bf16_a"], torch.bfloat16, (16, k), dev)
    Bb = dev_bits(g["bf16_b"], torch.bfloat16, (n, k), dev)
    for path in (1, 2):
        Cb = torch.zeros(16, n, dtype=torch.bfloat16, device=dev)
        mb.matmul(Ab, Bb, Cb, path=path)
        mb.synchronize_status(dev)
        assert ho.max_rel_err(Cb.float().cpu().numpy(), g["bf16_c"]) <= 1e-2


@pytest.mark.parametrize("kind", ["f16", "bf16", "s8", "e4m3", "f32"])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 1024), (384, 520, 1008), (1, 8, 16), (130, 72, 4096),
                                   (1024, 1024, 512), (520, 1040, 2000)])
def test_gemm_full_oracle(mb, ho, dev, kind, M, N, K):
    """Whole C against the oracle, ragged edges included, for every tile width and both
    output majors."""
    a, b, A, B, dt = operands(ho, kind, M, N, K, dev, (3, 4))
    ref = ho.gemm_samples(a, b, dt, M, N, K, np.arange(M, dtype=np.int32), threads=NTHREADS)
    out_dtype = {"f16": torch.float32, "bf16": torch.float32, "s8": torch.int32, "e4m3": torch.bfloat16,
                 "f32": torch.float32}[kind]
    if kind == "e4m3" and N % 8:
        pytest.skip("bf16 rows of D must be 16-byte multiples")
    for m_major in (False, True):
        if m_major and (M * torch.empty(0, dtype=out_dtype).element_size()) % 16:
            continue
        # 1 single CTAs, 3 CTA pairs, 4 pairs on 256x512 tiles (with and without the stream-K tail), 5 split-K on
        # clusters of 2 / 4 / 8 CTAs (K = 64 or 16 gives cluster ranks without any K block), 0 the library's choice
        for path, tile_n, extra in ((1, 0, {}), (1, 64, {}), (1, 128, {}), (1, 256, {}), (3, 128, {}), (3, 256, {}),
                                    (4, 0, {"tail": False}), (4, 0, {"tail": True}), (0, 0, {}),
                                    (5, 0, {"split_k": 2}), (5, 128, {"split_k": 4}), (5, 256, {"split_k": 8}),
                                    (5, 0, {})):
            C = out_tensor(M, N, out_dtype, dev, m_major)
            mb.matmul(A, B, C, tile_n=tile_n, path=path, **extra, **kw_of(kind))
            mb.synchronize_status(dev)
            got = C.float().cpu().numpy() if kind != "s8" else C.cpu().numpy()
            if kind == "s8":
                assert np.array_equal(got, ref), (m_major, path, tile_n, extra)
            else:
                assert ho.max_rel_err(got, ref) <= TOL[kind], (m_major, path, tile_n, extra)


def col_major(t):
    """Same values, stride 1 along the first mode (MoYe's column-major default)."""
    return t.t().contiguous().t()


@pytest.mark.parametrize("kind", ["f16", "bf16", "f32", "s8", "e4m3"])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 1024), (384, 528, 1008), (144, 80, 4096), (2048, 1024, 512)])
def test_gemm_mn_major_operands(mb, ho, dev, kind, M, N, K):
    """A and / or B stored column-major, i.e. MN-major as in reference examples/gemm.jl:92-93
    (A = randn(M, K), B = randn(N, K) in Julia), on both dense kernels."""
    a, b, A, B, dt = operands(ho, kind, M, N, K, dev, (3, 4))
    ref = ho.gemm_samples(a, b, dt, M, N, K, np.arange(M, dtype=np.int32), threads=NTHREADS)
    for a_mn, b_mn in ((True, True), (True, False), (False, True)):
        Ax = col_major(A) if a_mn else A
        Bx = col_major(B) if b_mn else B
        assert Ax.stride() == ((1, M) if a_mn else (K, 1))
        for path in (1, 3, 4):
            for m_major in (False, True):
                C = out_tensor(M, N, torch.int32 if kind == "s8" else torch.float32, dev, m_major)
                mb.matmul(Ax, Bx, C, path=path, **kw_of(kind), **({"tail": True} if path == 4 else {}))
                mb.synchronize_status(dev)
                if kind == "s8":
                    assert np.array_equal(C.cpu().numpy(), ref), (a_mn, b_mn, path, m_major)
                else:
                    assert ho.max_rel_err(C.cpu().numpy(), ref) <= TOL[kind], (a_mn, b_mn, path, m_major)


def test_examples_gemm_jl_storage(mb, ho, dev):
    """The reference example end to end in its own storage: column-major A (M,K), B (N,K), C (M,N)
    built as MoYeArrays over flat buffers, C = A * B' (reference examples/gemm.jl:66-100)."""
    M, N, K = 2048, 2048, 256
    a_bits, b_bits = ho.uniform_pm1_f16_bits(3, (M * K,)), ho.uniform_pm1_f16_bits(4, (N * K,))   # column-major buffers
    A = mb.MoYeArray(dev_bits(a_bits, torch.float16, (M * K,), dev), mb.make_layout((M, K)))
    B = mb.MoYeArray(dev_bits(b_bits, torch.float16, (N * K,), dev), mb.make_layout((N, K)))
    Cbuf = torch.zeros(M * N, device=dev)
    C = mb.MoYeArray(Cbuf, mb.make_layout((M, N)))
    mb.matmul(A, B, C)
    mb.synchronize_status(dev)
    a32 = ho.half_to_float(a_bits)
    b32 = ho.half_to_float(b_bits)
    rows = np.arange(0, M, 16)
    want = np.stack([ho.gemm_f32(a32[r::M].copy(), (0, 1), b32, (1, N), 1, N, K, c_strides=(N, 1)) for r in rows])
    got = Cbuf.view(N, M).t()[torch.from_numpy(rows).to(dev)].cpu().numpy()
    assert ho.max_rel_err(got, want) <= 1e-2


def test_examples_gemm_jl_float32(mb, ho, dev):
    """The reference example with its own element type and sizes: Float32, 2048 x 2048 x 256, column-major
    (reference examples/gemm.jl:91-96).  Float32 operands run on the tf32 tensor-core kind, which drops the low
    13 mantissa bits of every operand: against the oracle on those truncated operands the result agrees like
    every other float kind; against the fp32 host gemm! on the raw operands it is within 2^-9 sum|a||b| (2^-10 per operand)."""
    M, N, K = 2048, 2048, 256
    a, b = ho.rng(3).standard_normal(M * K, dtype=np.float32), ho.rng(4).standard_normal(N * K, dtype=np.float32)
    A = mb.MoYeArray(torch.from_numpy(a).to(dev), mb.make_layout((M, K)))
    B = mb.MoYeArray(torch.from_numpy(b).to(dev), mb.make_layout((N, K)))
    Cbuf = torch.zeros(M * N, device=dev)
    mb.matmul(A, B, mb.MoYeArray(Cbuf, mb.make_layout((M, N))), allow_tf32=True)
    mb.synchronize_status(dev)
    got = Cbuf.cpu().numpy()
    want = ho.gemm_f32(ho.tf32_trunc(a), (1, M), ho.tf32_trunc(b), (1, N), M, N, K)   # host gemm!, column-major, tf32 view
    assert ho.max_rel_err(got, want) <= TOL["f32"]
    raw = ho.gemm_f32(a, (1, M), b, (1, N), M, N, K)                                    # host gemm! on the raw Float32
    bound = ho.gemm_f32(np.abs(a), (1, M), np.abs(b), (1, N), M, N, K)
    assert np.all(np.abs(got - raw) <= 2.0 ** -9 * bound)
    # the default for Float32 operands: three tf32 products of high and low parts, Float32 accuracy
    Cbuf.zero_()
    mb.matmul(A, B, mb.MoYeArray(Cbuf, mb.make_layout((M, N))))
    mb.synchronize_status(dev)
    exact = ho.gemm_f64(a.astype(np.float64), (1, M), b.astype(np.float64), (1, N), M, N, K)
    f32_as_accurate_as_host(ho, Cbuf.cpu().numpy(), raw, exact)


def test_config1_fp32_against_committed_golden(mb, ho, dev):
    """Configuration 1 as the reference runs it on its host path (256 x 256 x 256 Float32, column-major, seeds 0 / 1;
    test/host/tiling_matmul.jl:20-41), on the device: within the tf32 input truncation of the committed fp32 golden,
    and like every float kind against the oracle on the truncated operands."""
    M = N = K = 256
    a, b = ho.uniform_pm1(0, (M * K,)), ho.uniform_pm1(1, (N * K,))
    gold = np.load(os.path.join(GOLD, "cfg1_host_gemm_f32_256.npz"))["C"]          # (M, N), fp32 sequential-k host gemm!
    A = mb.MoYeArray(torch.from_numpy(a).to(dev), mb.make_layout((M, K)))
    B = mb.MoYeArray(torch.from_numpy(b).to(dev), mb.make_layout((N, K)))
    for path in (1, 3, 0):
        cbuf = torch.zeros(M * N, device=dev)
        mb.matmul(A, B, mb.MoYeArray(cbuf, mb.make_layout((M, N))), path=path, allow_tf32=True)
        mb.synchronize_status(dev)
        got = cbuf.cpu().numpy().reshape(N, M).T
        bound = ho.gemm_f32(np.abs(a), (1, M), np.abs(b), (1, N), M, N, K).reshape(N, M).T
        assert np.all(np.abs(got - gold) <= 2.0 ** -9 * bound), path
        want = ho.gemm_f32(ho.tf32_trunc(a), (1, M), ho.tf32_trunc(b), (1, N), M, N, K).reshape(N, M).T
        assert ho.max_rel_err(got, want) <= TOL["f32"], path
        # Float32 accuracy (the default): as close to the exact product as the committed Float32 golden is
        cbuf.zero_()
        mb.matmul(A, B, mb.MoYeArray(cbuf, mb.make_layout((M, N))), path=path)
        mb.synchronize_status(dev)
        exact = ho.gemm_f64(a.astype(np.float64), (1, M), b.astype(np.float64), (1, N), M, N, K).reshape(N, M).T
        f32_as_accurate_as_host(ho, cbuf.cpu().numpy().reshape(N, M).T, gold, exact)


def test_alpha_beta_and_low_precision_outputs(mb, ho, dev):
    M, N, K = 256, 384, 512
    a, b, A, B, dt = operands(ho, "f16", M, N, K, dev, (3, 4))
    ref = ho.gemm_samples(a, b, dt, M, N, K, np.arange(M, dtype=np.int32), threads=NTHREADS)
    Cin = torch.randn(M, N, device=dev)
    D = torch.zeros(M, N, device=dev)
    mb.gemm_(mb.MoYeArray(D), mb.MoYeArray(A), mb.MoYeArray(B), mb.MoYeArray(Cin), alpha=0.5, beta=2.0)
    mb.synchronize_status(dev)
    assert ho.max_rel_err(D.cpu().numpy(), 0.5 * ref + 2.0 * Cin.cpu().numpy()) <= 1e-2
    # in place: gemm!(A, B, C) is gemm!(C, A, B, C) (reference src/algorithm/blas.jl:11)
    C = Cin.clone()
    mb.gemm_(mb.MoYeArray(A), mb.MoYeArray(B), mb.MoYeArray(C), beta=1.0)
    mb.synchronize_status(dev)
    assert ho.max_rel_err(C.cpu().numpy(), ref + Cin.cpu().numpy()) <= 1e-2
    H = torch.zeros(M, N, device=dev, dtype=torch.float16)
    mb.matmul(A, B, H)
    mb.synchronize_status(dev)
    assert ho.max_rel_err(H.float().cpu().numpy(), ref) <= 1e-2
    # s8 with beta = 1 stays exact
    a8, b8, A8, B8, _ = operands(ho, "s8", M, N, K, dev, (5, 6))
    ref8 = ho.gemm_samples(a8, b8, ho.S8, M, N, K, np.arange(M, dtype=np.int32), threads=NTHREADS)
    C8 = torch.randint(-1000, 1000, (M, N), device=dev, dtype=torch.int32)
    keep = C8.clone()
    mb.gemm_(mb.MoYeArray(A8), mb.MoYeArray(B8), mb.MoYeArray(C8), beta=1.0)
    mb.synchronize_status(dev)
    assert np.array_equal(C8.cpu().numpy(), ref8 + keep.cpu().numpy())


@pytest.mark.parametrize("kind,out", [("f16", torch.float32), ("bf16", torch.bfloat16), ("e4m3", torch.bfloat16),
                                      ("f32", torch.float32)])
def test_fused_bias_activation_epilogue(mb, ho, dev, kind, out):
    """D = act(alpha*A.B^T + beta*C + bias) in one launch, against the oracle's `fused_epilogue` on the oracle's
    accumulator: both bias directions, the three activations, ragged edges, both output majors, every dense path."""
    M, N, K = 384, 520, 1008
    a, b, A, B, dt = operands(ho, kind, M, N, K, dev, (3, 4))
    acc = ho.gemm_samples(a, b, dt, M, N, K, np.arange(M, dtype=np.int32), threads=NTHREADS)
    sc = float(np.abs(acc).max())
    bcol = ho.rng(31).standard_normal(N).astype(np.float32) * np.float32(0.5 * sc)
    brow = ho.rng(32).standard_normal(M).astype(np.float32) * np.float32(0.5 * sc)
    cin = (ho.rng(33).standard_normal((M, N)).astype(np.float32) * np.float32(0.3 * sc))
    Bc, Br = torch.from_numpy(bcol).to(dev), torch.from_numpy(brow).to(dev)
    tol = {torch.float32: TOL[kind], torch.bfloat16: max(TOL[kind], 1e-2)}[out]
    cases = [(1, 256, False, "col", "relu", 0.0), (1, 64, True, "row", "gelu", 0.0), (3, 256, False, "row", "silu", 0.5),
             (3, 128, True, "col", None, 0.0), (4, 0, False, "col", "gelu", 0.0), (4, 0, True, "row", "relu", 1.0),
             (0, 0, False, None, "silu", 0.0), (0, 0, False, "col", None, 2.0), (5, 0, False, "col", "gelu", 0.5),
             (5, 128, True, "row", "relu", 0.0)]
    for path, tile_n, m_major, which, act, beta in cases:
        if m_major and (M * torch.empty(0, dtype=out).element_size()) % 16:
            continue
        alpha = 1.0 / sc                                   # brings x to O(1), where the activations bend
        bias = {None: None, "col": bcol * np.float32(alpha), "row": brow * np.float32(alpha)}[which]
        Cin = torch.from_numpy(cin * np.float32(alpha)).to(dev).to(out)
        if m_major:
            Cin = Cin.t().contiguous().t()
        D = out_tensor(M, N, out, dev, m_major)
        tb = None if which is None else ((Bc if which == "col" else Br) * alpha).contiguous()
        mb.gemm_(mb.MoYeArray(D), mb.MoYeArray(A), mb.MoYeArray(B), mb.MoYeArray(Cin) if beta else None, alpha=alpha,
                 beta=beta, tile_n=tile_n, path=path, bias=tb, activation=act, **kw_of(kind),
                 **({"tail": True} if path == 4 else {}))
        mb.synchronize_status(dev)
        want = ho.fused_epilogue(acc, alpha, beta, Cin.float().cpu().numpy(), bias, which, act)
        err = ho.max_rel_err(D.float().cpu().numpy(), want)
        assert err <= tol, (path, tile_n, m_major, which, act, beta, err)


def test_fused_epilogue_argument_errors(mb, ho, dev):
    M, N, K = 128, 128, 64
    a, b, A, B, _ = operands(ho, "f16", M, N, K, dev, (3, 4))
    D = torch.zeros(M, N, device=dev)
    bias = torch.zeros(N, device=dev)
    with pytest.raises(mb.MoyeError):          # square D: the direction must be named
        mb.gemm_(mb.MoYeArray(D), mb.MoYeArray(A), mb.MoYeArray(B), None, bias=bias)
    with pytest.raises(mb.MoyeError):
        mb.gemm_(mb.MoYeArray(D), mb.MoYeArray(A), mb.MoYeArray(B), None, bias=(torch.zeros(7, device=dev), "col"))
    with pytest.raises(mb.MoyeError):
        mb.gemm_(mb.MoYeArray(D), mb.MoYeArray(A), mb.MoYeArray(B), None, activation="tanh")
    a8, b8, A8, B8, _ = operands(ho, "s8", M, N, K, dev, (5, 6))
    with pytest.raises(mb.MoyeError):          # the integer path stays exact integer arithmetic
        mb.gemm_(mb.MoYeArray(torch.zeros(M, N, device=dev, dtype=torch.int32)), mb.MoYeArray(A8), mb.MoYeArray(B8), None,
                 activation="relu")
    mb.gemm_(mb.MoYeArray(D), mb.MoYeArray(A), mb.MoYeArray(B), None, bias=(bias, "row"), activation="relu")
    mb.synchronize_status(dev)


def widen(ho, x, kind):
    """Raw operand values as the oracle widens them (exact)."""
    if kind == "f16":
        return ho.half_to_float(x)
    if kind == "bf16":
        return ho.bf16_to_float(x)
    if kind == "e4m3":
        return ho.e4m3_to_float(x)
    return x


def checksum_check(ho, kind, a, b, C, M, N, K, scale, tol):
    """A checksum over every element of C, computed on the host without a GPU library: the row sums of C must equal
    A . (sum over n of B[n, :]) -- exactly for s8 (int64); for the float kinds within 8 standard deviations of the
    output rounding (eps_out * sqrt(sum C^2)) plus 1e-5 * sum |C| for the fp32 accumulation order, which is far
    below what one wrong 32-column chunk of a row would change."""
    wide = np.int64 if kind == "s8" else np.float64
    bsum = np.zeros(K, dtype=wide)
    for n0 in range(0, N, 1024):
        bsum += widen(ho, b[n0 * K:(n0 + 1024) * K], kind).reshape(-1, K).astype(wide).sum(axis=0)
    want = np.empty(M, dtype=wide)
    for m0 in range(0, M, 1024):
        want[m0:m0 + 1024] = widen(ho, a[m0 * K:(m0 + 1024) * K], kind).reshape(-1, K).astype(wide) @ bsum
    if kind == "s8":
        assert np.array_equal(C.sum(dim=1, dtype=torch.int64).cpu().numpy(), want)
    else:
        Cd = C.double()
        got = Cd.sum(dim=1).cpu().numpy()
        eps = {torch.float32: 2.0 ** -24, torch.bfloat16: 2.0 ** -9, torch.float16: 2.0 ** -11}[C.dtype]
        bound = 8.0 * eps * (Cd * Cd).sum(dim=1).sqrt().cpu().numpy() + 1e-5 * Cd.abs().sum(dim=1).cpu().numpy()
        del Cd
        assert np.all(np.abs(got - want * float(scale)) <= bound)


def sampled_check(mb, ho, dev, kind, M, N, K, seeds, out_dtype, tol, nsample=128, **kw):
    a, b, A, B, dt = operands(ho, kind, M, N, K, dev, seeds)
    C = torch.zeros(M, N, dtype=out_dtype, device=dev)
    mb.matmul(A, B, C, **kw)
    mb.synchronize_status(dev)
    rs = np.random.Generator(np.random.PCG64(99))
    rows = np.sort(rs.choice(M, size=min(nsample, M), replace=False)).astype(np.int32)
    cols = np.sort(rs.choice(N, size=min(nsample, N), replace=False)).astype(np.int32)
    scale = np.float32(kw.get("scale_a", 1.0) * kw.get("scale_b", 1.0))
    ref_r = ho.gemm_samples(a, b, dt, M, N, K, rows, by_rows=True, threads=NTHREADS)
    ref_c = ho.gemm_samples(a, b, dt, M, N, K, cols, by_rows=False, threads=NTHREADS)
    got_r = C[torch.from_numpy(rows).to(dev).long()].cpu()
    got_c = C[:, torch.from_numpy(cols).to(dev).long()].t().cpu()
    if kind == "s8":
        assert np.array_equal(got_r.numpy(), ref_r) and np.array_equal(got_c.numpy(), ref_c)
    else:
        assert ho.max_rel_err(got_r.float().numpy(), ref_r * scale) <= tol
        assert ho.max_rel_err(got_c.float().numpy(), ref_c * scale) <= tol
    checksum_check(ho, kind, a, b, C, M, N, K, scale, tol)
    return A, B, C


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("n", [4096, 8192])
def test_config3_fp16_dense(mb, ho, dev, n, kind):
    """fp16 x fp16 -> fp32 (and bf16), M=N=K=n, seeds 3/4: 128 full rows and 128 full columns
    against the oracle, and the whole matrix against a second, independent device product."""
    A, B, C = sampled_check(mb, ho, dev, kind, n, n, n, (3, 4), torch.float32, 1e-2)
    other = torch.matmul(A.float(), B.float().t())  # secondary cross-check only (fp32 cuBLAS)
    err = ((C - other).abs().max() / other.abs().max()).item()
    assert err <= 1e-3
    # linearity in A (a size-independent property): (2A).B^T == 2 (A.B^T) exactly in fp16/fp32
    C2 = torch.zeros_like(C)
    mb.matmul((A * 2).contiguous(), B, C2)
    mb.synchronize_status(dev)
    assert torch.equal(C2, C * 2)


def test_config4_quantised(mb, ho, dev):
    M, N, K = 16384, 8192, 8192
    A, B, C = sampled_check(mb, ho, dev, "s8", M, N, K, (5, 6), torch.int32, 0)
    if hasattr(torch, "_int_mm"):
        assert torch.equal(torch._int_mm(A, B.t()), C)  # secondary, whole matrix
    del A, B, C
    torch.cuda.empty_cache()
    sampled_check(mb, ho, dev, "e4m3", M, N, K, (7, 8), torch.bfloat16, 3e-2, scale_a=0.05, scale_b=0.02)


def test_config5_decode_skinny(mb, ho, dev):
    """X 16x8192, W 28672x8192 bf16 N(0,0.02), Y bf16: every element against the oracle, on
    both kernels, and the stream-K result must not depend on timing."""
    M, N, K = 16, 28672, 8192
    x, w, X, W, dt = operands(ho, "bf16", M, N, K, dev, (9, 10))
    ref = ho.gemm_samples(x, w, dt, M, N, K, np.arange(M, dtype=np.int32), threads=NTHREADS)
    outs = []
    for path in (2, 2, 1):
        Y = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        mb.matmul(X, W, Y, path=path)
        mb.synchronize_status(dev)
        assert ho.max_rel_err(Y.float().cpu().numpy(), ref) <= 1e-2
        outs.append(Y)
    assert torch.equal(outs[0], outs[1])
    # column-major Y (MoYe's own layout) through the same kernel
    Yt = torch.zeros(N, M, dtype=torch.bfloat16, device=dev).t()
    mb.matmul(X, W, Yt, path=2)
    mb.synchronize_status(dev)
    assert torch.equal(Yt.contiguous(), outs[0])


@pytest.mark.parametrize("M,N,K", [(1, 512, 512), (7, 1000, 2048), (16, 1024, 1024), (17, 640, 8192), (32, 4096, 4096),
                                   (3, 129, 520), (16, 148 * 128, 64), (33, 1000, 2048), (64, 4096, 4096),
                                   (100, 640, 8192), (128, 148 * 128, 192), (128, 28672, 1024),
                                   # more row-blocks than SMs: whole row-blocks per CTA after the cut ones (185 = 148 + 37,
                                   # 296 = 2 x 148 with nothing cut, 149 = one over: 16 units, one each for 16 CTAs)
                                   (16, 185 * 128, 512), (5, 296 * 128 - 40, 512), (16, 149 * 128, 1024),
                                   # few, short row-blocks: 17 row-blocks of 2 K blocks on 4 CTAs, one left over with two
                                   # units for two of the CTAs
                                   (75, 2064, 128), (16, 185 * 128, 2048),
                                   # slightly fewer row-blocks than SMs: one whole row-block per CTA on fewer CTAs
                                   (16, 112 * 128, 2048), (3, 140 * 128 - 24, 1024),
                                   # a few left-over row-blocks cut over all CTAs: 2 shared by 74 CTAs each, 12 by 12-13
                                   (8, 150 * 128, 4800), (16, 160 * 128, 2048)])
def test_skinny_shapes(mb, ho, dev, M, N, K):
    x, w, X, W, dt = operands(ho, "bf16", M, N, K, dev, (9, 10))
    ref = ho.gemm_samples(x, w, dt, M, N, K, np.arange(M, dtype=np.int32), threads=NTHREADS)
    for out_dtype in (torch.bfloat16, torch.float32):
        Y = torch.zeros(M, N, dtype=out_dtype, device=dev)
        mb.matmul(X, W, Y, path=2, alpha=1.5)
        mb.synchronize_status(dev)
        assert ho.max_rel_err(Y.float().cpu().numpy(), 1.5 * ref) <= 1e-2


@pytest.mark.parametrize("M,N,K", [(16, 1000, 2048), (100, 4096, 1024)])
def test_skinny_fused_bias_activation(mb, ho, dev, M, N, K):
    """The stream-K kernel's epilogue applies bias and activation after the partial sums are combined."""
    x, w, X, W, dt = operands(ho, "bf16", M, N, K, dev, (9, 10))
    acc = ho.gemm_samples(x, w, dt, M, N, K, np.arange(M, dtype=np.int32), threads=NTHREADS)
    sc = float(np.abs(acc).max())
    bcol = ho.rng(41).standard_normal(N).astype(np.float32)
    brow = ho.rng(42).standard_normal(M).astype(np.float32)
    for which, act in (("col", "gelu"), ("row", "relu"), (None, "silu"), ("col", None)):
        bias = {None: None, "col": bcol, "row": brow}[which]
        tb = None if bias is None else (torch.from_numpy(bias).to(dev), which)
        for out_dtype in (torch.bfloat16, torch.float32):
            Y = torch.zeros(M, N, dtype=out_dtype, device=dev)
            mb.gemm_(mb.MoYeArray(Y), mb.MoYeArray(X), mb.MoYeArray(W), None, alpha=1.0 / sc, path=2, bias=tb, activation=act)
            mb.synchronize_status(dev)
            want = ho.fused_epilogue(acc, 1.0 / sc, 0.0, None, bias, which, act)
            assert ho.max_rel_err(Y.float().cpu().numpy(), want) <= 1e-2, (which, act, out_dtype)


def test_gemm_argument_errors(mb, dev):
    lib, h = mb._lib.load(), mb._lib.handle(dev.index)
    st = mb.current_stream_ptr(dev)
    buf = torch.zeros(1 << 16, dtype=torch.float16, device=dev)
    out = torch.zeros(1 << 16, dtype=torch.float32, device=dev)
    T = mb._lib.make_tensor
    F16, F32 = mb._lib.F16, mb._lib.F32
    A = T(buf.data_ptr(), F16, [128, 64], [64, 1])
    B = T(buf.data_ptr(), F16, [128, 64], [64, 1])
    D = T(out.data_ptr(), F32, [128, 128], [128, 1])
    p = mb._lib.GemmParams(1.0, 0.0, 1.0, 1.0, 0, 0, 0, 0)

    def call(D=D, A=A, B=B, C=None, p=p):
        return lib.moye_b200_gemm(h, ctypes.byref(D), ctypes.byref(A), ctypes.byref(B),
                                  ctypes.byref(C) if C is not None else None, ctypes.byref(p), st)

    assert call() == 0
    assert call(A=T(buf.data_ptr(), F16, [128, 64], [1, 128])) == 0                   # A column-major (MN-major) is fine
    assert call(A=T(buf.data_ptr(), F16, [128, 64], [2, 256])) == -3                  # no unit stride at all
    assert call(A=T(buf.data_ptr(), F16, [128, 60], [60, 1]), B=T(buf.data_ptr(), F16, [128, 60], [60, 1])) == -5
    assert call(A=T(buf.data_ptr() + 2, F16, [128, 64], [64, 1])) == -5               # misaligned base
    assert call(B=T(buf.data_ptr(), F16, [128, 32], [32, 1])) == -4                   # K mismatch
    assert call(B=T(buf.data_ptr(), mb._lib.BF16, [128, 64], [64, 1])) == -2          # mixed operand types
    assert call(D=T(out.data_ptr(), mb._lib.S32, [128, 128], [128, 1])) == -2         # f16 -> s32 unsupported
    assert call(A=T(buf.data_ptr(), F32, [128, 32], [32, 1]), B=T(buf.data_ptr(), F32, [128, 32], [32, 1])) == 0   # f32: three tf32 products
    assert call(A=T(buf.data_ptr(), F32, [128, 32], [32, 1]), B=T(buf.data_ptr(), F32, [128, 32], [32, 1]),
                p=mb._lib.GemmParams(1.0, 0.0, 1.0, 1.0, 0, 0, 0, mb._lib.GEMM_ALLOW_TF32)) == 0               # f32: one tf32 product
    assert call(A=T(buf.data_ptr(), mb._lib.U8, [128, 64], [64, 1]), B=T(buf.data_ptr(), mb._lib.U8, [128, 64], [64, 1])) == -2  # u8 -> f32
    assert call(p=mb._lib.GemmParams(1.0, 0.0, 1.0, 1.0, 0, 0, 4, mb._lib.GEMM_TAIL_ON | mb._lib.GEMM_TAIL_OFF)) == -1   # contradictory bits
    assert call(p=mb._lib.GemmParams(1.0, 0.0, 1.0, 1.0, 0, 0, 0, 0x1000)) == -1                                   # unknown bit
    assert call(p=mb._lib.GemmParams(1.0, 1.0, 1.0, 1.0, 0, 0, 0, 0)) == -1           # beta without C
    assert call(p=mb._lib.GemmParams(1.0, 0.0, 1.0, 1.0, 96, 0, 0, 0)) == -1          # bad tile_n
    big = T(buf.data_ptr(), F16, [256, 64], [64, 1])
    assert call(A=big, D=T(out.data_ptr(), F32, [256, 128], [128, 1]), p=mb._lib.GemmParams(1.0, 0.0, 1.0, 1.0, 0, 0, 2, 0)) == -4  # skinny path with M > 128
    assert call(D=T(out.data_ptr(), F32, [128, 128], [2, 256])) == -3                 # D without a unit stride
    assert lib.moye_b200_gemm(h, None, ctypes.byref(A), ctypes.byref(B), None, ctypes.byref(p), st) == -1
    A8 = T(buf.data_ptr(), mb._lib.S8, [128, 64], [64, 1])
    D32 = T(out.data_ptr(), mb._lib.S32, [128, 128], [128, 1])
    assert call(D=D32, A=A8, B=A8, p=mb._lib.GemmParams(2.0, 0.0, 1.0, 1.0, 0, 0, 0, 0)) == -1  # s8 path is exact
    assert call(D=D32, A=T(buf.data_ptr(), mb._lib.S8, [128, 64], [1, 128]), B=A8) == 0    # 8-bit operands may be MN-major
    assert call(D=D32, A=T(buf.data_ptr(), mb._lib.S8, [128, 64], [2, 256]), B=A8) == -3   # but need one unit stride
    mb.synchronize_status(dev)


def test_prepared_plans_match_direct_calls(mb, ho, dev):
    """plan_gemm / plan_copy marshal the arguments once; repeated launches must equal the direct call."""
    M, N, K = 512, 384, 256
    a, b, A, B, dt = operands(ho, "f16", M, N, K, dev, (3, 4))
    want = torch.zeros(M, N, device=dev)
    mb.matmul(A, B, want)
    got = torch.zeros(M, N, device=dev)
    plan = mb.plan_gemm(mb.make_tiled_mma(mb.sm100_mma_op("F16", 256)), got, A, B, None)
    for _ in range(3):
        got.zero_()
        plan()
        mb.synchronize_status(dev)
        assert torch.equal(got, want)
    src = torch.rand(96, 1024, device=dev).half()
    dst = torch.zeros_like(src)
    lay = mb.make_layout((1024, 96))
    cp = mb.plan_copy(mb.make_tma_tiled_copy(mb._lib.F16), mb.MoYeArray(dst, lay), mb.MoYeArray(src, lay))
    cp(mb.current_stream_ptr(dev))
    mb.synchronize_status(dev)
    assert torch.equal(src, dst)
    with pytest.raises(mb.MoyeError):
        mb.plan_copy(mb.MoYeArray(dst, mb.make_layout((96, 1024), (1024, 1))), mb.MoYeArray(src, lay))


def test_host_pipeline_steps_are_each_correct(mb, ho, dev):
    """Five host-to-host steps with different operands through the three-stream pipeline."""
    M, N, K = 256, 384, 512
    pipe = mb.HostGemmPipeline(M, N, K, torch.float16, torch.float32, dev, depth=2)
    hosts, outs, refs = [], [], []
    for i in range(5):
        a, b = ho.uniform_pm1_f16_bits(30 + i, (M * K,)), ho.uniform_pm1_f16_bits(40 + i, (N * K,))
        hA = torch.from_numpy(a.view(np.int16)).view(torch.float16).view(M, K).pin_memory()
        hB = torch.from_numpy(b.view(np.int16)).view(torch.float16).view(N, K).pin_memory()
        hC = torch.zeros(M, N).pin_memory()
        hosts.append((hA, hB))
        outs.append(hC)
        refs.append(ho.gemm_samples(a, b, ho.F16, M, N, K, np.arange(0, M, 5, dtype=np.int32), threads=NTHREADS))
        pipe.submit(hA, hB, hC)
    pipe.join()
    torch.cuda.synchronize()
    mb.synchronize_status(dev)
    for hC, ref in zip(outs, refs):
        assert ho.max_rel_err(hC.numpy()[::5], ref) <= 1e-2


def test_bounded_wait_gives_up_and_the_context_survives(mb, ho, dev):
    """The error path of every kernel's waits, end to end: a wait on a barrier nothing arrives at runs out, the
    kernel returns, `moye_b200_status` reports TIMEOUT with the site code once, and the next launches work."""
    lib, h = mb._lib.load(), mb._lib.handle(dev.index)
    st = mb.current_stream_ptr(dev)
    assert lib.moye_b200_selftest_bounded_wait(h, st) == 0
    site = ctypes.c_int32(0)
    assert lib.moye_b200_status(h, st, ctypes.byref(site)) == -7 and site.value == 901
    assert b"bounded" in lib.moye_b200_last_error()
    assert lib.moye_b200_status(h, st, ctypes.byref(site)) == 0 and site.value == 0      # reported once, then clear
    M, N, K = 256, 512, 256
    a, b, A, B, dt = operands(ho, "f16", M, N, K, dev, (3, 4))
    C = torch.zeros(M, N, device=dev)
    mb.matmul(A, B, C)
    mb.synchronize_status(dev)
    ref = ho.gemm_samples(a, b, dt, M, N, K, np.arange(M, dtype=np.int32), threads=NTHREADS)
    assert ho.max_rel_err(C.cpu().numpy(), ref) <= 1e-2


def test_stale_stream_k_tickets_are_cleared_after_a_timeout(mb, ho, dev):
    """A kernel that gives up can leave stream-K tickets half counted.  Provoked without a fault: the self-test
    kernel runs out of patience (the only kernel that ever should), the host scribbles non-zero tickets into both
    scratch areas as a broken kernel would have, `moye_b200_status` reports the time-out -- and must leave both
    ticket areas zero, so that the next stream-K products on that handle are right."""
    lib, h = mb._lib.load(), mb._lib.handle(dev.index)
    st = mb.current_stream_ptr(dev)
    M, N, K = 16, 2048, 2048
    x, w, X, W, dt = operands(ho, "bf16", M, N, K, dev, (9, 10))
    ref = ho.gemm_samples(x, w, dt, M, N, K, np.arange(M, dtype=np.int32), threads=NTHREADS)
    Y = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    mb.matmul(X, W, Y, path=2)                      # makes sure the skinny scratch exists
    Md, Nd, Kd = 512, 1024, 1024
    a, b, A, B, dtd = operands(ho, "f16", Md, Nd, Kd, dev, (3, 4))
    refd = ho.gemm_samples(a, b, dtd, Md, Nd, Kd, np.arange(Md, dtype=np.int32), threads=NTHREADS)
    C = torch.zeros(Md, Nd, device=dev)
    mb.matmul(A, B, C, path=4, tail=True)           # ... and the dense tail's
    mb.synchronize_status(dev)
    assert lib.moye_b200_selftest_dirty_tickets(h, st) == 0
    assert lib.moye_b200_selftest_bounded_wait(h, st) == 0
    site = ctypes.c_int32(0)
    assert lib.moye_b200_status(h, st, ctypes.byref(site)) == -7 and site.value == 901
    Y.zero_()
    mb.matmul(X, W, Y, path=2)
    C.zero_()
    mb.matmul(A, B, C, path=4, tail=True)
    mb.synchronize_status(dev)
    assert ho.max_rel_err(Y.float().cpu().numpy(), ref) <= 1e-2
    assert ho.max_rel_err(C.cpu().numpy(), refd) <= 1e-2


def test_stream_k_on_two_streams_of_one_handle(mb, ho, dev):
    """Stream-K launches of one handle share its scratch.  Alternating products on two streams must not disturb
    each other: the library orders them with an event."""
    M, N, K = 16, 4096, 4096
    x, w, X, W, dt = operands(ho, "bf16", M, N, K, dev, (9, 10))
    x2, w2, X2, W2, _ = operands(ho, "bf16", M, N, K, dev, (11, 12))
    ref = ho.gemm_samples(x, w, dt, M, N, K, np.arange(M, dtype=np.int32), threads=NTHREADS)
    ref2 = ho.gemm_samples(x2, w2, dt, M, N, K, np.arange(M, dtype=np.int32), threads=NTHREADS)
    s1, s2 = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    torch.cuda.synchronize()
    Y1 = [torch.zeros(M, N, dtype=torch.bfloat16, device=dev) for _ in range(8)]
    Y2 = [torch.zeros(M, N, dtype=torch.bfloat16, device=dev) for _ in range(8)]
    for i in range(8):
        mb.matmul(X, W, Y1[i], path=2, stream=ctypes.c_void_p(s1.cuda_stream))
        mb.matmul(X2, W2, Y2[i], path=2, stream=ctypes.c_void_p(s2.cuda_stream))
    torch.cuda.synchronize()
    mb.synchronize_status(dev)
    for i in range(8):
        assert ho.max_rel_err(Y1[i].float().cpu().numpy(), ref) <= 1e-2, i
        assert ho.max_rel_err(Y2[i].float().cpu().numpy(), ref2) <= 1e-2, i
        assert torch.equal(Y1[i], Y1[0]) and torch.equal(Y2[i], Y2[0])


def test_split_k_clusters_share_scratch_across_streams_and_launches(mb, ho, dev):
    """The cluster split-K kernel sums its partial tiles through the handle's scratch (shared with the K-split tail of
    the 256 x 512 kernel) and is launched so that its set-up may overlap the previous grid.  Back-to-back launches on
    one stream and alternating launches on two streams, mixed with products that take the tail, must all be right and
    bit-equal from run to run; a request with more CTAs than the scratch has images is refused."""
    M, N, K = 200, 2048, 2048
    a, b, A, B, dt = operands(ho, "bf16", M, N, K, dev, (9, 10))
    a2, b2, A2, B2, _ = operands(ho, "bf16", M, N, K, dev, (11, 12))
    rows = np.arange(M, dtype=np.int32)
    ref, ref2 = (ho.gemm_samples(x, w, dt, M, N, K, rows, threads=NTHREADS) for x, w in ((a, b), (a2, b2)))
    Mt, Nt, Kt = 512, 1024, 1024
    at, bt, At, Bt, dtt = operands(ho, "f16", Mt, Nt, Kt, dev, (3, 4))
    reft = ho.gemm_samples(at, bt, dtt, Mt, Nt, Kt, np.arange(Mt, dtype=np.int32), threads=NTHREADS)
    s1, s2 = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    torch.cuda.synchronize()
    Y1 = [torch.zeros(M, N, dtype=torch.bfloat16, device=dev) for _ in range(8)]
    Y2 = [torch.zeros(M, N, dtype=torch.bfloat16, device=dev) for _ in range(8)]
    Ct = [torch.zeros(Mt, Nt, device=dev) for _ in range(4)]
    for i in range(8):
        mb.matmul(A, B, Y1[i], path=5, split_k=4 if i % 2 else 2, stream=ctypes.c_void_p(s1.cuda_stream))
        mb.matmul(A2, B2, Y2[i], path=5, tile_n=128, stream=ctypes.c_void_p(s2.cuda_stream))
        if i % 2:
            mb.matmul(At, Bt, Ct[i // 2], path=4, tail=True, stream=ctypes.c_void_p(s1.cuda_stream))
    torch.cuda.synchronize()
    mb.synchronize_status(dev)
    for i in range(8):
        assert ho.max_rel_err(Y1[i].float().cpu().numpy(), ref) <= 1e-2, i
        assert ho.max_rel_err(Y2[i].float().cpu().numpy(), ref2) <= 1e-2, i
        assert torch.equal(Y1[i], Y1[i % 2]) and torch.equal(Y2[i], Y2[0])
    for c in Ct:
        assert ho.max_rel_err(c.cpu().numpy(), reft) <= 1e-2
    big = torch.zeros(4096, 4096, dtype=torch.bfloat16, device=dev)
    with pytest.raises(mb.MoyeError) as e:
        mb.matmul(big[:, :256], big[:, :256], torch.zeros(4096, 4096, dtype=torch.bfloat16, device=dev), path=5, split_k=8)
    assert e.value.code == -9 and "image" in str(e.value)
    mb.synchronize_status(dev)


@pytest.mark.parametrize("M,N,K", [(4096, 4096, 4096), (1024, 8192, 8192), (300, 520, 1008), (2304, 1536, 768)])
def test_stream_k_tail_equals_whole_tiles(mb, ho, dev, M, N, K):
    """The stream-K tail only changes who computes which K blocks: s8 results are identical to the whole-tile
    schedule, fp16 results agree with the oracle and do not depend on timing (two runs are bit-equal)."""
    a8, b8, A8, B8, _ = operands(ho, "s8", M, N, K, dev, (5, 6))
    outs = []
    for tail in (False, True, True):
        C = torch.zeros(M, N, dtype=torch.int32, device=dev)
        mb.matmul(A8, B8, C, path=4, tail=tail)
        mb.synchronize_status(dev)
        outs.append(C)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])
    rows = np.arange(0, M, max(1, M // 64), dtype=np.int32)
    assert np.array_equal(outs[1].cpu().numpy()[rows], ho.gemm_samples(a8, b8, ho.S8, M, N, K, rows, threads=NTHREADS))
    del outs, A8, B8
    a, b, A, B, dt = operands(ho, "f16", M, N, K, dev, (3, 4))
    ref = ho.gemm_samples(a, b, dt, M, N, K, rows, threads=NTHREADS)
    got = []
    for m_major in (False, True, False):
        C = out_tensor(M, N, torch.float32, dev, m_major)
        mb.matmul(A, B, C, path=4, tail=True)
        mb.synchronize_status(dev)
        assert ho.max_rel_err(C.cpu().numpy()[rows], ref) <= 1e-2
        got.append(C.contiguous())
    assert torch.equal(got[0], got[1]) and torch.equal(got[0], got[2])


@pytest.mark.parametrize("ka,kb", [("u8", "u8"), ("u8", "s8"), ("s8", "u8")])
def test_unsigned_8bit_operands(mb, ho, dev, ka, kb):
    """UInt8 operands, also mixed with Int8 (the reference's S32U8U8S32 / S32U8S8S32 / S32S8U8S32 ops,
    src/arch/mma/make_mma_ops.jl:143-160): bit-exact against the host gemm! in Int32 on widened inputs."""
    M, N, K = 384, 520, 1008
    rs = ho.rng(71)
    a = rs.integers(0, 256, M * K, dtype=np.int64) if ka == "u8" else rs.integers(-128, 128, M * K, dtype=np.int64)
    b = rs.integers(0, 256, N * K, dtype=np.int64) if kb == "u8" else rs.integers(-128, 128, N * K, dtype=np.int64)
    ref = ho.gemm_s32(a.astype(np.int32), (K, 1), b.astype(np.int32), (K, 1), M, N, K, c_strides=(N, 1)).reshape(M, N)
    A = torch.from_numpy(a.astype(np.uint8 if ka == "u8" else np.int8)).to(dev).view(M, K)
    B = torch.from_numpy(b.astype(np.uint8 if kb == "u8" else np.int8)).to(dev).view(N, K)
    for path, extra in ((1, {}), (3, {}), (4, {"tail": True}), (5, {}), (0, {})):
        C = torch.zeros(M, N, dtype=torch.int32, device=dev)
        mb.matmul(A, B, C, path=path, **extra)
        mb.synchronize_status(dev)
        assert np.array_equal(C.cpu().numpy(), ref), (path, extra)


@pytest.mark.parametrize("M,N,K", [(256, 512, 1024), (384, 520, 1008), (2048, 2048, 512)])
def test_float32_three_product_split(mb, ho, dev, M, N, K):
    """Float32 operands without allow_tf32: hi/lo split on the tf32 tensor-core kind, as accurate as the fp32 host
    gemm! on the raw operands (the arithmetic the reference's Float32 example runs, examples/gemm.jl:91-96), row- and
    column-major, with alpha / beta and a fused bias."""
    a, b = ho.uniform_pm1(3, (M * K,)), ho.uniform_pm1(4, (N * K,))
    raw = ho.gemm_f32(a, (K, 1), b, (K, 1), M, N, K, c_strides=(N, 1)).reshape(M, N)
    exact = ho.gemm_f64(a.astype(np.float64), (K, 1), b.astype(np.float64), (K, 1), M, N, K, c_strides=(N, 1)).reshape(M, N)
    A, B = torch.from_numpy(a).to(dev).view(M, K), torch.from_numpy(b).to(dev).view(N, K)
    for a_mn, b_mn, m_major in ((False, False, False), (True, True, True), (True, False, False)):
        if (a_mn and M % 4) or (b_mn and N % 4) or (m_major and M % 4):
            continue
        C = out_tensor(M, N, torch.float32, dev, m_major)
        mb.matmul(col_major(A) if a_mn else A, col_major(B) if b_mn else B, C)
        mb.synchronize_status(dev)
        f32_as_accurate_as_host(ho, C.cpu().numpy(), raw, exact)
    cin = ho.rng(5).standard_normal((M, N)).astype(np.float32) * np.float32(K ** 0.5)
    bias = ho.rng(6).standard_normal(N).astype(np.float32)
    D = torch.zeros(M, N, device=dev)
    mb.gemm_(mb.MoYeArray(D), mb.MoYeArray(A), mb.MoYeArray(B), mb.MoYeArray(torch.from_numpy(cin).to(dev)), alpha=0.5,
             beta=2.0, bias=(torch.from_numpy(bias).to(dev), "col"), activation="relu")
    mb.synchronize_status(dev)
    want = ho.fused_epilogue(raw, 0.5, 2.0, cin, bias, "col", "relu")
    want64 = ho.fused_epilogue(exact, 0.5, 2.0, cin, bias, "col", "relu")   # evaluated in float64, returned as float32
    f32_as_accurate_as_host(ho, D.cpu().numpy(), want, want64)


def test_parity_under_the_debug_build(dev):
    """The debug library (`build.py --debug`, selected with MOYE_B200_DEBUG=1) checks on the device every global
    address the kernels form by hand, every TMA coordinate and staging buffer, and the tensor-memory columns; a
    violation would surface as a status code.  The small parity tests must pass under it unchanged -- this is the
    stand-in for a memory checker on machines where none may run."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sel = ("test_small_goldens_all_dtypes or test_alpha_beta_and_low_precision_outputs or test_skinny_shapes or "
           "(test_gemm_full_oracle and 384-520-1008) or (test_stream_k_tail_equals_whole_tiles and 300-520-1008) or "
           "(test_float32_three_product_split and 256-512-1024)")
    env = dict(os.environ, MOYE_B200_DEBUG="1")
    res = subprocess.run([sys.executable, "-m", "pytest", os.path.join(root, "tests", "test_gpu_gemm.py"),
                          os.path.join(root, "tests", "test_gpu_layout_copy.py"), "-q", "-x", "-m", "gpu", "-k",
                          sel + " or ldmatrix or transpos"], capture_output=True, text=True, env=env, timeout=1500)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-1000:]
    assert "libmoye_b200_debug.so" in subprocess.run(
        [sys.executable, "-c", "import __graft_entry__ as g; print(g.load_package()._lib.LIB_PATH)"], capture_output=True,
        text=True, env=env, cwd=root).stdout


_LOG_SCRIPT = r"""
import sys
import torch
sys.path.insert(0, sys.argv[1])
import __graft_entry__ as ge
mb = ge.load_package()
dev = torch.device("cuda", 0)
for M, N, K in ((512, 1024, 256), (16, 2048, 1024)):
    A = torch.randn(M, K, device=dev).bfloat16(); B = torch.randn(N, K, device=dev).bfloat16()
    D = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    mb.matmul(A, B, D)
src = torch.randn(256, 512, device=dev)
dst = torch.empty(512, 256, device=dev).t()
mb.copyto_(mb.MoYeArray(dst), mb.MoYeArray(src))
mb.synchronize_status(dev)
"""


def test_log_level_one_names_the_kernel_chosen(dev):
    """MOYE_B200_LOG=1: one line per call on stderr with the shape and the kernel / tile the dispatch chose."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-c", _LOG_SCRIPT, root], capture_output=True, text=True,
                         env=dict(os.environ, MOYE_B200_LOG="1"), timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stderr.splitlines() if l.startswith("[moye_b200]")]
    assert any("gemm 512 x 1024 x 256" in l and "tile_n" in l for l in lines), lines
    assert any("gemm 16 x 2048 x 1024" in l for l in lines), lines
    assert any(l.startswith("[moye_b200] copy") for l in lines), lines


def test_cpp_caller_through_the_c_abi(dev, tmp_path):
    """tests/c_abi_smoke.cpp -- a C++ caller with the header, the CUDA runtime and the library, nothing else: an exact
    integer-valued fp16 product on ragged sizes, its transposing copy, the status call, and a refused operand."""
    import subprocess
    from test_abi import build_c_abi_smoke
    res = subprocess.run([build_c_abi_smoke(tmp_path)], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "C_ABI_SMOKE_OK" in res.stdout, res.stdout + res.stderr


@pytest.mark.parametrize("seed", [3, 11, 12])
def test_random_shapes_and_paths_against_the_gpu_float64_product(mb, dev, seed):
    """A secondary cross-check, not the parity definition (that is the oracle, above): a few hundred random shapes,
    kernels, tile widths, cluster sizes, output types and majors, alpha / beta, each compared with a float64 product
    computed on the GPU -- the oracle is too slow to sweep that many shapes, and a sweep like this found a stream-K
    schedule (75 x 2064 x 128: an empty run between the owners of a cut row-block) that no hand-picked shape had hit.
    s8 must be exact; a refusal (MoyeError) of an unsupported combination is fine, a wrong number is not."""
    import random
    rnd = random.Random(seed)
    ran = 0
    for case in range(300):
        kind = rnd.choice(["bf16", "bf16", "f16", "s8"])
        path = rnd.choice([0, 0, 1, 2, 3, 4, 5, 5, 2])
        if path == 2:
            kind = "bf16" if kind == "s8" else kind
            M = rnd.randint(1, 128)
            N = rnd.choice([rnd.randint(1, 400) * 8, rnd.randint(140, 330) * 128, rnd.randint(1, 64) * 128 + rnd.randint(0, 15) * 8])
            K = rnd.choice([64, 128, 512, 520, 1024, 2048, 4096, rnd.randint(8, 512) * 8])
        else:
            M = rnd.choice([rnd.randint(1, 700), rnd.randint(1, 2500), 128, 256, 512])
            N = rnd.randint(1, 300) * 8 if rnd.random() < 0.7 else rnd.randint(1, 40) * 128
            K = rnd.choice([16, 64, 128, 1024, 2048, rnd.randint(2, 512) * 16])
        kw = {}
        if path == 5:
            kw = {"split_k": rnd.choice([0, 2, 4, 8]), "tile_n": rnd.choice([0, 128, 256])}
        elif path == 1:
            kw = {"tile_n": rnd.choice([0, 64, 128, 256])}
        elif path == 3:
            kw = {"tile_n": rnd.choice([128, 256])}
        elif path == 4:
            kw = {"tail": rnd.choice([True, False])}
        if kind == "s8":
            A = torch.randint(-128, 128, (M, K), device=dev, dtype=torch.int8)
            B = torch.randint(-128, 128, (N, K), device=dev, dtype=torch.int8)
            C = torch.zeros(M, N, device=dev, dtype=torch.int32)
        else:
            dt = torch.bfloat16 if kind == "bf16" else torch.float16
            A = (torch.rand(M, K, device=dev) * 2 - 1).to(dt)
            B = (torch.rand(N, K, device=dev) * 2 - 1).to(dt)
            out_dt = rnd.choice([torch.float32, dt])
            C = torch.zeros(M, N, device=dev, dtype=out_dt)
            if rnd.random() < 0.3 and path != 2 and (M * C.element_size()) % 16 == 0:
                C = torch.zeros(N, M, device=dev, dtype=out_dt).t()                     # M-major D
        ref = A.double() @ B.double().t()
        alpha = rnd.choice([1.0, 1.0, 0.5]) if kind != "s8" else 1.0
        beta, Cin = 0.0, None
        if kind != "s8" and path != 2 and rnd.random() < 0.25:
            beta = rnd.choice([1.0, -0.5])
            Cin = (torch.rand(M, N, device=dev) * 2 - 1).to(C.dtype)
            if C.stride(0) == 1:
                Cin = Cin.t().contiguous().t()
            ref = ref + beta / alpha * Cin.double()
        try:
            if Cin is not None:
                mb.gemm_(mb.MoYeArray(C), mb.MoYeArray(A), mb.MoYeArray(B), mb.MoYeArray(Cin), path=path, alpha=alpha, beta=beta, **kw)
            else:
                mb.matmul(A, B, C, path=path, alpha=alpha, **kw)
            mb.synchronize_status(dev)
        except mb.MoyeError as e:
            assert e.code in (-1, -2, -3, -4, -5, -9), (case, kind, path, M, N, K, kw, str(e))
            continue
        ran += 1
        what = (case, kind, path, M, N, K, kw, C.dtype, beta, C.stride(0) == 1)
        if kind == "s8":
            assert torch.equal(C.double(), ref), what
        else:
            err = ((C.double() - alpha * ref).abs().max() / (alpha * ref).abs().max().clamp_min(1e-6)).item()
            assert err <= (5e-3 if C.dtype == torch.float32 else 2e-2), what + (err,)
    assert ran >= 250


@pytest.mark.parametrize("seed", [1, 2])
def test_random_decode_shapes_around_the_schedule_boundaries(mb, dev, seed):
    """Same kind of secondary cross-check for the stream-K kernel's schedule rules: row-block counts around the SM
    count (whole row-blocks per CTA, a few left over, one fewer, slightly fewer on a smaller grid), 1 to 128 rows, short
    and long K, through the automatic choice and `path = 2`, with bias / relu now and then, against float64 on the GPU."""
    import random
    rnd = random.Random(seed)
    for case in range(200):
        M = rnd.choice([1, 2, 4, 7, 16, 17, 31, 32, 33, 64, 100, 128])
        T = rnd.choice([rnd.randint(70, 160), rnd.randint(140, 156), rnd.randint(145, 300), 148, 296, 149, 147, 74, 111, 112])
        N = T * 128 - rnd.choice([0, 0, 8, 64, 120])
        K = rnd.choice([512, 520, 576, 1024, 2048, 3000 // 8 * 8, 4096, 64 * rnd.randint(8, 60)])
        path = rnd.choice([0, 2])
        dt = rnd.choice([torch.bfloat16, torch.float16])
        A = (torch.rand(M, K, device=dev) * 2 - 1).to(dt)
        B = (torch.rand(N, K, device=dev) * 2 - 1).to(dt)
        C = torch.zeros(M, N, device=dev, dtype=rnd.choice([torch.float32, dt]))
        kw = {}
        ref = A.double() @ B.double().t()
        if rnd.random() < 0.3:
            which = rnd.choice(["col", "row"])
            bvec = torch.randn(N if which == "col" else M, device=dev)
            kw = {"bias": (bvec, which), "activation": rnd.choice([None, "relu"])}
            ref = ref + (bvec.double()[None, :] if which == "col" else bvec.double()[:, None])
            if kw["activation"] == "relu":
                ref = ref.clamp_min(0)
        mb.gemm_(mb.MoYeArray(C), mb.MoYeArray(A), mb.MoYeArray(B), None, path=path, **kw)
        mb.synchronize_status(dev)
        err = ((C.double() - ref).abs().max() / ref.abs().max().clamp_min(1e-6)).item()
        assert err <= (5e-3 if C.dtype == torch.float32 else 2e-2), (case, M, N, K, path, C.dtype, err)
