"""TEST INFRASTRUCTURE -- Python face of the C oracle (oracle/moye_host.c) plus the seeded
input generators every parity test and the benchmark share.

Only tests, the smoke check and the CPU-baseline / reference arm of the benchmark import
this module.  The reference (MoYe.jl) is Julia and cannot run here; what is restated, and
why the widened-input form is the parity definition, is explained at the top of moye_host.c.
Julia's RNG cannot be reproduced, so inputs are defined by numpy PCG64 seeds and shared by
the oracle and the GPU path.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libmoye_oracle.so")
_lib = None

# the values of moye_dtype_t the sampled GEMM understands
F32, F16, BF16, S8, E4M3 = 0, 1, 2, 3, 5


def build():
    """Compile the C oracle with the committed Makefile."""
    subprocess.run(["make", "-C", _HERE, "-s"], check=True)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
        _lib.moye_oracle_fma_literal_s8.restype = ctypes.c_int32
        _lib.moye_oracle_fma_literal_s8.argtypes = [ctypes.c_int8, ctypes.c_int8, ctypes.c_int32]
        _lib.moye_oracle_fma_literal_f16.restype = ctypes.c_float
        _lib.moye_oracle_fma_literal_f16.argtypes = [ctypes.c_uint16, ctypes.c_uint16, ctypes.c_float]
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _i64(v):
    return ctypes.c_int64(int(v))


# ----------------------------------------------------------------------------- codecs
def _codec(name, src, out_dtype):
    src = np.ascontiguousarray(src)
    out = np.empty(src.shape, dtype=out_dtype)
    getattr(lib(), name)(_p(src), _p(out), _i64(src.size))
    return out


def half_to_float(bits): return _codec("moye_oracle_half_to_float", bits.astype(np.uint16, copy=False), np.float32)
def float_to_half(x): return _codec("moye_oracle_float_to_half", x.astype(np.float32, copy=False), np.uint16)
def bf16_to_float(bits): return _codec("moye_oracle_bf16_to_float", bits.astype(np.uint16, copy=False), np.float32)
def float_to_bf16(x): return _codec("moye_oracle_float_to_bf16", x.astype(np.float32, copy=False), np.uint16)
def e4m3_to_float(bits): return _codec("moye_oracle_e4m3_to_float", bits.astype(np.uint8, copy=False), np.float32)
def float_to_e4m3(x): return _codec("moye_oracle_float_to_e4m3", x.astype(np.float32, copy=False), np.uint8)


def fma_literal_s8(a, b, c):
    return lib().moye_oracle_fma_literal_s8(a, b, c)


def fma_literal_f16(a_bits, b_bits, c):
    return lib().moye_oracle_fma_literal_f16(a_bits, b_bits, c)


# ----------------------------------------------------------------------------- seeded inputs
def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def uniform_pm1(seed, shape):
    """i.i.d. uniform[-1, 1) float32."""
    return (rng(seed).random(shape, dtype=np.float32) * 2.0 - 1.0).astype(np.float32)


def uniform_pm1_f16_bits(seed, shape):
    return float_to_half(uniform_pm1(seed, shape))


def uniform_s8(seed, shape):
    return rng(seed).integers(-128, 128, size=shape, dtype=np.int8)


def normal_e4m3_bits(seed, shape):
    """N(0,1) clamped to +-448, rounded RNE-satfinite to e4m3."""
    x = rng(seed).standard_normal(shape, dtype=np.float32)
    return float_to_e4m3(np.clip(x, -448.0, 448.0))


def normal_bf16_bits(seed, shape, std):
    x = rng(seed).standard_normal(shape, dtype=np.float32) * np.float32(std)
    return float_to_bf16(x)


# ----------------------------------------------------------------------------- layout / copy
def layout_eval(shape, stride, first, n):
    shape = np.asarray(shape, dtype=np.int64)
    stride = np.asarray(stride, dtype=np.int64)
    out = np.empty(n, dtype=np.int64)
    lib().moye_oracle_layout_eval(len(shape), _p(shape), _p(stride), _i64(first), _i64(n), _p(out))
    return out


def copy_layout(dst, dshape, dstride, src, sshape, sstride):
    """dst[Ld(i)] = src[Ls(i)] over flat numpy buffers of one dtype."""
    ds, dd = np.asarray(dshape, dtype=np.int64), np.asarray(dstride, dtype=np.int64)
    ss, sd = np.asarray(sshape, dtype=np.int64), np.asarray(sstride, dtype=np.int64)
    n = int(np.prod(ss))
    assert int(np.prod(ds)) == n and dst.dtype == src.dtype
    lib().moye_oracle_copy_layout(_p(dst), len(ds), _p(ds), _p(dd), _p(src), len(ss), _p(ss), _p(sd), _i64(n),
                                  dst.dtype.itemsize)


def copy_kernel(dst, src, m, n, bm=32, bn=32, tm=32, tn=8):
    """The reference's copy_kernel over column-major (m, n) buffers (flat numpy arrays)."""
    rc = lib().moye_oracle_copy_kernel(_p(dst), _i64(m), _p(src), _i64(m), _i64(m), _i64(n), bm, bn, tm, tn,
                                       dst.dtype.itemsize)
    if rc != 0:
        raise ValueError("tile / thread layout does not divide the matrix")


# ----------------------------------------------------------------------------- GEMM
def _strides(arr_ld, major):
    return arr_ld


def gemm_f32(A, a_strides, B, b_strides, M, N, K, c_strides=None):
    """Plain sequential-k triple loop on float32 buffers.  Strides are element strides
    (row, k) for A and B, (m, n) for C.  Returns C as a flat float32 array."""
    c_strides = c_strides or (1, M)
    C = np.zeros(M * N, dtype=np.float32)
    lib().moye_oracle_gemm_f32(_p(A), _i64(a_strides[0]), _i64(a_strides[1]), _p(B), _i64(b_strides[0]),
                               _i64(b_strides[1]), _p(C), _i64(c_strides[0]), _i64(c_strides[1]), _i64(M), _i64(N),
                               _i64(K))
    return C


def gemm_s32(A, a_strides, B, b_strides, M, N, K, c_strides=None):
    c_strides = c_strides or (1, M)
    C = np.zeros(M * N, dtype=np.int32)
    lib().moye_oracle_gemm_s32(_p(A), _i64(a_strides[0]), _i64(a_strides[1]), _p(B), _i64(b_strides[0]),
                               _i64(b_strides[1]), _p(C), _i64(c_strides[0]), _i64(c_strides[1]), _i64(M), _i64(N),
                               _i64(K))
    return C


def gemm_f64(A, a_strides, B, b_strides, M, N, K, c_strides=None):
    c_strides = c_strides or (1, M)
    C = np.zeros(M * N, dtype=np.float64)
    lib().moye_oracle_gemm_f64(_p(A), _i64(a_strides[0]), _i64(a_strides[1]), _p(B), _i64(b_strides[0]),
                               _i64(b_strides[1]), _p(C), _i64(c_strides[0]), _i64(c_strides[1]), _i64(M), _i64(N),
                               _i64(K))
    return C


def matmul_kernel_f32(A, B, M, N, K, bM=128, bN=128, bK=8, tA=(32, 8), tC=(16, 16), use_tower=True):
    """The emulated `matmul_kernel`: column-major A (M,K), B (N,K) -> column-major C (M,N)."""
    C = np.full(M * N, np.nan, dtype=np.float32)
    rc = lib().moye_oracle_matmul_kernel_f32(_p(A), _p(B), _p(C), _i64(M), _i64(N), _i64(K), bM, bN, bK, tA[0], tA[1],
                                             tC[0], tC[1], 1 if use_tower else 0)
    if rc != 0:
        raise ValueError("tiles do not divide the problem")
    return C


def gemm_samples(A, B, dtype, M, N, K, idx, by_rows=True, threads=1):
    """Widened-input host gemm! for selected rows (or columns) of C = A.B^T; A (M,K) and
    B (N,K) K-major, given as flat arrays of the raw element type.  Returns
    float32 (int32 for s8) of shape (len(idx), N) or (len(idx), M)."""
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    other = N if by_rows else M
    out = np.empty((len(idx), other), dtype=np.int32 if dtype == S8 else np.float32)
    rc = lib().moye_oracle_gemm_samples(_p(A), _i64(K), _p(B), _i64(K), dtype, _i64(M), _i64(N), _i64(K), _p(idx),
                                        _i64(len(idx)), 1 if by_rows else 0, _p(out), int(threads))
    assert rc == 0
    return out


def matmul_threads_f32(A, B, M, N, K, thread_layout=(4, 4), m_limit=0):
    """The reference's threaded host GEMM (column-major operands).  Returns flat C."""
    C = np.empty(M * N, dtype=np.float32)
    rc = lib().moye_oracle_matmul_threads_f32(_p(A), _p(B), _p(C), _i64(M), _i64(N), _i64(K), thread_layout[0],
                                              thread_layout[1], _i64(m_limit))
    assert rc == 0
    return C


def fused_epilogue(acc, alpha=1.0, beta=0.0, C=None, bias=None, bias_mode=None, activation=None):
    """D = act(alpha*acc + beta*C + bias) on an (M, N) float32 accumulator, in float64.  alpha / beta follow
    the reference's `axpby!` (src/algorithm/blas.jl:1-9: the beta*C term is skipped when beta == 0); bias and
    activation have no counterpart there and are defined here: bias_mode "col" adds bias[n], "row" adds bias[m];
    relu = max(x, 0), gelu = x/2 (1 + erf(x / sqrt 2)), silu = x / (1 + exp(-x))."""
    import math
    x = np.asarray(acc, dtype=np.float64) * float(alpha)
    if beta != 0.0:
        x = x + float(beta) * np.asarray(C, dtype=np.float64)
    if bias is not None:
        b = np.asarray(bias, dtype=np.float64)
        x = x + (b[None, :] if bias_mode == "col" else b[:, None])
    if activation == "relu":
        x = np.maximum(x, 0.0)
    elif activation == "gelu":
        x = 0.5 * x * (1.0 + np.frompyfunc(math.erf, 1, 1)(x / math.sqrt(2.0)).astype(np.float64))
    elif activation == "silu":
        x = x / (1.0 + np.exp(-x))
    elif activation not in (None, "none"):
        raise ValueError(activation)
    return x.astype(np.float32)


def axpby(a, x, b, y):
    """`axpby!(a, X, b, Y)` of reference src/algorithm/blas.jl:1-9 over two equally shaped float32 arrays (16-bit
    element types are widened by the caller, exactly): every element `a*x` when b == 0 (Y is not read), else
    `a*x + b*y` with both products rounded to Float32 before the add -- Julia does not contract the expression.
    Returns float32; the caller rounds to the element type (round to nearest even) like the store does."""
    a32, b32 = np.float32(a), np.float32(b)
    x = np.asarray(x, dtype=np.float32)
    ax = a32 * x
    if b32 == 0:
        return ax
    return ax + b32 * np.asarray(y, dtype=np.float32)


def tf32_trunc(x):
    """Float32 values as the tf32 tensor-core kind reads them: sign, 8 exponent bits and the top 10 mantissa
    bits; the low 13 bits are dropped without rounding (measured on sm_100a: truncation reproduces the device
    result to fp32 accumulation order, round-to-nearest does not)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    return (x.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)


def max_rel_err(got, ref):
    """max |got-ref| / max(|ref|, 1e-3 * max|ref|): the tolerance metric of every GEMM test."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.maximum(np.abs(ref), 1e-3 * np.abs(ref).max())
    return float((np.abs(got - ref) / den).max())
