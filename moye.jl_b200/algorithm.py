"""`copyto_` and `gemm_`: MoYe's L5 algorithms (`copyto!`, `gemm!`) at host level.

In MoYe these are per-thread device functions inlined into a user kernel (reference
src/algorithm/copy.jl, src/algorithm/blas.jl).  Here the same calls, made on arrays that live
in global memory, hand the whole tiled operation to libmoye_b200 through its C ABI:

    copyto_(tiled_copy, dst, src)   ->  moye_b200_copy         (reference copy.jl:106-130)
    copyto_(dst, src)               ->  moye_b200_copy or moye_b200_layout_copy (copy.jl:42-64)
    gemm_(tiled_mma, D, A, B, C)    ->  moye_b200_gemm         (reference blas.jl:11-131)
    matmul(A, B, C)                 ->  the `matmul` of examples/gemm.jl:66-89

There is no CPU implementation behind these names: operands in host memory are rejected.
"""
import ctypes

import torch

from . import _lib
from .array import MoYeArray, isgmem
from .atom import TiledCopy, TiledMMA, make_tiled_mma, sm100_mma_op
from .layout import coalesce, size

__all__ = ["copyto_", "copy_dispatch", "gemm_", "matmul", "layout_eval", "synchronize_status", "current_stream_ptr",
           "gemm_skinny_static_", "gemm_skinny_static_status", "plan_gemm", "plan_copy", "LaunchPlan", "axpby_"]


def current_stream_ptr(device=None):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _need_gmem(*arrays):
    for x in arrays:
        if not isgmem(x):
            raise RuntimeError("libmoye_b200 runs on device global memory only; got an array on "
                               f"{x.device} (there is no CPU fallback)")
    dev = arrays[0].device
    for x in arrays[1:]:
        if x.device != dev:
            raise RuntimeError("operands live on different devices")
    return dev


def _as_rank2(x):
    """(shape, stride) of a rank-2 view whose modes are single strides, or None."""
    l = x.layout
    if len(l) != 2:
        return None
    modes = [coalesce(l[0]), coalesce(l[1])]
    if any(isinstance(m.shape, tuple) for m in modes):
        return None
    return [int(m.shape) for m in modes], [int(m.stride) for m in modes]


def _tensor_arg(x, what):
    if x._abi is not None:
        return x._abi
    sd = _as_rank2(x)
    if sd is None:
        raise _lib.MoyeError(-3, f"{what} must be a rank-2 array with one stride per mode, got layout {x.layout}")
    x._abi = _lib.make_tensor(x.ptr, x.dtype, sd[0], sd[1])
    return x._abi


def copy_dispatch(dst, src, tiled_copy=None):
    """Which device path a `copyto!` takes, decided on the host from shapes, strides and alignment alone:
    "tiled" (`moye_b200_copy`: 128-bit / TMA tiles, or the transposing kernel) or "elementwise"
    (`moye_b200_layout_copy`: one index computation per element through both layouts).  Returns (path, reason);
    `reason` says why two rank-2 arrays that look tileable are not (None otherwise)."""
    sd_d, sd_s = _as_rank2(dst), _as_rank2(src)
    if sd_d is None or sd_s is None or sd_d[0] != sd_s[0]:
        return "elementwise", None
    same_first = sd_d[1][0] == 1 and sd_s[1][0] == 1
    one_unit_each = tiled_copy is None and 1 in sd_d[1] and 1 in sd_s[1]
    if not (same_first or one_unit_each):
        return "elementwise", None
    eb = dst.elem_bytes
    for x, sd in ((dst, sd_d), (src, sd_s)):
        if x.ptr % 16:
            return "elementwise", "a base address is not 16-byte aligned"
        pitch = [st for sh, st in zip(sd[0], sd[1]) if st != 1 and sh > 1]
        if any((st * eb) % 16 for st in pitch):
            return "elementwise", "a pitch is not a multiple of 16 bytes"
    if not same_first and eb not in (1, 2, 4, 8):
        return "elementwise", "the transposing kernel moves elements of 1, 2, 4 or 8 bytes"
    return "tiled", None


_warned_slow_copy = set()


def copyto_(*args, stream=None, elementwise_ok=False):
    """`copyto!(dst, src)` or `copyto!(tiled_copy, dst, src)` on global-memory arrays.

    With a TiledCopy the tiled kernel runs or the call fails.  Without one the meaning is the reference's elementwise
    copy through both layouts (src/algorithm/copy.jl:4-16); two rank-2 arrays of equal shape, each contiguous along
    one mode and 16-byte aligned, take the tiled kernels, everything else the per-element kernel.  The choice is made
    here, on the host (`copy_dispatch`): no call is tried and retried.  When only alignment keeps two matrices off the
    fast path a warning says so once per reason, unless `elementwise_ok=True`."""
    if len(args) == 3:
        tiled_copy, dst, src = args
    else:
        (dst, src), tiled_copy = args, None
    dev = _need_gmem(dst, src)
    lib, h = _lib.load(), _lib.handle(dev.index)
    st = stream if stream is not None else current_stream_ptr(dev)
    if size(dst.layout) != size(src.layout):
        raise _lib.MoyeError(-4, f"copyto!: sizes differ ({size(dst.layout)} vs {size(src.layout)})")
    if dst.storage.dtype != src.storage.dtype:
        raise _lib.MoyeError(-2, "copyto!: element types differ")
    if size(src.layout) == 0:
        return dst
    params = None
    if tiled_copy is not None:
        if not isinstance(tiled_copy, TiledCopy):
            raise TypeError("first argument must be a TiledCopy")
        mode = tiled_copy.copy_atom.op.mode
        if mode == _lib.COPY_LDSM:
            return _ldsm_copy(tiled_copy, dst, src, lib, h, st)
        if mode is None:
            raise _lib.MoyeError(-3, f"{tiled_copy.copy_atom.op} has no device copy kernel: the kernels move 128-bit "
                                     "atoms, TMA tiles or ldmatrix fragments")
        tm, tn = tiled_copy.tiler_mn[0], tiled_copy.tiler_mn[1] if len(tiled_copy.tiler_mn) > 1 else 1
        if mode == _lib.COPY_UNIVERSAL128:
            # the tiler of one pass is (threads x vector) wide; the kernel loops it over a CTA tile of
            # 64 columns like the reference's copy kernel loops its partition
            tn = max(tn, 64)
        params = _lib.CopyParams(mode, tm, tn, 0)
        sd_d, sd_s = _as_rank2(dst), _as_rank2(src)
        if not (sd_d is not None and sd_s is not None and sd_d[0] == sd_s[0] and sd_d[1][0] == 1 and sd_s[1][0] == 1):
            raise _lib.MoyeError(-3, "a tiled copy needs rank-2 operands of equal shape, contiguous along the first mode")
        path = "tiled"
    else:
        path, reason = copy_dispatch(dst, src)
        if reason is not None and not elementwise_ok and reason not in _warned_slow_copy:
            import warnings
            _warned_slow_copy.add(reason)
            warnings.warn(f"copyto!: {reason}; these matrices take the per-element kernel, which is many times slower "
                          "than the tiled one (pass elementwise_ok=True to silence this)", RuntimeWarning, stacklevel=2)
    if path == "tiled":
        sd_d, sd_s = _as_rank2(dst), _as_rank2(src)
        td = _lib.make_tensor(dst.ptr, dst.dtype, sd_d[0], sd_d[1])
        ts = _lib.make_tensor(src.ptr, src.dtype, sd_s[0], sd_s[1])
        _lib.check(lib.moye_b200_copy(h, ctypes.byref(td), ctypes.byref(ts), ctypes.byref(params) if params else None, st))
        return dst
    # elementwise through both layouts
    ds, dd = dst.layout.flat()
    ss, sdd = src.layout.flat()
    if len(ds) > _lib.MAX_FLAT_RANK or len(ss) > _lib.MAX_FLAT_RANK:
        raise _lib.MoyeError(-4, "layout has too many modes")
    ld, ls = _lib.make_flat_layout(ds, dd), _lib.make_flat_layout(ss, sdd)
    _lib.check(lib.moye_b200_layout_copy(h, ctypes.c_void_p(dst.ptr), ctypes.byref(ld), ctypes.c_void_p(src.ptr),
                                         ctypes.byref(ls), dst.elem_bytes, st))
    return dst


def _ldsm_copy(tiled_copy, dst, src, lib, h, st):
    """`copyto!(tiled_copy, dst, src)` for an ldmatrix TiledCopy: dst and src are the same tile layout over two
    buffers (the `t_g_in` / `t_g_out` of reference test/device/tiled_copy.jl:2-23); the tile goes through shared
    memory and every thread's `ldmatrix` fragments."""
    from .atom import ldsm_tiled_copy_tables
    if dst.elem_bytes != 2:
        raise _lib.MoyeError(-2, "ldmatrix moves 16-bit elements")
    if dst.layout != src.layout:
        raise _lib.MoyeError(-3, "an ldmatrix tiled copy takes source and destination with the same tile layout")
    try:
        span, iters, so, do = ldsm_tiled_copy_tables(tiled_copy, src.layout)
    except ValueError as exc:
        raise _lib.MoyeError(-3, str(exc))
    op = tiled_copy.copy_atom.op
    src_t = (ctypes.c_int32 * len(so))(*so)
    dst_t = (ctypes.c_int32 * len(do))(*do)
    _lib.check(lib.moye_b200_ldsm_copy(h, ctypes.c_void_p(dst.ptr), ctypes.c_void_p(src.ptr), span, op.matrices,
                                       1 if op.transposed else 0, len(tiled_copy), iters, src_t, dst_t, st))
    return dst


_AB_TAG = {_lib.F16: "F16", _lib.BF16: "BF16", _lib.S8: "S8", _lib.U8: "U8", _lib.E4M3: "E4M3", _lib.F32: "TF32"}


def _epilogue(bias, activation, D, dev):
    """(flags, bias pointer, keep-alive) of the fused epilogue D = act(... + bias).  `bias` is a float32 CUDA
    tensor with one value per column of D (length N) or per row (length M); when M == N pass `(tensor, "col")`
    or `(tensor, "row")`."""
    if activation not in _lib.EPI_ACT:
        raise _lib.MoyeError(-1, f"unknown activation {activation!r}; one of relu, gelu, silu")
    flags, ptr = _lib.EPI_ACT[activation], None
    if bias is not None:
        which = None
        if isinstance(bias, tuple):
            bias, which = bias
        if not (torch.is_tensor(bias) and bias.is_cuda and bias.dtype == torch.float32 and bias.is_contiguous()
                and bias.device == dev):
            raise _lib.MoyeError(-1, "bias must be a contiguous float32 tensor on the device of D")
        m, n = D.layout.shape[0], D.layout.shape[1]
        if which is None:
            if m == n and bias.numel() == n:
                raise _lib.MoyeError(-1, "D is square: say (bias, 'col') or (bias, 'row')")
            which = "col" if bias.numel() == n else ("row" if bias.numel() == m else None)
        if which not in ("col", "row") or bias.numel() != (n if which == "col" else m):
            raise _lib.MoyeError(-3, f"bias has {bias.numel()} values; D is {m} x {n}")
        flags |= _lib.EPI_BIAS_COL if which == "col" else _lib.EPI_BIAS_ROW
        ptr = bias.data_ptr()
    return flags, ptr, bias


def _choice_flags(allow_tf32, tail):
    """The kernel-choice bits: `allow_tf32` lets Float32 operands run as ONE tf32 product (10-bit mantissas, about
    1e-3 relative) instead of the three-product split that keeps Float32 accuracy; `tail` forces the stream-K tail
    of the 256 x 512 kernel on (True) or off (False), None leaves the choice to the library."""
    f = _lib.GEMM_ALLOW_TF32 if allow_tf32 else 0
    if tail is not None:
        f |= _lib.GEMM_TAIL_ON if tail else _lib.GEMM_TAIL_OFF
    return f


def gemm_(*args, alpha=1.0, beta=0.0, scale_a=1.0, scale_b=1.0, tile_n=0, path=0, stream=None, bias=None,
          activation=None, split_k=0, allow_tf32=False, tail=None):
    """`gemm!([tiled_mma,] D, A, B, C)`: D = alpha*scale_a*scale_b * A.B^T + beta*C with
    A:(M,K), B:(N,K), C and D:(M,N) in global memory.  `gemm_(A, B, C)` is `gemm!(C, A, B, C)`
    like the reference's three-argument form (src/algorithm/blas.jl:11).  `bias` (float32, one
    value per column or per row of D) and `activation` ("relu", "gelu", "silu") are fused into the
    epilogue: D = act(alpha*... + beta*C + bias), in fp32 before the output conversion.  `path` picks the
    kernel (0: the library chooses; 1 single CTAs, 2 stream-K, 3 CTA pairs, 4 pairs on 256x512 tiles, 5 split-K on
    clusters with `split_k` = 2, 4 or 8 CTAs per tile).  Float32 operands are multiplied to Float32 accuracy unless
    `allow_tf32=True` (see `_choice_flags`, also for `tail`)."""
    tiled_mma = None
    if args and isinstance(args[0], TiledMMA):
        tiled_mma, args = args[0], args[1:]
    if len(args) == 3:
        A, B, C = args
        D = C
    elif len(args) == 4:
        D, A, B, C = args
    else:
        raise TypeError("gemm_([tiled_mma,] D, A, B, C) or gemm_([tiled_mma,] A, B, C)")
    ops = [D, A, B] + ([C] if (C is not None and beta != 0.0) else [])
    dev = _need_gmem(*ops)
    if tiled_mma is not None:
        op = tiled_mma.atom.op
        if op.arch != "sm_100a":
            raise _lib.MoyeError(-2, f"{op} is not a tcgen05 op; device-level gemm! needs an MMAOP_SM100_* atom")
        if op.valtype_a != A.dtype or op.valtype_b != B.dtype:
            raise _lib.MoyeError(-2, f"{op} does not take these operand types")
        if tile_n == 0:
            tile_n = op.shape_mnk[1]  # one atom per CTA: the tile is the instruction's N
    lib, h = _lib.load(), _lib.handle(dev.index)
    st = stream if stream is not None else current_stream_ptr(dev)
    flags, bias_ptr, _ = _epilogue(bias, activation, D, dev) if (bias is not None or activation) else (0, None, None)
    flags |= _choice_flags(allow_tf32, tail)
    p = _lib.GemmParams(alpha, beta, scale_a, scale_b, tile_n, split_k, path, flags, bias_ptr)
    tD, tA, tB = _tensor_arg(D, "D"), _tensor_arg(A, "A"), _tensor_arg(B, "B")
    tC = _tensor_arg(C, "C") if (C is not None and beta != 0.0) else None
    _lib.check(lib.moye_b200_gemm(h, ctypes.byref(tD), ctypes.byref(tA), ctypes.byref(tB),
                                  ctypes.byref(tC) if tC is not None else None, ctypes.byref(p), st))
    return D


def matmul(A, B, C, **kw):
    """`matmul(A, B, C)` of reference examples/gemm.jl:66-89: C = A * B' for device arrays,
    with the tcgen05 atom chosen from the operand type.  Accepts MoYeArrays or torch tensors
    (a torch (rows, cols) tensor is taken with its own strides).  Without `tile_n` the library
    picks the tile width and the kernel from the problem shape; with `tile_n` (64, 128, 256) the
    product runs on the atom of that width."""
    A, B, C = (x if isinstance(x, MoYeArray) else MoYeArray(x) for x in (A, B, C))
    if A.dtype not in _AB_TAG:
        raise _lib.MoyeError(-2, "matmul takes f16, bf16, f32, s8, u8 or e4m3 operands on sm_100a")
    tile_n = kw.pop("tile_n", 0)
    if tile_n == 0:
        return gemm_(C, A, B, None, **kw)
    key = (A.dtype, tile_n)
    mma = _MMA_CACHE.get(key)
    if mma is None:
        mma = _MMA_CACHE[key] = make_tiled_mma(sm100_mma_op(_AB_TAG[key[0]], key[1]))
    return gemm_(mma, C, A, B, None, **kw)


_MMA_CACHE = {}


class LaunchPlan:
    """A prepared call: every argument of the C entry point is built once, so repeating the
    launch costs one foreign call.  Kernel authors in MoYe pay the tiling cost at compile time
    (static layouts); this is the host-level analogue for a caller that launches the same
    operation many times (a benchmark loop, a serving step).  The arrays are kept alive by the
    plan.  `plan()` launches on the current stream, `plan(stream_ptr)` on the given one."""

    __slots__ = ("_fn", "_args", "_device", "_keep")

    def __init__(self, fn, args, device, keep):
        self._fn, self._args, self._device, self._keep = fn, args, device, keep

    def __call__(self, stream=None):
        rc = self._fn(*self._args, stream if stream is not None else current_stream_ptr(self._device))
        if rc:
            _lib.check(rc)


def plan_gemm(*args, alpha=1.0, beta=0.0, scale_a=1.0, scale_b=1.0, tile_n=0, path=0, bias=None, activation=None,
              split_k=0, allow_tf32=False, tail=None):
    """`gemm_` with the argument marshalling done once; returns a `LaunchPlan`."""
    tiled_mma = None
    if args and isinstance(args[0], TiledMMA):
        tiled_mma, args = args[0], args[1:]
    if len(args) == 3:
        A, B, C = args
        D = C
    else:
        D, A, B, C = args
    D, A, B = (x if isinstance(x, MoYeArray) else MoYeArray(x) for x in (D, A, B))
    if C is not None and not isinstance(C, MoYeArray):
        C = MoYeArray(C)
    use_c = C is not None and beta != 0.0
    dev = _need_gmem(*([D, A, B] + ([C] if use_c else [])))
    if tiled_mma is not None:
        op = tiled_mma.atom.op
        if op.arch != "sm_100a" or op.valtype_a != A.dtype or op.valtype_b != B.dtype:
            raise _lib.MoyeError(-2, f"{op} cannot multiply these operands on sm_100a")
        tile_n = tile_n or op.shape_mnk[1]
    lib, h = _lib.load(), _lib.handle(dev.index)
    flags, bias_ptr, bias = _epilogue(bias, activation, D, dev) if (bias is not None or activation) else (0, None, None)
    flags |= _choice_flags(allow_tf32, tail)
    p = _lib.GemmParams(alpha, beta, scale_a, scale_b, tile_n, split_k, path, flags, bias_ptr)
    tD, tA, tB = _tensor_arg(D, "D"), _tensor_arg(A, "A"), _tensor_arg(B, "B")
    tC = _tensor_arg(C, "C") if use_c else None
    argv = (h, ctypes.byref(tD), ctypes.byref(tA), ctypes.byref(tB), ctypes.byref(tC) if use_c else None,
            ctypes.byref(p))
    return LaunchPlan(lib.moye_b200_gemm, argv, dev, (D, A, B, C, p, tD, tA, tB, tC, bias))


def plan_copy(*args):
    """`copyto_([tiled_copy,] dst, src)` for the tiled (rank-2, contiguous first mode) case, prepared once.
    Without a TiledCopy the operands may be contiguous along different modes (the transposing copy)."""
    if len(args) == 3:
        tiled_copy, dst, src = args
    else:
        (dst, src), tiled_copy = args, None
    dev = _need_gmem(dst, src)
    sd_d, sd_s = _as_rank2(dst), _as_rank2(src)
    same_first = sd_d is not None and sd_s is not None and sd_d[1][0] == 1 and sd_s[1][0] == 1
    one_unit_each = tiled_copy is None and sd_d is not None and sd_s is not None and 1 in sd_d[1] and 1 in sd_s[1]
    if sd_d is None or sd_s is None or sd_d[0] != sd_s[0] or not (same_first or one_unit_each):
        raise _lib.MoyeError(-3, "a tiled copy needs rank-2 operands of equal shape, contiguous along the first mode "
                                 "(without a TiledCopy: each contiguous along one mode)")
    if dst.storage.dtype != src.storage.dtype:
        raise _lib.MoyeError(-2, "copyto!: element types differ")
    params = None
    if tiled_copy is not None:
        mode = tiled_copy.copy_atom.op.mode
        if mode is None:
            raise _lib.MoyeError(-3, f"{tiled_copy.copy_atom.op} is narrower than 128 bits")
        tm = tiled_copy.tiler_mn[0]
        tn = tiled_copy.tiler_mn[1] if len(tiled_copy.tiler_mn) > 1 else 1
        params = _lib.CopyParams(mode, tm, max(tn, 64) if mode == _lib.COPY_UNIVERSAL128 else tn, 0)
    lib, h = _lib.load(), _lib.handle(dev.index)
    td = _lib.make_tensor(dst.ptr, dst.dtype, sd_d[0], sd_d[1])
    ts = _lib.make_tensor(src.ptr, src.dtype, sd_s[0], sd_s[1])
    argv = (h, ctypes.byref(td), ctypes.byref(ts), ctypes.byref(params) if params is not None else None)
    return LaunchPlan(lib.moye_b200_copy, argv, dev, (dst, src, td, ts, params))


def layout_eval(layout, n=None, first=1, device=None, stream=None):
    """Evaluate `layout(first), ..., layout(first+n-1)` on the device; returns an int64 tensor."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    n = size(layout) if n is None else n
    fs, fd = layout.flat()
    fl = _lib.make_flat_layout(fs, fd)
    out = torch.empty(n, dtype=torch.int64, device=device)
    lib, h = _lib.load(), _lib.handle(device.index)
    st = stream if stream is not None else current_stream_ptr(device)
    _lib.check(lib.moye_b200_layout_eval(h, ctypes.byref(fl), first, n, ctypes.c_void_p(out.data_ptr()), st))
    return out


def synchronize_status(device=None, stream=None):
    """Synchronise the stream and raise if a device-side bounded wait gave up."""
    device = torch.cuda.current_device() if device is None else torch.device(device).index
    lib, h = _lib.load(), _lib.handle(device)
    st = stream if stream is not None else current_stream_ptr(device)
    site = ctypes.c_int32(0)
    _lib.check(lib.moye_b200_status(h, st, ctypes.byref(site)))


def gemm_skinny_static_(D, A, B, alpha=1.0, device_status=None, stream=None):
    """D = alpha * A . B^T for a decode-shaped product (A has at most 32 rows) through the
    entry point that allocates nothing (`moye_b200_gemm_skinny_static`).

    Meant for callers that may not allocate device memory once they are running -- a serving
    loop with a fixed memory budget, a plugin under a no-allocation rule, code without a
    library handle: the stream-K scratch is a 5 MiB static array inside the library instead of
    handle-owned memory.  Limits: A.rows <= 32, B.rows <= 524288.  All calls share that one
    array, so calls that could overlap on the GPU must be ordered (same stream or events); the
    first call on a device does a one-time set-up and should happen before any stream capture.
    `device_status` may be a 1-element int32 CUDA tensor that receives a non-zero code if a
    bounded wait inside the kernel gave up.
    """
    D, A, B = (x if isinstance(x, MoYeArray) else MoYeArray(x) for x in (D, A, B))
    dev = _need_gmem(D, A, B)
    st = stream if stream is not None else current_stream_ptr(dev)
    status_ptr = ctypes.c_void_p(device_status.data_ptr()) if device_status is not None else None
    with torch.cuda.device(dev):
        _lib.check(_lib.load().moye_b200_gemm_skinny_static(
            ctypes.byref(_tensor_arg(D, "D")), ctypes.byref(_tensor_arg(A, "A")), ctypes.byref(_tensor_arg(B, "B")),
            ctypes.c_float(alpha), status_ptr, st))
    return D


def gemm_skinny_static_status(device=None, stream=None):
    """Synchronise `stream` and raise if a bounded wait inside a `gemm_skinny_static_` call that was given no
    `device_status` ran out.  Allocates nothing, like the call it belongs to."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    st = stream if stream is not None else current_stream_ptr(device)
    site = ctypes.c_int32(0)
    with torch.cuda.device(device):
        _lib.check(_lib.load().moye_b200_gemm_skinny_static_status(st, ctypes.byref(site)))


def axpby_(a, X, b, Y, stream=None):
    """`axpby!(a, X, b, Y)`: Y = a*X + b*Y elementwise on global-memory arrays (reference
    src/algorithm/blas.jl:1-9); Y is not read when b == 0.  Returns Y."""
    X, Y = (x if isinstance(x, MoYeArray) else MoYeArray(x) for x in (X, Y))
    dev = _need_gmem(Y, X)
    lib, h = _lib.load(), _lib.handle(dev.index)
    st = stream if stream is not None else current_stream_ptr(dev)

    def arg(x, what):
        l = coalesce(x.layout)
        if not isinstance(l.shape, tuple):  # one mode after coalescing: a vector in memory order
            if int(l.stride) != 1 and int(l.shape) != 1:
                raise _lib.MoyeError(-3, f"axpby!: {what} is not contiguous")
            return _lib.make_tensor(x.ptr, x.dtype, [int(l.shape)], [1])
        return _tensor_arg(x, what)

    tx, ty = arg(X, "X"), arg(Y, "Y")
    if tx.rank != ty.rank:  # one of them coalesced to a vector, the other is pitched: use the rank-2 forms
        tx, ty = _tensor_arg(X, "X"), _tensor_arg(Y, "Y")
    _lib.check(lib.moye_b200_axpby(h, ctypes.byref(ty), ctypes.byref(tx), ctypes.c_float(a), ctypes.c_float(b), st))
    return Y
