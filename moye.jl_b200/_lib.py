"""ctypes binding of libmoye_b200 (the C ABI declared in include/moye_b200.h).

The shared library is built in-tree (``moye.jl_b200/lib/libmoye_b200.so``) by
``build.py``.  There is no CPU fallback: if the library is missing, or no sm_100 device is
visible when a handle is requested, the call raises.
"""
import ctypes
import os
import threading

MAX_RANK = 4
MAX_FLAT_RANK = 12

# moye_dtype_t
F32, F16, BF16, S8, U8, E4M3, S32, U16, U32, U64, U128 = range(11)
DTYPE_BYTES = {F32: 4, F16: 2, BF16: 2, S8: 1, U8: 1, E4M3: 1, S32: 4, U16: 2, U32: 4, U64: 8, U128: 16}

COPY_AUTO, COPY_UNIVERSAL128, COPY_TMA, COPY_TRANSPOSE = 0, 1, 2, 3
COPY_LDSM = 100  # host-side tag of the ldmatrix tiled copy (its own entry point, moye_b200_ldsm_copy)

STATUS_NAMES = {
    0: "OK", -1: "INVALID_ARG", -2: "UNSUPPORTED_DTYPE", -3: "UNSUPPORTED_LAYOUT", -4: "UNSUPPORTED_SHAPE",
    -5: "MISALIGNED", -6: "CUDA", -7: "TIMEOUT", -8: "NO_DEVICE", -9: "TOO_LARGE", -10: "NCCL",
}


class MoyeError(RuntimeError):
    """A non-zero return code from the C ABI (code + the library's message)."""

    def __init__(self, code, message):
        super().__init__(f"libmoye_b200: {STATUS_NAMES.get(code, code)}: {message}")
        self.code = code


class Tensor(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("dtype", ctypes.c_int32), ("rank", ctypes.c_int32),
                ("shape", ctypes.c_int64 * MAX_RANK), ("stride", ctypes.c_int64 * MAX_RANK)]


class FlatLayout(ctypes.Structure):
    _fields_ = [("rank", ctypes.c_int32), ("reserved", ctypes.c_int32),
                ("shape", ctypes.c_int64 * MAX_FLAT_RANK), ("stride", ctypes.c_int64 * MAX_FLAT_RANK)]


class GemmParams(ctypes.Structure):
    _fields_ = [("alpha", ctypes.c_float), ("beta", ctypes.c_float), ("scale_a", ctypes.c_float),
                ("scale_b", ctypes.c_float), ("tile_n", ctypes.c_int32), ("split_k", ctypes.c_int32),
                ("path", ctypes.c_int32), ("flags", ctypes.c_int32), ("bias", ctypes.c_void_p)]


# fused-epilogue selectors of GemmParams.flags (MOYE_EPI_* in the header)
EPI_ACT = {None: 0, "none": 0, "relu": 1, "gelu": 2, "silu": 3}
EPI_BIAS_COL, EPI_BIAS_ROW = 0x10, 0x20
# kernel-choice bits of GemmParams.flags (MOYE_GEMM_* in the header)
GEMM_TAIL_OFF, GEMM_TAIL_ON, GEMM_ALLOW_TF32 = 0x100, 0x200, 0x400


class CopyParams(ctypes.Structure):
    _fields_ = [("mode", ctypes.c_int32), ("tile_m", ctypes.c_int32), ("tile_n", ctypes.c_int32),
                ("flags", ctypes.c_int32)]


# MOYE_B200_DEBUG=1 selects the debug build of the same library (`build.py --debug`): identical entry points, with
# the kernels' address arithmetic checked on the device (a violation is reported through moye_b200_status).
LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib",
                        "libmoye_b200_debug.so" if os.environ.get("MOYE_B200_DEBUG") == "1" else "libmoye_b200.so")

EXPORTS = {
    "moye_b200_create": (ctypes.c_int, [ctypes.POINTER(ctypes.c_void_p)]),
    "moye_b200_destroy": (ctypes.c_int, [ctypes.c_void_p]),
    "moye_b200_version": (ctypes.c_int, []),
    "moye_b200_last_error": (ctypes.c_char_p, []),
    "moye_b200_status": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)]),
    "moye_b200_selftest_bounded_wait": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
    "moye_b200_selftest_dirty_tickets": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
    "moye_b200_gemm": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(Tensor), ctypes.POINTER(Tensor),
                                      ctypes.POINTER(Tensor), ctypes.POINTER(Tensor), ctypes.POINTER(GemmParams),
                                      ctypes.c_void_p]),
    "moye_b200_copy": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(Tensor), ctypes.POINTER(Tensor),
                                      ctypes.POINTER(CopyParams), ctypes.c_void_p]),
    "moye_b200_layout_copy": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(FlatLayout),
                                             ctypes.c_void_p, ctypes.POINTER(FlatLayout), ctypes.c_int32,
                                             ctypes.c_void_p]),
    "moye_b200_gemm_skinny_static": (ctypes.c_int, [ctypes.POINTER(Tensor), ctypes.POINTER(Tensor),
                                                    ctypes.POINTER(Tensor), ctypes.c_float, ctypes.c_void_p,
                                                    ctypes.c_void_p]),
    "moye_b200_gemm_skinny_static_status": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)]),
    "moye_b200_axpby": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(Tensor), ctypes.POINTER(Tensor), ctypes.c_float,
                                       ctypes.c_float, ctypes.c_void_p]),
    "moye_b200_comm_unique_id": (ctypes.c_int, [ctypes.c_char_p]),
    "moye_b200_comm_init": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_char_p]),
    "moye_b200_comm_destroy": (ctypes.c_int, [ctypes.c_void_p]),
    "moye_b200_allgather": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(Tensor), ctypes.POINTER(Tensor),
                                           ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p]),
    "moye_b200_bcast": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(Tensor), ctypes.c_int32, ctypes.c_void_p]),
    "moye_b200_ldsm_copy": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32,
                                           ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                           ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32), ctypes.c_void_p]),
    "moye_b200_layout_eval": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(FlatLayout), ctypes.c_int64,
                                             ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]),
}

_lib = None
_lock = threading.Lock()


def load():
    """dlopen the in-tree library and type its exports.  Raises if it has not been built."""
    global _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise FileNotFoundError(
                    f"{LIB_PATH} is missing: build it with `python moye.jl_b200/build.py` "
                    "(there is no fallback implementation)")
            lib = ctypes.CDLL(LIB_PATH)
            for name, (res, args) in EXPORTS.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def check(rc):
    if rc != 0:
        raise MoyeError(rc, load().moye_b200_last_error().decode())


_handles = {}


def handle(device=None):
    """The per-(thread, device) library handle, created on first use with `device` current."""
    import torch
    if device is None:
        device = torch.cuda.current_device()
    key = (threading.get_ident(), int(device))
    h = _handles.get(key)
    if h is None:
        lib = load()
        out = ctypes.c_void_p()
        with torch.cuda.device(device):
            check(lib.moye_b200_create(ctypes.byref(out)))
        h = out
        _handles[key] = h
    return h


def make_tensor(ptr, dtype, shape, stride):
    t = Tensor()
    t.ptr = ptr
    t.dtype = dtype
    t.rank = len(shape)
    for i, (s, d) in enumerate(zip(shape, stride)):
        t.shape[i] = s
        t.stride[i] = d
    return t


def make_flat_layout(shape, stride):
    l = FlatLayout()
    l.rank = len(shape)
    for i, (s, d) in enumerate(zip(shape, stride)):
        l.shape[i] = s
        l.stride[i] = d
    return l
