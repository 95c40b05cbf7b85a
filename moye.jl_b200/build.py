"""Builds libmoye_b200.so in-tree (moye.jl_b200/lib/) with nvcc for sm_100a.

Usage: python moye.jl_b200/build.py [--force] [--verbose] [--debug]
nvcc cross-compiles, so this works on a machine without a GPU.  Every source is compiled to its
own object (kept under lib/obj/, rebuilt only when it or a header changed), the objects side by
side, then linked.  `--debug` builds lib/libmoye_b200_debug.so with -DMOYE_DEBUG: the kernels
then check every TMA coordinate, tensor-memory column and stage index on the device and report
a violation through the status word instead of touching memory.
"""
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OUT = os.path.join(LIBDIR, "libmoye_b200.so")
OUT_DEBUG = os.path.join(LIBDIR, "libmoye_b200_debug.so")
SOURCES = ["api.cu", "gemm_sm100.cu", "gemm_single.cu", "gemm_pair.cu", "gemm_wide.cu", "gemm_splitk.cu",
           "gemm_skinny.cu", "copy_sm100.cu", "transpose_sm100.cu", "layout_sm100.cu", "axpby_sm100.cu", "ldsm_sm100.cu",
           "comm_nccl.cu"]
HEADERS = ["common.h", "ptx.cuh", "gemm_common.cuh", os.path.join("..", "..", "include", "moye_b200.h")]
CFLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]


def _newer(path, deps):
    if not os.path.exists(path):
        return True
    t = os.path.getmtime(path)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False, debug=False):
    """Compile every CUDA source of the library for sm_100a; returns the path of the .so."""
    out = OUT_DEBUG if debug else OUT
    objdir = os.path.join(LIBDIR, "obj_debug" if debug else "obj")
    headers = [os.path.join(CSRC, x) for x in HEADERS] + [os.path.abspath(__file__)]
    srcs = [os.path.join(CSRC, s) for s in SOURCES]
    objs = [os.path.join(objdir, s[:-3] + ".o") for s in SOURCES]
    todo = [(s, o) for s, o in zip(srcs, objs) if force or _newer(o, [s] + headers)]
    if not todo and not _newer(out, objs):
        return out
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; libmoye_b200 cannot be built")
    os.makedirs(objdir, exist_ok=True)
    flags = CFLAGS + (["-DMOYE_DEBUG"] if debug else []) + (["-Xptxas", "-v"] if verbose else [])

    def compile_one(job):
        src, obj = job
        res = subprocess.run([nvcc] + flags + ["-c", src, "-o", obj], capture_output=True, text=True)
        return src, res

    with ThreadPoolExecutor(max_workers=max(1, min(len(todo), os.cpu_count() or 1))) as pool:
        results = list(pool.map(compile_one, todo))
    failed = False
    for src, res in results:
        if verbose or res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
        failed = failed or res.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed building libmoye_b200")
    # NCCL is not linked: comm_nccl.cu looks the library up at run time, so that the .so loads without it
    res = subprocess.run([nvcc, "-shared", "-o", out] + objs + ["-ldl"], capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("linking libmoye_b200 failed")
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, debug="--debug" in sys.argv))
