"""Builds libmoye_b200.so in-tree (moye.jl_b200/lib/) with nvcc for sm_100a.

Usage: python moye.jl_b200/build.py [--force] [--verbose]
nvcc cross-compiles, so this works on a machine without a GPU.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "lib", "libmoye_b200.so")
SOURCES = ["api.cu", "gemm_sm100.cu", "gemm_skinny.cu", "copy_sm100.cu", "transpose_sm100.cu", "layout_sm100.cu"]
HEADERS = ["common.h", "ptx.cuh", os.path.join("..", "..", "include", "moye_b200.h")]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "-shared", "--threads", "0"]  # the sources compile side by side: about 1.5 minutes from scratch on 8 cores


def _stale():
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile every CUDA source of the library for sm_100a; returns the path of the .so."""
    if not force and not _stale():
        return OUT
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; libmoye_b200 cannot be built")
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    cmd = [nvcc] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", OUT] + \
          [os.path.join(CSRC, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libmoye_b200")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
