"""The C ABI as a binary contract: the library loads without a GPU, exports every symbol the
header declares, refuses to create a handle when no device exists (there is no CPU path),
and its structs have the layout the ctypes binding assumes."""
import ctypes
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "moye_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(moye_b200_[a-z_0-9]+)\s*\(", text)))


def test_header_declares_expected_entry_points():
    names = declared_functions()
    for n in ("moye_b200_create", "moye_b200_destroy", "moye_b200_gemm", "moye_b200_copy", "moye_b200_layout_copy",
              "moye_b200_layout_eval", "moye_b200_status", "moye_b200_last_error", "moye_b200_version"):
        assert n in names


def test_library_exports_every_declared_symbol(mb):
    lib = mb._lib.load()
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in include/moye_b200.h but not exported"
        assert name in mb._lib.EXPORTS, f"{name} has no ctypes prototype"
    assert lib.moye_b200_version() == 100


def test_header_compiles_as_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "moye_b200.h"\nint main(void){moye_tensor_t t; moye_gemm_params_t p; (void)t; (void)p; '
                   "return sizeof(moye_layout_t) == 8 + 2 * 8 * MOYE_MAX_FLAT_RANK ? 0 : 1;}\n")
    exe = tmp_path / "t"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)],
                   check=True)
    assert subprocess.run([str(exe)]).returncode == 0


def test_struct_layouts(mb):
    L = mb._lib
    assert ctypes.sizeof(L.Tensor) == 8 + 4 + 4 + 8 * 4 + 8 * 4
    assert ctypes.sizeof(L.FlatLayout) == 8 + 16 * L.MAX_FLAT_RANK
    assert ctypes.sizeof(L.GemmParams) == 40 and L.GemmParams.bias.offset == 32 and ctypes.sizeof(L.CopyParams) == 16
    assert L.Tensor.shape.offset == 16 and L.Tensor.stride.offset == 48


def test_no_device_is_an_error_not_a_fallback(mb):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    lib = mb._lib.load()
    out = ctypes.c_void_p()
    rc = lib.moye_b200_create(ctypes.byref(out))
    assert rc == -8 and not out.value
    assert b"no CPU path" in lib.moye_b200_last_error()
    assert lib.moye_b200_destroy(None) == 0


def test_product_does_not_import_the_oracle():
    """The package must not reach into oracle/ (the oracle is the checker, never the product)."""
    pkg = os.path.join(ROOT, "moye.jl_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower().replace("no cpu", ""), f"{f} mentions the oracle"


def test_forbidden_copy_qualifier_is_absent():
    # The qualifier assembled below (the cluster-wide broadcast form of bulk copies) must not appear in
    # any source: such a copy reading another GPU's memory has hung GPUs, and multi-GPU launches are
    # refused while a source file names one.
    token = "multi" + "cast" + "::" + "clus" + "ter"
    for base in ("moye.jl_b200", "oracle", "tests", "include"):
        for dirpath, _, files in os.walk(os.path.join(ROOT, base)):
            for f in files:
                if f.endswith((".cu", ".cuh", ".h", ".c", ".py", ".jl")):
                    assert token not in open(os.path.join(dirpath, f), errors="ignore").read(), f
    for f in ("bench.py", "__graft_entry__.py"):
        assert token not in open(os.path.join(ROOT, f)).read()


def test_log_environment_variable_reports_errors_on_stderr():
    """MOYE_B200_LOG=2: every error message goes to stderr as it is set; unset: silence.  (Level 1 also prints one
    line per entry-point call with the kernel chosen; that needs a device and is covered by the GPU tests.)"""
    import sys
    script = ("import ctypes, sys; sys.path.insert(0, %r); import __graft_entry__ as g; lib = g.load_package()._lib.load(); "
              "assert lib.moye_b200_gemm(None, None, None, None, None, None, None) == -1" % ROOT)
    loud = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=dict(os.environ, MOYE_B200_LOG="2"))
    assert loud.returncode == 0 and "[moye_b200] error: null handle" in loud.stderr
    env = {k: v for k, v in os.environ.items() if k != "MOYE_B200_LOG"}
    quiet = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=env)
    assert quiet.returncode == 0 and "[moye_b200]" not in quiet.stderr


def build_c_abi_smoke(tmp_path):
    """Compiles tests/c_abi_smoke.cpp against the header and the in-tree library with g++ (no nvcc, no Python)."""
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    libdir = os.path.join(ROOT, "moye.jl_b200", "lib")
    exe = tmp_path / "c_abi_smoke"
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"),
                    os.path.join(ROOT, "tests", "c_abi_smoke.cpp"), "-o", str(exe), "-L", libdir, "-lmoye_b200",
                    "-L", os.path.join(cuda, "lib64"), "-lcudart", f"-Wl,-rpath,{libdir}",
                    f"-Wl,-rpath,{os.path.join(cuda, 'lib64')}"], check=True)
    return str(exe)


def test_cpp_caller_links_and_reports_no_device(mb, tmp_path):
    """A C++ program that uses only include/moye_b200.h and the shared library builds and links; without a device it
    gets MOYE_ERR_NO_DEVICE from moye_b200_create (exit code 3), not a crash and not a CPU result."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present: the GPU test runs the same program to the end")
    mb._lib.load()
    res = subprocess.run([build_c_abi_smoke(tmp_path)], capture_output=True, text=True)
    assert res.returncode == 3 and "no CPU path" in res.stdout, res.stdout + res.stderr
