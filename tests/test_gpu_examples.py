"""The scripts under examples/ run as they are on a B200 (they mirror the reference's examples/gemm.jl and
test/host/copy_async.jl)."""
import importlib.util
import os

import pytest

pytestmark = pytest.mark.gpu
EX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "examples")


def _load(name):
    spec = importlib.util.spec_from_file_location("example_" + name, os.path.join(EX, name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_example_gemm():
    assert _load("gemm").test() < 1e-5


def test_example_pipeline():
    """docs/src/manual/pipeline.md:89-202 on the tcgen05 atoms."""
    ex = _load("pipeline")
    assert ex.host_side()["tAgA"] == ((2, 1), 2, 1, 32)
    assert ex.test() < 1e-5


def test_example_tensor_core():
    """docs/src/manual/tensor_core.md:265-391 (TF32, make_tiled_copy_A / _B, ldmatrix atom) on the kind::tf32 atom."""
    ex = _load("tensor_core")
    assert ex.host_side()["threads"] == 128
    assert ex.test() < 1e-5


def test_example_transpose_and_copy():
    ex = _load("transpose")
    ex.test_copy_async(2048, 2048)
    ex.test_transpose(2048, 2048)
