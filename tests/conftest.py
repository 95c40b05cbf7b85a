import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
ORACLE = os.path.join(ROOT, "oracle")
if ORACLE not in sys.path:
    sys.path.insert(0, ORACLE)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu on a B200")


@pytest.fixture(scope="session")
def mb():
    """The product package (moye.jl_b200 loaded as moye_b200)."""
    import __graft_entry__ as ge
    return ge.load_package()


@pytest.fixture(scope="session")
def ho():
    """The C oracle's Python face (test infrastructure)."""
    import host_oracle
    host_oracle.lib()
    return host_oracle


@pytest.fixture(scope="session")
def lo():
    """The layout-algebra oracle (test infrastructure)."""
    import layout_oracle
    return layout_oracle


@pytest.fixture(scope="session")
def dev():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device; there is no CPU fallback to test")
    torch.cuda.set_device(0)
    return torch.device("cuda", 0)
