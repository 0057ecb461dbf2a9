import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def pkg():
    """The product package (ctypes binding over librwkv7_b200.so)."""
    entry.build()
    return entry.load_package()


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (checker only)."""
    o = entry.load_oracle()
    o.build()
    return o


@pytest.fixture(scope="session")
def workloads(pkg):
    from rwkv_rs_stable_b200 import workloads as w
    return w


@pytest.fixture(scope="session")
def cuda(pkg):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
