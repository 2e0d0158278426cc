"""pytest configuration: the `gpu` marker and shared fixtures.

CPU tests (-m "not gpu") pin the oracle against the golden fixtures and check
the host logic and the C ABI's symbol table; GPU tests (-m gpu) are the parity
tests of the CUDA kernels, called through the C ABI.
"""
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def ora():
    from oracle.oracle import Oracle

    return Oracle()


@pytest.fixture(scope="session")
def ref():
    """The reference's own CPU code, where oracle/_ref/libie_ref.so exists."""
    from oracle.oracle import Ref

    if not Ref.available():
        pytest.skip("oracle/_ref/libie_ref.so not built (reference tree absent)")
    return Ref()


@pytest.fixture(scope="session")
def golden_kernels():
    return np.load(GOLDEN / "kernels.npz")


@pytest.fixture(scope="session")
def lib():
    from amd_c_b200 import _lib

    return _lib.load()


@pytest.fixture(scope="session")
def cuda(lib):
    """A CUDA device through torch (device memory and streams only)."""
    import torch

    from amd_c_b200 import _lib

    _lib.require_gpu()
    assert torch.cuda.is_available()
    return torch.device("cuda:0")


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
