import os
import pathlib
import sys

import numpy as np
import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle, built on first use (and the reference's quantizers when its checkout is present)."""
    from oracle import cpu
    cpu.build()
    return cpu


@pytest.fixture(scope="session")
def golden():
    path = ROOT / "tests" / "golden" / "moe_golden.npz"
    return np.load(path)


@pytest.fixture(scope="session")
def lib():
    from strixite_b200 import build, _lib
    build.build()  # incremental: a library older than its sources would fail at load with a missing symbol
    return _lib.load()


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("this test is marked gpu and needs a CUDA device; there is no CPU path to fall back to")
    from strixite_b200 import _lib
    _lib.load()
    return torch.device("cuda:0")
