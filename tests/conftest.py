import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_cpu.npz"))


@pytest.fixture(scope="session")
def lib():
    """The C-ABI library, initialised on the GPU.  Fails (does not skip) when the
    library is missing: GPU tests must never pass on a fallback."""
    import dali_b200
    L = dali_b200.load_library()
    L.init(0)
    return L
