import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return np.load(os.path.join(ROOT, "tests", "golden", "reference_host.npz"))


@pytest.fixture(scope="session")
def lib():
    """The built C-ABI library (built here if missing or stale; nvcc needs no GPU)."""
    import modern_llm_v1_b200  # noqa: F401
    from modern_llm_v1_b200 import _lib, build

    build.build()
    return _lib.load()
