import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_PATH = os.path.join(ROOT, "tests", "golden", "na2d_golden.npz")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200); deselected on CPU-only hosts with -m 'not gpu'")


@pytest.fixture(scope="session")
def golden():
    """Vectors produced by running the reference itself (tests/golden/make_golden.py)."""
    return np.load(GOLDEN_PATH)


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """Build libna2d.so if it is missing or stale (nvcc cross-compiles without a GPU)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("na2d_build", os.path.join(ROOT, "e_natten_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)       # by path: importing the package would need the library first
    mod.build()
