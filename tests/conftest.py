import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.binding import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def ref():
    """The reference's own compiled functions; skipped where oracle/_ref was never built."""
    from oracle.binding import Ref, build_ref
    try:
        build_ref()
    except Exception:
        pass
    if not Ref.available():
        pytest.skip("oracle/_ref/libggnpu_ref.so not present (reference tree unavailable)")
    return Ref()


@pytest.fixture(scope="session")
def vectors():
    return np.load(os.path.join(GOLDEN, "ref_vectors.npz"))


@pytest.fixture(scope="session")
def grid_vectors():
    return np.load(os.path.join(GOLDEN, "ref_grid_vectors.npz"))


@pytest.fixture(scope="session")
def cli_vectors():
    return np.load(os.path.join(GOLDEN, "ref_cli.npz"))


@pytest.fixture(scope="session")
def backend():
    """The CUDA backend through the C ABI.  GPU tests only; never falls back."""
    from ggnpu_b200.build import build
    from ggnpu_b200.backend import CudaBackend
    build()
    b = CudaBackend(0)
    yield b
    b.close()


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))
