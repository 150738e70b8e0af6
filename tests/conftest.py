import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))


@pytest.fixture(scope="session")
def golden():
    """Outputs of the reference's own CUDA kernels on a B200 (tests/golden/make_golden.py)."""
    return dict(np.load(os.path.join(ROOT, "tests", "golden", "ref_small.npz")))


@pytest.fixture(scope="session")
def oracle_cpu():
    from oracle import cpu
    cpu.lib()
    return cpu


@pytest.fixture(scope="session")
def engine():
    """The CUDA library through its C ABI; GPU tests fail loudly if it is not built."""
    from tsne_cuda_b200 import _lib
    return _lib


def mixture(n, d, seed, k=4):
    rng = np.random.default_rng(seed)
    mu = rng.normal(0, 10, (k, d))
    return (mu[np.arange(n) % k] + rng.normal(0, 1, (n, d))).astype(np.float32)
