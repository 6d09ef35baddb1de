import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def make_sparse(M, K, sparsity, seed, sigma=0.02):
    """fp16 weights ~ N(0, sigma^2) with a seeded Bernoulli mask; kept values never round to zero."""
    rng = np.random.default_rng(seed)
    A = (rng.standard_normal((M, K)) * sigma).astype(np.float16)
    tiny = (A.view(np.uint16) & 0x7FFF) == 0
    A[tiny] = np.float16(6.1035e-05)
    A[rng.random((M, K)) < sparsity] = 0
    return A


def make_dense(N, K, seed, dist="uniform"):
    rng = np.random.default_rng(seed)
    if dist == "uniform":
        return rng.uniform(-1, 1, (N, K)).astype(np.float16)
    return rng.standard_normal((N, K)).astype(np.float16)


@pytest.fixture(scope="session")
def lib_built():
    from spmspm_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        from spmspm_b200.build import build
        build()
    return _lib.load()
