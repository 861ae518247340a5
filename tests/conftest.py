import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def O():
    """The CPU oracle binding (built on first use)."""
    from oracle import oracle
    oracle.build()
    return oracle


def assert_close_ref(got, want, tol, what=""):
    """The reference's own comparison: |g - w| <= tol * max(|w|, 1)  (xn-core/tests/cuda_tests.rs:2050-2055)."""
    import numpy as np
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    err = np.abs(got - want) / np.maximum(np.abs(want), 1.0)
    i = int(np.argmax(err)) if err.size else 0
    assert err.size == 0 or err.max() <= tol, f"{what}: max err {err.max():.3e} > {tol} at {i}: got {got.flat[i]}, want {want.flat[i]}"
