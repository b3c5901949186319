import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# tolerance of the parity gate for fp32-accumulated tensor-core math: |gpu - cpu| <= ABS + REL * |cpu|
ABS_TOL = 1e-4
REL_TOL = 1e-3


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def assert_close(got, want, what="", abs_tol=ABS_TOL, rel_tol=REL_TOL):
    got = np.asarray(got, dtype=np.float32).ravel()
    want = np.asarray(want, dtype=np.float32).ravel()
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    assert np.all(np.isfinite(got)), f"{what}: non-finite values in the GPU result"
    err = np.abs(got - want)
    bound = abs_tol + rel_tol * np.abs(want)
    bad = err > bound
    if bad.any():
        i = int(np.argmax(err - bound))
        raise AssertionError(
            f"{what}: {int(bad.sum())} of {got.size} outside |d| <= {abs_tol} + {rel_tol}|ref|; "
            f"worst at {i}: got {got[i]!r}, want {want[i]!r}, max abs err {float(err.max()):.3e}"
        )


@pytest.fixture(scope="session")
def backend():
    """Initialises the CUDA backend once; fails (does not skip) when the library is missing."""
    from mimir_framework_b200 import runtime

    runtime.init(0, 0)
    yield runtime
    runtime.shutdown()
