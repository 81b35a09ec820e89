import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "quant_golden.npz"))


@pytest.fixture(scope="session")
def ctx():
    """One library context on cuda:0 for the whole GPU session."""
    import skainet_b200 as skn
    c = skn.Context(0)
    yield c
    c.close()


FP32_TOL = 1e-5   # the stated tolerance of fp32-accumulated dot products against the fp64 oracle
BF16_TOL = 1e-2   # bf16-operand prefill


def assert_close_dot(y, y_ref, absdot, tol, what=""):
    """Parity criterion for dot products: every output within tol * sum_k |w_k x_k| of the
    fp64 oracle, and the whole result within tol in relative L2 norm."""
    y = np.asarray(y, dtype=np.float64)
    err = np.abs(y - y_ref)
    bound = tol * absdot
    worst = np.max(err - bound) if err.size else 0.0
    assert np.all(err <= bound), f"{what}: element error exceeds {tol} * sum|w x| by {worst:.3e}"
    den = np.linalg.norm(y_ref)
    if den > 0:
        rel = np.linalg.norm(y - y_ref) / den
        assert rel <= tol, f"{what}: relative L2 error {rel:.3e} > {tol}"
