import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU; run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    from oracle import ks_oracle
    ks_oracle.lib()  # builds the parity library if needed
    return ks_oracle


@pytest.fixture(scope="session")
def ctx():
    from ksearch_b200 import CudaContext
    c = CudaContext(0)
    yield c
    c.close()


def assert_close(got, ref64, rtol=1e-3, atol=1e-4, what=""):
    """The path's tolerance: |got - ref| <= atol + rtol*|ref| element-wise, ref in f64."""
    got = np.asarray(got, np.float64).ravel()
    ref = np.asarray(ref64, np.float64).ravel()
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    err = np.abs(got - ref)
    tol = atol + rtol * np.abs(ref)
    bad = np.nonzero(~(err <= tol))[0]
    assert bad.size == 0, (f"{what}: {bad.size}/{got.size} outside 1e-3 rel / 1e-4 abs; worst idx {bad[np.argmax(err[bad])]} "
                           f"got {got[bad[np.argmax(err[bad])]]} ref {ref[bad[np.argmax(err[bad])]]}")


@pytest.fixture(scope="session")
def golden_cases():
    z = np.load(os.path.join(ROOT, "tests", "golden", "cases.npz"))
    return {k: z[k] for k in z.files}
