import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def rel_l2(a, b):
    """Relative L2 distance of a to the reference value b."""
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


@pytest.fixture(scope="session")
def oracle():
    from oracle.oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    """The unmodified reference compiled from its own sources; only where that build exists."""
    from oracle.oracle import Reference
    if not Reference.available():
        try:
            from oracle.oracle import build
            build()
        except Exception:
            pass
    if not Reference.available():
        pytest.skip("reference library not built on this machine (tests/golden fixtures cover it)")
    return Reference()


@pytest.fixture(scope="session")
def ctx():
    from lutmac_b200.api import Context
    return Context(0)


@pytest.fixture(scope="session")
def ctx_lut():
    """A context whose ternary weights use the table-lookup kernel (the reference's LUT
    formulation) instead of the default integer tensor-core kernel."""
    from lutmac_b200 import _lib
    from lutmac_b200.api import Context
    c = Context(0)
    c.set_option(_lib.OPT_TERNARY_LUT, 1)
    return c
