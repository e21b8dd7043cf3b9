import os
import sys

import pytest

# The tests exercise the planner's own heuristics: no tuned-plan table (tests that want
# entries register them through the API).
os.environ["NMSPMM_TUNED_PLANS"] = ""

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


@pytest.fixture(scope="session")
def pkg_host():
    """The package without the CUDA library (host-side helpers only)."""
    from __graft_entry__ import load_package
    return load_package(native=False)


@pytest.fixture(scope="session")
def pkg():
    """The package with the CUDA library loaded; fails loudly if it was not built."""
    from __graft_entry__ import load_package
    return load_package(native=True)


@pytest.fixture(scope="session")
def orc():
    import oracle
    return oracle.restatement()


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    here = os.path.join(ROOT, "tests", "golden")
    return {"pre": np.load(os.path.join(here, "preprocess.npz")), "gemm": np.load(os.path.join(here, "gemm.npz"))}
