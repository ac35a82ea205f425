import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def orc():
    import oracle
    return oracle.oracle()


@pytest.fixture(scope="session")
def ref():
    """The reference's own CPU sources compiled in place, or a skip where they cannot be had."""
    import oracle
    r = oracle.reference()
    if r is None:
        pytest.skip("no reference checkout and no prebuilt oracle/_ref library")
    return r


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    d = os.path.join(ROOT, "tests", "golden")
    return {k: np.load(os.path.join(d, k + "_golden.npz"), allow_pickle=False) for k in ("dequant", "route", "layer")}
