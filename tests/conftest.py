import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "appmult-aware-retraining_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")
GOLDEN_NAMES = ["mult7_med63", "mul8u_17C8", "trunc6"]


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


def pytest_collection_modifyitems(config, items):
    # keep the no-allocation entry point's test last so that a -x run has seen everything else first
    items.sort(key=lambda it: 1 if "test_zz_" in it.nodeid else 0)


@pytest.fixture(scope="session")
def oracle_c():
    from oracle import OracleC
    return OracleC()


@pytest.fixture(scope="session", params=GOLDEN_NAMES)
def golden(request):
    return dict(np.load(os.path.join(GOLDEN_DIR, f"golden_{request.param}.npz")))


def load_golden(name):
    return dict(np.load(os.path.join(GOLDEN_DIR, f"golden_{name}.npz")))
