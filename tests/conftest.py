import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def port():
    from oracle import Port
    return Port()


@pytest.fixture(scope="session")
def ref():
    from oracle import Ref, have_ref
    if not have_ref():
        pytest.skip("oracle/_ref/libmme_ref.so is not built here")
    return Ref()


@pytest.fixture(scope="session")
def best_oracle():
    """The compiled reference when available, else the C restatement (Gaudi3 model)."""
    from oracle import Port, Ref, have_ref
    return Ref() if have_ref() else Port()


@pytest.fixture(scope="session")
def calc():
    import intel_gaudi3_software_b200 as pkg
    c = pkg.Calculator(device=0)
    yield c
    c.close()


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "golden_small.npz")
    return np.load(path)
