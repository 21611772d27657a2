"""Shared fixtures.  Tests marked ``gpu`` need a B200 and call the CUDA library through its C ABI;
everything else runs on CPU."""
import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def golden():
    with open(os.path.join(ROOT, "tests", "golden", "known_answers.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def orc():
    import oracle
    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def be():
    """The device backend; fails loudly (no skip, no fallback) when the CUDA library cannot run."""
    from minitensor_b200.backend import get_backend
    return get_backend(0)


@pytest.fixture()
def rng():
    return np.random.default_rng(7)


def fval(v):
    """JSON stand-ins for non-finite floats."""
    if v == "nan":
        return float("nan")
    if v == "inf":
        return float("inf")
    if v == "-inf":
        return float("-inf")
    return float(v)
