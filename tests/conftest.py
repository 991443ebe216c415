import pathlib
import sys

import numpy as np
import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = pathlib.Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


def load_golden(name):
    """Golden file -> {case: {field: ndarray}}."""
    flat = np.load(GOLDEN / f"{name}.npz")
    cases = {}
    for key in flat.files:
        case, field = key.split("/", 1)
        cases.setdefault(case, {})[field] = flat[key]
    return cases


@pytest.fixture(scope="session")
def golden():
    return load_golden
