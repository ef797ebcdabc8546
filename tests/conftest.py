import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    # Keep the allocation-free entry point's test last, whatever the file order.
    items.sort(key=lambda item: 1 if "test_zz_" in item.nodeid else 0)


@pytest.fixture(scope="session")
def golden():
    def load(name: str):
        return np.load(GOLDEN / f"{name}.npz")
    return load


@pytest.fixture(scope="session")
def native():
    from rns_llm_b200 import _native
    from rns_llm_b200.csrc import build
    build.build()
    return _native


@pytest.fixture(scope="session")
def c_oracle():
    from oracle import c_oracle as mod
    mod.build()
    return mod
