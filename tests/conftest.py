import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


def pytest_sessionstart(session):
    # The C-ABI library is built in-tree (nvcc cross-compiles without a GPU); build it if it is not there yet.
    import importlib.util
    spec = importlib.util.spec_from_file_location("_dg_build", os.path.join(ROOT, "deepgemm_amd_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build_library()


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_python.npz"))
