import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")
    # the CUDA library is a build product (not in the source tree's history): compile it once if it is not there yet
    # (aiter_b200/build.py is loaded by path: importing the package itself needs the library)
    import importlib.util

    spec = importlib.util.spec_from_file_location("_aiter_b200_build", os.path.join(ROOT, "aiter_b200", "build.py"))
    build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(build)
    if not os.path.exists(build.LIB_PATH):
        build.build_library(force=True)


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return np.load(os.path.join(ROOT, "tests", "golden", "mx_golden.npz"))
