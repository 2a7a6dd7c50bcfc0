import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    # keep files whose name starts with test_zz at the very end of the run
    items.sort(key=lambda it: (os.path.basename(str(it.fspath)).startswith("test_zz"),))


@pytest.fixture(scope="session")
def wl():
    from golden_cases import load_workloads
    return load_workloads()
