import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    # Keep files in name order so the last-named file is collected last.
    items.sort(key=lambda it: it.fspath.basename)


@pytest.fixture(scope="session")
def orc():
    import oracle

    oracle.lib()
    return oracle
