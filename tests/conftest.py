import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU and the built libgt_b200.so")


@pytest.fixture(scope="session")
def gt():
    """The loaded library plus its context; fails (does not skip) when either is missing."""
    from gradtuity_b200 import _lib

    _lib.load_library()
    _lib.context()
    return _lib
