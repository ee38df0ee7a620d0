import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def port():
    from oracle import Oracle
    return Oracle("port")


@pytest.fixture(scope="session")
def reference():
    from oracle import Oracle
    try:
        return Oracle("reference")
    except FileNotFoundError:
        pytest.skip("reference CPU backend not built (reference tree absent)")
