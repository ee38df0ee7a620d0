import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_sessionfinish(session, exitstatus):
    """B200CONV_PARITY_REPORT=<file>: the error figures the contraction tests recorded (tests/util.py:record_parity)."""
    path = os.environ.get("B200CONV_PARITY_REPORT")
    if not path:
        return
    import json
    from tests.util import PARITY_REPORT
    with open(path, "w") as f:
        json.dump({k: dict(dot_rel_err=v[0], survey_rel_err=v[1]) for k, v in sorted(PARITY_REPORT.items())}, f, indent=1)


@pytest.fixture(scope="session")
def port_mt():
    """The checker with its batched routines spread over the host's cores (full-size configurations): the reference's
    compiled CPU backend where it is built, else the restatement -- the two are bit-identical."""
    from oracle import Oracle
    n = os.cpu_count() or 1
    try:
        return Oracle("reference", threads=n)
    except FileNotFoundError:
        return Oracle("port", threads=n)


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
