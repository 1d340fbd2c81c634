import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA sm_100 device")


@pytest.fixture(scope="session")
def pkg():
    entry._load_build_module().build()
    return entry.load_package()


@pytest.fixture(scope="session")
def oracle():
    from oracle import pyoracle
    return pyoracle.oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own CPU path, or None where it was never built."""
    from oracle import pyoracle
    return pyoracle.reference()


@pytest.fixture(scope="session")
def dev(pkg):
    d = pkg.Device()
    yield d
    d.release()
