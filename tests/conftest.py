import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def rx():
    """The host package bound to librx_b200.so (built on demand)."""
    if not os.path.exists(os.path.join(entry.PKG_DIR, "librx_b200.so")):
        entry.build()
    return entry.load_package()


@pytest.fixture(scope="session")
def ref():
    return entry.load_oracle()[0]


@pytest.fixture(scope="session")
def cpu():
    return entry.load_oracle()[1]


@pytest.fixture(scope="session")
def client(rx):
    """One client on cuda:0 shared by the GPU tests."""
    c = rx.Client(allowed_devices=[0])
    yield c
    c.close()
