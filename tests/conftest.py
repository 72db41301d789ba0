import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs on the B200 box)")


@pytest.fixture(scope="session")
def port():
    from oracle import bindings
    return bindings.port()


@pytest.fixture(scope="session")
def ref():
    """The reference's own kernels compiled in place; skips where never built."""
    from oracle import bindings
    r = bindings.ref()
    if r is None:
        pytest.skip("oracle/_ref/libemel_ref.so not built (needs the reference checkout)")
    return r


@pytest.fixture(scope="session")
def checker(port):
    """Strongest available checker: the reference build if present, else the port."""
    from oracle import bindings
    return bindings.ref() or port
