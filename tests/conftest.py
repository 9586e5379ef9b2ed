import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.pyoracle import Oracle, build
    build(reference=False)
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference engine's own CPU code; skipped where oracle/_ref has not been built."""
    from oracle.pyoracle import Reference
    if not Reference.available():
        pytest.skip("oracle/_ref/libguffin_ref.so not built on this machine")
    return Reference()


@pytest.fixture(scope="session")
def gf():
    """The CUDA library through its C ABI; fails (never skips) when it is missing on a GPU box."""
    from guffin_b200 import lib
    lib.load()
    assert lib.device_count() > 0, "no CUDA device visible"
    return lib
