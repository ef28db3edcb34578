import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    import oracle as O
    O.lib()  # builds liboracle.so on first use
    return O


@pytest.fixture(scope="session")
def tc():
    """The product binding; building the library first if it has not been built yet."""
    import tensorcore_b200 as T
    if not os.path.exists(T.LIB_PATH):
        from tensorcore_b200.build import build
        build()
    T.lib()
    return T


@pytest.fixture(scope="session")
def ctx(tc):
    c = tc.Context()
    yield c
    c.close()
