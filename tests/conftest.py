import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def orc():
    from tests import oracle_lib
    return oracle_lib.load()


@pytest.fixture(scope="session")
def ref():
    """The reference project's own CUDA kernels (prebuilt oracle/_ref/libet_ref.so), or skip."""
    from tests import oracle_lib
    r = oracle_lib.load_ref()
    if r is None:
        pytest.skip("oracle/_ref/libet_ref.so not built")
    return r
