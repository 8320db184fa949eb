import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def built_lib():
    """The in-tree CUDA library (compiled here if stale; nvcc needs no GPU)."""
    from inferno_b200 import build
    return build.build()


@pytest.fixture(scope="session")
def oracle_mod():
    from oracle import oracle as orc
    orc.build(ref=False)
    return orc
