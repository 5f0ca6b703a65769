import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
TESTS = os.path.dirname(os.path.abspath(__file__))
if TESTS not in sys.path:
    sys.path.insert(0, TESTS)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200, sm_100a)")


@pytest.fixture(scope="session", autouse=True)
def native_build():
    """Native libraries are built in-tree once per session (a no-op when up to date)."""
    from bsipytorch_b200 import build
    build.build()
    from oracle import build as obuild
    obuild.build_oracle()
    yield
