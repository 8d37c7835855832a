import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def cs1():
    """The product library; built in-tree when missing. No fallback of any kind."""
    from system1_omni_b200 import build, lib
    if not os.path.exists(lib.LIB_PATH):
        build.build()
    return lib.load()


@pytest.fixture(scope="session")
def stream(cs1):
    from system1_omni_b200 import lib
    lib.set_device(0)
    return lib.Stream()


@pytest.fixture
def plan_override(cs1):
    """Forces the tcgen05 GEMM planners (tile width, K shares, contiguous runs, single-block row
    limit) for one test and puts the automatic choice back afterwards."""
    def force(bn=0, splits=0, runs=2, small_rows=0):
        assert cs1.s1_gemm_plan_override(bn, splits, runs, small_rows) == 0
    yield force
    cs1.s1_gemm_plan_override(0, 0, 2, 0)
