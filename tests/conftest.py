import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "general-nvgpu-testing_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def built_library():
    """Path of libbeam_b200.so; builds it (nvcc cross-compiles without a GPU) when missing or stale."""
    import build as beam_build  # general-nvgpu-testing_b200/build.py
    return beam_build.build()


@pytest.fixture(scope="session")
def oracle_mod():
    from oracle import build_oracle
    build_oracle.build()
    import oracle
    return oracle
