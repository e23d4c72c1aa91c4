import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); deselect with -m 'not gpu'")


@pytest.fixture(scope="session", autouse=True)
def _built_libraries():
    """Build the CUDA library and the C oracle if they are missing (both compile
    without a GPU)."""
    from grouped_gemm_b200.csrc import build as build_lib
    from oracle import build as build_oracle
    build_lib.build()
    build_oracle.build()
