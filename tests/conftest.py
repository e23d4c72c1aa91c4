import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); deselect with -m 'not gpu'")


def _build_libraries():
    """Build the CUDA library and the C oracle if they are missing or older than
    their sources (both compile without a GPU).  The build script is loaded by
    path: importing the package would try to load the library being built."""
    import importlib.util
    path = os.path.join(ROOT, "grouped_gemm_b200", "csrc", "build.py")
    spec = importlib.util.spec_from_file_location("b200gmm_build", path)
    build_lib = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(build_lib)
    build_lib.build_all()
    from oracle import build as build_oracle
    build_oracle.build()


# at import of conftest, i.e. before any test module imports the package
_build_libraries()
