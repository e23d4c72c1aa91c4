"""B200-native grouped GEMM with the Python API of tgale96/grouped_gemm.

``import grouped_gemm_b200 as grouped_gemm`` gives ``grouped_gemm.ops.gmm`` and
``grouped_gemm.backend.gmm`` (grouped_gemm/__init__.py:1-2 in the reference).
"""
from grouped_gemm_b200 import backend, ops  # noqa: F401

__all__ = ["backend", "ops"]
