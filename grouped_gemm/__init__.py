"""``grouped_gemm``: the import name of tgale96/grouped_gemm, served by the
B200 implementation in ``grouped_gemm_b200``.

Same two submodules as the reference (grouped_gemm/__init__.py:1-2), so code
written against it (``import grouped_gemm``; ``grouped_gemm.ops.gmm``;
``grouped_gemm.backend.gmm``) runs unchanged.
"""
import grouped_gemm.ops
import grouped_gemm.backend
