"""``grouped_gemm.ops`` (reference grouped_gemm/ops.py): ``gmm`` and the
``GroupedGemm`` autograd function; ``ops.backend`` is ``grouped_gemm.backend`` as
in the reference (ops.py:1), which its own tests rely on (ops_test.py:154)."""
from grouped_gemm import backend  # noqa: F401

from grouped_gemm_b200.ops import GroupedGemm, gmm  # noqa: F401
