"""``grouped_gemm.backend`` (reference grouped_gemm/backend.py): the module-level
name ``backend`` is the compiled module ``grouped_gemm_backend`` exactly as in the
reference (backend.py:8), ``gmm`` and ``_allocate_output`` are the B200 ones."""
# torch first so that libc10 is loaded before the extension (reference backend.py:1-3)
import torch  # noqa: F401

import grouped_gemm_backend as backend  # noqa: F401

from grouped_gemm_b200.backend import (  # noqa: F401
    _allocate_output,
    device_status,
    gmm,
    gmm_gather,
    gmm_gather_wgrad,
    gmm_scatter,
    gmm_swiglu,
    output_shape,
)
