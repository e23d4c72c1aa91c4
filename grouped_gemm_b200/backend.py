"""``backend.gmm``: output allocation and the call into the native op.

Same contract as grouped_gemm/backend.py:11-28 of the reference: ``gmm(a, b,
batch_sizes, trans_a=False, trans_b=False, c=None)`` allocates ``c`` when the
caller gives none, writes the grouped product into it and returns it.  The
module-level name ``backend`` is the native binding, as in the reference, so
``ops.backend.gmm`` and ``backend.backend.gmm`` resolve the same way.
"""
import torch

from grouped_gemm_b200 import _capi
from grouped_gemm_b200 import grouped_gemm_backend as backend

# Import fails here, loudly, when the CUDA library has not been built: there is
# no other implementation to fall back to.
_capi.load()


def output_shape(a, b, batch_sizes, trans_a, trans_b):
    """Shape of the result (reference backend.py:17-21)."""
    if trans_a:
        return (batch_sizes.shape[0], a.shape[1], b.shape[1])
    return (a.shape[0], b.shape[1] if trans_b else b.shape[2])


def _allocate_output(a, b, batch_sizes, trans_a, trans_b):
    # Same assertions (AssertionError, not RuntimeError) as reference backend.py:12-15.
    assert not (trans_a and trans_b)
    assert batch_sizes.ndim == 1, "Expected 1d tensor for batch_sizes"
    assert a.ndim == 2, "Expected 2d tensor for 'a'"
    assert b.ndim == (2 if trans_a else 3)
    return torch.empty(output_shape(a, b, batch_sizes, trans_a, trans_b),
                       device=a.device, dtype=a.dtype)


def gmm(a, b, batch_sizes, trans_a=False, trans_b=False, c=None):
    out = c if c is not None else _allocate_output(a, b, batch_sizes, trans_a, trans_b)
    backend.gmm(a, b, out, batch_sizes, trans_a, trans_b)
    return out


def device_status(device="cuda"):
    """Status bits raised by the kernels on ``device`` since the process began
    (0 = none; see B200GMM_STATUS_* in include/b200gmm.h).  Synchronises."""
    return int(backend.device_status(device).item())
