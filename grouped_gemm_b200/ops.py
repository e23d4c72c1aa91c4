"""``ops.gmm`` and the ``GroupedGemm`` autograd function.

Same contract as grouped_gemm/ops.py:5-33 of the reference:

* forward: ``c[rows_i] = a[rows_i] @ (b[i].T if trans_b else b[i])`` in one launch;
* backward w.r.t. ``a`` (dgrad): the same grouped product against the other
  orientation of ``b`` (``trans_b`` flipped), giving ``[tokens, hidden_in]``;
* backward w.r.t. ``b`` (wgrad): per expert ``lhs[rows_i].T @ rhs[rows_i]`` with
  ``trans_a=True``; the operands are ordered so that the result has ``b``'s own
  layout (``[z, k, n]`` after a plain forward, ``[z, n, k]`` after ``trans_b``).

Each gradient is computed only when autograd asks for it.
"""
import torch

from grouped_gemm_b200 import backend


def _dgrad(grad, b, batch_sizes, fwd_trans_b):
    """Gradient of the forward output w.r.t. ``a`` (reference ops.py:19-22)."""
    return backend.gmm(grad, b, batch_sizes, trans_a=False, trans_b=not fwd_trans_b)


def _wgrad(a, grad, batch_sizes, fwd_trans_b):
    """Gradient w.r.t. ``b``, in ``b``'s layout (reference ops.py:24-28)."""
    if fwd_trans_b:
        return backend.gmm(grad, a, batch_sizes, trans_a=True, trans_b=False)
    return backend.gmm(a, grad, batch_sizes, trans_a=True, trans_b=False)


class GroupedGemm(torch.autograd.Function):
    """``GroupedGemm.apply(a, b, batch_sizes, trans_b)``."""

    @staticmethod
    def forward(ctx, a, b, batch_sizes, trans_b):
        ctx.trans_b = bool(trans_b)
        ctx.save_for_backward(a, b, batch_sizes)
        return backend.gmm(a, b, batch_sizes, trans_a=False, trans_b=ctx.trans_b)

    @staticmethod
    def backward(ctx, grad):
        a, b, batch_sizes = ctx.saved_tensors
        want_a, want_b = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if want_a or want_b:
            grad = grad.contiguous()
        agrad = _dgrad(grad, b, batch_sizes, ctx.trans_b) if want_a else None
        bgrad = _wgrad(a, grad, batch_sizes, ctx.trans_b) if want_b else None
        return agrad, bgrad, None, None


def gmm(a, b, batch_sizes, trans_b=False):
    """Drop-in for ``grouped_gemm.ops.gmm`` (reference ops.py:32-33)."""
    return GroupedGemm.apply(a, b, batch_sizes, trans_b)
