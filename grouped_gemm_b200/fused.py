"""Autograd wrappers for the fused neighbours of ``gmm`` (no counterpart in the
reference, whose callers permute, un-permute and weight in kernels of their own).

``gmm_gather(x, row_index, b, batch_sizes, trans_b)`` equals
``ops.gmm(x[row_index], b, batch_sizes, trans_b)`` in value and in gradients, but
the permuted copy ``x[row_index]`` exists neither in the forward nor in the
backward pass:

* forward: ``backend.gmm_gather`` (rows of ``x`` fetched by the kernel's A-tile load);
* gradient w.r.t. ``x``: the grouped product ``grad @ b^T`` (``trans_b`` flipped, as in
  the reference's ops.py:19-22) whose rows are added into a zeroed ``[R, k]`` tensor at
  ``row_index`` by the kernel's epilogue (``backend.gmm_scatter(..., accumulate=True)``):
  a token that was routed to several experts receives the sum of its rows.  The
  additions round to bf16 in memory in no fixed order, so this gradient can differ in
  the last bit from run to run;
* gradient w.r.t. ``b``: ``x[row_index]^T @ grad`` per expert with the gather again
  inside the kernel (``backend.gmm_gather_wgrad``).  After a ``trans_b`` forward the
  reference's operand order (ops.py:24-28) puts the gathered tensor on the right,
  which the kernel does not gather; that one case permutes ``x`` with
  ``index_select`` first.
"""
import torch

from grouped_gemm_b200 import backend


class GatheredGroupedGemm(torch.autograd.Function):
    """``GatheredGroupedGemm.apply(x, row_index, b, batch_sizes, trans_b)``."""

    @staticmethod
    def forward(ctx, x, row_index, b, batch_sizes, trans_b):
        ctx.trans_b = bool(trans_b)
        ctx.save_for_backward(x, row_index, b, batch_sizes)
        return backend.gmm_gather(x, row_index, b, batch_sizes, trans_b=ctx.trans_b)

    @staticmethod
    def backward(ctx, grad):
        x, row_index, b, batch_sizes = ctx.saved_tensors
        want_x, want_b = ctx.needs_input_grad[0], ctx.needs_input_grad[2]
        if want_x or want_b:
            grad = grad.contiguous()
        xgrad = bgrad = None
        if want_x:
            xgrad = torch.zeros_like(x)
            backend.gmm_scatter(grad, b, batch_sizes, xgrad, row_index.to(torch.int64),
                                trans_b=not ctx.trans_b, accumulate=True)
        if want_b:
            if ctx.trans_b:
                bgrad = backend.gmm(grad, x.index_select(0, row_index), batch_sizes, trans_a=True)
            else:
                bgrad = backend.gmm_gather_wgrad(x, row_index, grad, batch_sizes)
        return xgrad, None, bgrad, None, None


def gmm_gather(x, row_index, b, batch_sizes, trans_b=False):
    """``ops.gmm(x[row_index], b, batch_sizes, trans_b)`` with the gather inside the
    kernels of both passes.  ``x`` bf16 [R, k]; ``row_index`` integer [T] (rows sorted
    by expert, values in [0, R), repeats allowed); ``b`` as for ``ops.gmm``."""
    return GatheredGroupedGemm.apply(x, row_index, b, batch_sizes, trans_b)
