"""Autograd wrappers for the fused neighbours of ``gmm`` (no counterpart in the
reference, whose callers permute, un-permute, weight and gate in kernels of their
own): ``gmm_gather`` below, ``gmm_swiglu`` at the end of the file.

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


class GatedGroupedGemm(torch.autograd.Function):
    """``GatedGroupedGemm.apply(a, b_gate, b_up, batch_sizes, trans_b)``:
    ``silu(a @ b_gate) * (a @ b_up)`` per expert, forward and backward, without the
    two products ever being stored.

    * forward: ``backend.gmm_swiglu`` (one kernel, activation in the epilogue);
    * backward: ``backend.gmm_swiglu_backward`` recomputes both products in one
      kernel and turns the output gradient into the gradients of the two products;
      from there on it is the reference's backward (ops.py:14-29) twice: the input
      gradient is the sum of two grouped products against the other orientation of
      the weights, each weight gradient one ``trans_a`` product.
    """

    @staticmethod
    def forward(ctx, a, b_gate, b_up, batch_sizes, trans_b):
        ctx.trans_b = bool(trans_b)
        ctx.save_for_backward(a, b_gate, b_up, batch_sizes)
        return backend.gmm_swiglu(a, b_gate, b_up, batch_sizes, trans_b=ctx.trans_b)

    @staticmethod
    def backward(ctx, grad):
        a, b_gate, b_up, batch_sizes = ctx.saved_tensors
        want_a, want_g, want_u = ctx.needs_input_grad[0], ctx.needs_input_grad[1], ctx.needs_input_grad[2]
        if not (want_a or want_g or want_u):
            return None, None, None, None, None
        d_gate, d_up = backend.gmm_swiglu_backward(a, b_gate, b_up, grad.contiguous(), batch_sizes, trans_b=ctx.trans_b)
        agrad = ggrad = ugrad = None
        if want_a:
            agrad = backend.gmm(d_gate, b_gate, batch_sizes, trans_b=not ctx.trans_b)
            agrad += backend.gmm(d_up, b_up, batch_sizes, trans_b=not ctx.trans_b)
        def wgrad(d):  # in the weights' own layout (reference ops.py:24-28)
            lhs, rhs = (d, a) if ctx.trans_b else (a, d)
            return backend.gmm(lhs, rhs, batch_sizes, trans_a=True)
        if want_g:
            ggrad = wgrad(d_gate)
        if want_u:
            ugrad = wgrad(d_up)
        return agrad, ggrad, ugrad, None, None


def gmm_swiglu(a, b_gate, b_up, batch_sizes, trans_b=False):
    """``silu(ops.gmm(a, b_gate)) * ops.gmm(a, b_up)`` with autograd; neither
    product is written to memory in either pass."""
    return GatedGroupedGemm.apply(a, b_gate, b_up, batch_sizes, trans_b)
