"""CPU restatement of the reference's grouped GEMM.  TEST INFRASTRUCTURE ONLY:
the product path never imports this file and has no CPU fallback.

Parity pin: the reference holds no golden vectors on disk; its tests compare
against a per-expert matmul loop (grouped_gemm/ops_test.py:44-53) on inputs from
its own generator (ops_test.py:39-41).  ``tests/golden/make_golden.py`` executes
exactly those two reference functions (source text read from the reference
checkout, run on CPU) and commits their outputs; ``tests/test_oracle.py`` checks
this restatement against them, and against the reference's one known-answer
case (ops_test.py:143-158).

Each function cites the reference lines it follows (paths inside
tgale96/grouped_gemm).
"""
import numpy as np
import torch

FILL_FIELDS = ("m", "n", "k", "lda", "ldb", "ldc", "a_offset", "b_offset", "c_offset")


def exclusive_cumsum(batch_sizes):
    """Exclusive prefix sum in int64 (csrc/fill_arguments.cuh:59-62; the host
    path keeps running element counts instead, csrc/grouped_gemm.cu:172-175)."""
    bs = np.asarray(batch_sizes, dtype=np.int64)
    out = np.zeros_like(bs)
    if bs.size > 1:
        np.cumsum(bs[:-1], out=out[1:])
    return out


def fill_offsets(batch_sizes, dim_a1, n, trans_a, trans_b):
    """Per-expert GEMM problems as the reference's argument fill builds them
    (csrc/fill_arguments.cuh:66-78; host twin csrc/grouped_gemm.cu:160-175),
    evaluated in int64.  Returns int64 array [z, 9] in FILL_FIELDS order.

    Leading dimensions follow ``Layout::packed(...).stride(0)``
    (fill_arguments.cuh:69-71): columns for a row-major operand, rows for a
    column-major one.  The descending-k sort of the wgrad problems
    (fill_arguments.cuh:80-86) only reorders work and is not part of the result.
    """
    assert not (trans_a and trans_b)
    bs = np.asarray(batch_sizes, dtype=np.int64)
    z = bs.shape[0]
    start = exclusive_cumsum(bs)
    e = np.arange(z, dtype=np.int64)
    out = np.zeros((z, 9), dtype=np.int64)
    if trans_a:
        m, k = np.int64(dim_a1), bs          # coord template (hidden_in, hidden_out, dynamic)
        out[:, 0], out[:, 1], out[:, 2] = m, n, k
        out[:, 3] = m                         # a read as column-major m x k
        out[:, 4] = n
        out[:, 5] = n
        out[:, 6] = m * start                 # dims.m() * cumsum
        out[:, 7] = start * n                 # cumsum * dims.n()
        out[:, 8] = e * m * n                 # expert_idx * dims.m() * dims.n()
    else:
        m, k = bs, np.int64(dim_a1)
        out[:, 0], out[:, 1], out[:, 2] = m, n, k
        out[:, 3] = k
        out[:, 4] = k if trans_b else n       # b[i] column-major k x n when trans_b
        out[:, 5] = n
        out[:, 6] = start * k
        out[:, 7] = e * k * n
        out[:, 8] = start * n
    return out


def gmm(a, b, batch_sizes, trans_a=False, trans_b=False, c=None, accumulate_dtype=torch.float32):
    """Per-expert matmul loop on CPU tensors.

    Not transposed / trans_b: grouped_gemm/ops_test.py:44-53
    (``a[start:start+size] @ (b[i].t() if trans_b else b[i])``, concatenated).
    trans_a: ``c[i] = a[rows_i].T @ b[rows_i]`` as CublasGroupedGemmVariableK does
    (csrc/grouped_gemm.cu:418-435), zeros for empty experts
    (csrc/fill_arguments.cuh:100-119).  Rows past sum(batch_sizes) keep whatever
    ``c`` held (the reference never writes them).  Operands are upcast to
    ``accumulate_dtype`` (fp32 accumulate), the result is rounded once to a's dtype.
    """
    assert not (trans_a and trans_b)
    sizes = [int(s) for s in torch.as_tensor(batch_sizes).cpu().tolist()]
    a_acc, b_acc = a.to(accumulate_dtype), b.to(accumulate_dtype)
    start = 0
    if trans_a:
        out = c if c is not None else torch.empty(len(sizes), a.shape[1], b.shape[1], dtype=a.dtype)
        for i, size in enumerate(sizes):
            out[i] = (a_acc[start:start + size].t() @ b_acc[start:start + size]).to(a.dtype)
            start += size
        return out
    n = b.shape[1] if trans_b else b.shape[2]
    out = c if c is not None else torch.zeros(a.shape[0], n, dtype=a.dtype)
    for i, size in enumerate(sizes):
        rhs = b_acc[i].t() if trans_b else b_acc[i]
        out[start:start + size] = (a_acc[start:start + size] @ rhs).to(a.dtype)
        start += size
    return out


def gmm_swiglu(a, b_gate, b_up, batch_sizes, trans_b=False):
    """``silu(gmm(a, b_gate)) * gmm(a, b_up)`` with both products and the gate in
    fp32 and one rounding to a's dtype at the end.  The reference has no such
    operator; this composes its gmm semantics (the loop above) with
    ``torch.nn.functional.silu`` to check the fused kernel."""
    gate = gmm(a.float(), b_gate.float(), batch_sizes, trans_b=trans_b)
    up = gmm(a.float(), b_up.float(), batch_sizes, trans_b=trans_b)
    return (torch.nn.functional.silu(gate) * up).to(a.dtype)


def gmm_backward(a, b, batch_sizes, grad, trans_b=False):
    """Gradients of ``gmm(a, b, batch_sizes, trans_b)`` for upstream ``grad``,
    with the operand choice of GroupedGemm.backward (grouped_gemm/ops.py:14-29):
    dgrad = gmm(grad, b, trans_b flipped); wgrad = gmm(lhs, rhs, trans_a=True)
    with (lhs, rhs) = (grad, a) if trans_b else (a, grad)."""
    agrad = gmm(grad, b, batch_sizes, trans_b=not trans_b)
    lhs, rhs = (grad, a) if trans_b else (a, grad)
    bgrad = gmm(lhs, rhs, batch_sizes, trans_a=True)
    return agrad, bgrad


def reference_allclose_pct(x, y):
    """The reference test's closeness statistic (grouped_gemm/ops_test.py:10-17):
    percentage of elements failing ``isclose(rtol=1e-5)``; it accepts <= 2 %."""
    mask = torch.isclose(x.float(), y.float(), rtol=1e-5)
    return float((mask.numel() - mask.sum()) / max(mask.numel(), 1) * 100)


def torch_loop_bf16(a, b, batch_sizes, trans_b=False):
    """The reference test's loop verbatim in behaviour (ops_test.py:44-53): bf16
    operands straight into ``@``.  This is the CPU baseline that bench.py times."""
    sizes = [int(s) for s in torch.as_tensor(batch_sizes).cpu().tolist()]
    out, start = [], 0
    for i, size in enumerate(sizes):
        rhs = b[i].t() if trans_b else b[i]
        out.append(a[start:start + size] @ rhs)
        start += size
    return torch.cat(out)


def torch_loop_tn_bf16(a, b, batch_sizes):
    """wgrad twin of torch_loop_bf16: ``a[rows_i].T @ b[rows_i]`` per expert
    (csrc/grouped_gemm.cu:418-435)."""
    sizes = [int(s) for s in torch.as_tensor(batch_sizes).cpu().tolist()]
    out, start = [], 0
    for size in sizes:
        out.append(a[start:start + size].t() @ b[start:start + size])
        start += size
    return torch.stack(out)
