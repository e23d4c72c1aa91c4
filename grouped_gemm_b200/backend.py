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


def _host_or_device_sizes(batch_sizes):
    """batch_sizes as the C ABI wants it: on the device as it is; on the host
    contiguous and pageable (the library's asynchronous copy reads a pinned array
    only when the stream gets there, by which time the caller may have changed it)."""
    if batch_sizes.is_cuda:
        return batch_sizes
    bs = batch_sizes.contiguous()
    return bs.clone() if bs.is_pinned() else bs


def gmm_scatter(a, b, batch_sizes, out, row_index, trans_b=False, row_weight=None, accumulate=False):
    """``gmm`` with the un-sort fused into the kernel: row ``i`` of the grouped
    result is written to ``out[row_index[i]]`` instead of ``c[i]`` (no
    counterpart in the reference, whose callers un-permute ``c`` themselves).

    ``a`` [T, k] holds the rows sorted by expert as for ``gmm``; ``out`` is a
    contiguous bf16 [R, n] tensor on the same device, ``row_index`` int64 [T] with
    values in [0, R).  Rows of ``out`` that no index names are left alone; if two
    indices coincide the later write wins in no defined order.  An index outside
    [0, R) is never written through: the row is dropped and status bit
    STATUS_BAD_ROW_DEST is raised.  Returns ``out``.

    ``row_weight`` (float32 [T], optional) multiplies row ``i`` in fp32 before the
    rounding to bf16; ``accumulate=True`` adds the rows to ``out`` instead of
    overwriting it, so that with top-k routing (k rows per token, all with the
    same index) one call on a zeroed ``out`` leaves the weighted sum.  The order
    of the additions to one row is not defined (last-bit differences between
    runs)."""
    assert a.ndim == 2 and b.ndim == 3 and batch_sizes.ndim == 1 and out.ndim == 2 and row_index.ndim == 1
    n = b.shape[1] if trans_b else b.shape[2]
    k = b.shape[2] if trans_b else b.shape[1]
    if not (a.is_cuda and b.is_cuda and out.is_cuda and row_index.is_cuda):
        raise RuntimeError("gmm_scatter: a, b, out and row_index must be CUDA tensors")
    if not (b.device == out.device == row_index.device == a.device) or (batch_sizes.is_cuda and batch_sizes.device != a.device):
        raise RuntimeError("gmm_scatter: a, b, out, row_index (and a CUDA batch_sizes) must be on one device")
    if not (a.dtype == b.dtype == out.dtype == torch.bfloat16) or row_index.dtype != torch.int64:
        raise RuntimeError("gmm_scatter: a, b, out must be bfloat16 and row_index int64")
    if a.shape[1] != k or out.shape[1] != n or row_index.shape[0] != a.shape[0] or batch_sizes.shape[0] != b.shape[0]:
        raise RuntimeError("gmm_scatter: shapes of a, b, out, row_index and batch_sizes do not fit together")
    if not (a.is_contiguous() and b.is_contiguous() and out.is_contiguous()):
        raise RuntimeError("gmm_scatter: a, b and out must be contiguous")
    if batch_sizes.dtype != torch.int64:
        raise RuntimeError("gmm_scatter: batch_sizes must be int64")
    if row_weight is not None and not (row_weight.is_cuda and row_weight.dtype == torch.float32
                                       and row_weight.shape == (a.shape[0],) and row_weight.is_contiguous()
                                       and row_weight.device == a.device):
        raise RuntimeError("gmm_scatter: row_weight must be a contiguous float32 CUDA tensor [T] on a's device")
    lib = _capi.load()
    z = batch_sizes.shape[0]
    with torch.cuda.device(a.device):
        dest = row_index * (n * 2) + out.data_ptr()          # byte address of every destination row
        window = (out.data_ptr(), out.numel() * 2)           # the kernel refuses addresses outside ``out``
        ws_bytes = _capi.workspace_bytes(z)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device)
        bs = _host_or_device_sizes(batch_sizes)
        status = backend.device_status(a.device).data_ptr()
        stream = torch.cuda.current_stream(a.device).cuda_stream
        if row_weight is None and not accumulate:
            rc = lib.b200gmm_run_scatter(
                a.data_ptr(), b.data_ptr(), dest.data_ptr(), *window, bs.data_ptr(), 1 if bs.is_cuda else 0, z,
                a.shape[0], a.shape[1], n, 1 if trans_b else 0, ws.data_ptr(), ws_bytes, status, stream)
        else:
            rc = lib.b200gmm_run_combine(
                a.data_ptr(), b.data_ptr(), dest.data_ptr(), *window,
                None if row_weight is None else row_weight.data_ptr(), 1 if accumulate else 0,
                bs.data_ptr(), 1 if bs.is_cuda else 0, z,
                a.shape[0], a.shape[1], n, 1 if trans_b else 0, ws.data_ptr(), ws_bytes, status, stream)
    _capi.check(rc, "b200gmm_run_scatter")
    return out


def gmm_gather(x, row_index, b, batch_sizes, trans_b=False, c=None, out=None, out_index=None):
    """``gmm(x[row_index], b, batch_sizes, trans_b)`` without materialising
    ``x[row_index]``: the kernel gathers the rows of ``x`` while it loads its
    operand tiles (no counterpart in the reference, whose callers permute the
    activations into a new tensor first).  It saves the memory of the permuted
    copy and its launch; in time it is on a par with ``x.index_select(0, idx)``
    followed by ``gmm`` (about 10 % behind ``gmm`` alone on large shapes).  A
    row index outside ``x`` is read as a row of zeros and raises status bit 8.

    ``x`` bf16 [R, k]; ``row_index`` integer [T] with values in [0, R), listing for
    every grouped row (sorted by expert, as ``gmm`` expects them) the row of ``x``
    it comes from.  Result rows go to ``c`` [T, n] (allocated if omitted), or, when
    ``out`` [R2, n] and ``out_index`` int64 [T] are given, row i goes to
    ``out[out_index[i]]`` (gather and un-sort both fused) and ``out`` is returned."""
    assert x.ndim == 2 and b.ndim == 3 and batch_sizes.ndim == 1 and row_index.ndim == 1
    n = b.shape[1] if trans_b else b.shape[2]
    k = b.shape[2] if trans_b else b.shape[1]
    if not (x.is_cuda and b.is_cuda and row_index.is_cuda):
        raise RuntimeError("gmm_gather: x, b and row_index must be CUDA tensors")
    if not (b.device == row_index.device == x.device) or (batch_sizes.is_cuda and batch_sizes.device != x.device):
        raise RuntimeError("gmm_gather: x, b, row_index (and a CUDA batch_sizes) must be on one device")
    if not (x.dtype == b.dtype == torch.bfloat16) or batch_sizes.dtype != torch.int64:
        raise RuntimeError("gmm_gather: x and b must be bfloat16, batch_sizes int64")
    if x.shape[1] != k or batch_sizes.shape[0] != b.shape[0] or not (x.is_contiguous() and b.is_contiguous()):
        raise RuntimeError("gmm_gather: shapes of x, b and batch_sizes do not fit together, or not contiguous")
    tokens = row_index.shape[0]
    idx32 = row_index.to(torch.int32).contiguous()
    lib = _capi.load()
    z = batch_sizes.shape[0]
    with torch.cuda.device(x.device):
        dest_ptr = None
        window = (None, 0)
        result = None
        if out is not None:
            if out_index is None or out.dtype != torch.bfloat16 or not out.is_contiguous() or out.shape[1] != n \
                    or out_index.shape[0] != tokens or out.device != x.device or out_index.device != x.device:
                raise RuntimeError("gmm_gather: out must be contiguous bf16 [R2, n] with out_index int64 [T], on x's device")
            dest = out_index.to(torch.int64) * (n * 2) + out.data_ptr()
            dest_ptr, result = dest.data_ptr(), out
            window = (out.data_ptr(), out.numel() * 2)
            c_ptr = None
        else:
            if c is None:
                c = torch.empty(tokens, n, device=x.device, dtype=x.dtype)
            elif c.shape != (tokens, n) or c.dtype != torch.bfloat16 or not c.is_contiguous() or c.device != x.device:
                raise RuntimeError("gmm_gather: c must be contiguous bf16 [len(row_index), n] on x's device")
            c_ptr, result = c.data_ptr(), c
        ws_bytes = _capi.workspace_bytes(z)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
        bs = _host_or_device_sizes(batch_sizes)
        rc = lib.b200gmm_run_gather(
            x.data_ptr(), x.shape[0], idx32.data_ptr(), b.data_ptr(), c_ptr, dest_ptr, *window, bs.data_ptr(),
            1 if bs.is_cuda else 0, z, tokens, k, n, 1 if trans_b else 0, ws.data_ptr(), ws_bytes,
            backend.device_status(x.device).data_ptr(), torch.cuda.current_stream(x.device).cuda_stream)
    _capi.check(rc, "b200gmm_run_gather")
    return result


def gmm_gather_wgrad(x, row_index, grad, batch_sizes, c=None):
    """``gmm(x[row_index], grad, batch_sizes, trans_a=True)`` without materialising
    ``x[row_index]``: the weight gradient of ``gmm_gather`` (no counterpart in the
    reference).  ``x`` bf16 [R, k]; ``row_index`` integer [T]; ``grad`` bf16 [T, n]
    grouped by expert; returns bf16 [z, k, n] (zeros for empty experts).  Measured
    at 1.7x the time of ``gmm(x.index_select(0, idx), grad, trans_a=True)`` on large
    shapes: it saves the copy, not time."""
    assert x.ndim == 2 and grad.ndim == 2 and batch_sizes.ndim == 1 and row_index.ndim == 1
    if not (x.is_cuda and grad.is_cuda and row_index.is_cuda):
        raise RuntimeError("gmm_gather_wgrad: x, grad and row_index must be CUDA tensors")
    if not (grad.device == row_index.device == x.device) or (batch_sizes.is_cuda and batch_sizes.device != x.device):
        raise RuntimeError("gmm_gather_wgrad: x, grad, row_index (and a CUDA batch_sizes) must be on one device")
    if not (x.dtype == grad.dtype == torch.bfloat16) or batch_sizes.dtype != torch.int64:
        raise RuntimeError("gmm_gather_wgrad: x and grad must be bfloat16, batch_sizes int64")
    tokens, n, k, z = grad.shape[0], grad.shape[1], x.shape[1], batch_sizes.shape[0]
    if row_index.shape[0] != tokens or not (x.is_contiguous() and grad.is_contiguous()):
        raise RuntimeError("gmm_gather_wgrad: shapes of x, row_index and grad do not fit together, or not contiguous")
    if c is None:
        c = torch.empty(z, k, n, device=x.device, dtype=x.dtype)
    elif c.shape != (z, k, n) or c.dtype != torch.bfloat16 or not c.is_contiguous() or c.device != x.device:
        raise RuntimeError("gmm_gather_wgrad: c must be contiguous bf16 [z, k, n] on x's device")
    idx32 = row_index.to(torch.int32).contiguous()
    lib = _capi.load()
    with torch.cuda.device(x.device):
        ws_bytes = _capi.workspace_bytes(z)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
        bs = _host_or_device_sizes(batch_sizes)
        rc = lib.b200gmm_run_gather_wgrad(
            x.data_ptr(), x.shape[0], idx32.data_ptr(), grad.data_ptr(), c.data_ptr(), bs.data_ptr(),
            1 if bs.is_cuda else 0, z, tokens, k, n, ws.data_ptr(), ws_bytes,
            backend.device_status(x.device).data_ptr(), torch.cuda.current_stream(x.device).cuda_stream)
    _capi.check(rc, "b200gmm_run_gather_wgrad")
    return c


def gmm_swiglu(a, b_gate, b_up, batch_sizes, trans_b=False, c=None):
    """``silu(gmm(a, b_gate)) * gmm(a, b_up)`` in one kernel: the gated first
    half of a SwiGLU expert layer (no counterpart in the reference, whose
    callers run ``gmm`` twice and apply the activation in a kernel of their own).
    Both products share one fp32 accumulator tile, the gate is applied to the
    fp32 values and the result is rounded to bf16 once, so neither product is
    ever written to memory.  ``fused.gmm_swiglu`` is the same with autograd.

    ``a`` bf16 [T, k] sorted by expert as for ``gmm``; ``b_gate`` and ``b_up``
    bf16 [z, k, n] (or [z, n, k] with ``trans_b``); returns ``c`` bf16 [T, n]."""
    assert a.ndim == 2 and b_gate.ndim == 3 and b_up.ndim == 3 and batch_sizes.ndim == 1
    n = b_gate.shape[1] if trans_b else b_gate.shape[2]
    k = b_gate.shape[2] if trans_b else b_gate.shape[1]
    if not (a.is_cuda and b_gate.is_cuda and b_up.is_cuda):
        raise RuntimeError("gmm_swiglu: a, b_gate and b_up must be CUDA tensors")
    if not (b_gate.device == b_up.device == a.device) or (batch_sizes.is_cuda and batch_sizes.device != a.device):
        raise RuntimeError("gmm_swiglu: a, b_gate, b_up (and a CUDA batch_sizes) must be on one device")
    if not (a.dtype == b_gate.dtype == b_up.dtype == torch.bfloat16) or batch_sizes.dtype != torch.int64:
        raise RuntimeError("gmm_swiglu: a, b_gate, b_up must be bfloat16, batch_sizes int64")
    if b_gate.shape != b_up.shape or a.shape[1] != k or batch_sizes.shape[0] != b_gate.shape[0]:
        raise RuntimeError("gmm_swiglu: shapes of a, b_gate, b_up and batch_sizes do not fit together")
    if not (a.is_contiguous() and b_gate.is_contiguous() and b_up.is_contiguous()):
        raise RuntimeError("gmm_swiglu: a, b_gate and b_up must be contiguous")
    tokens = a.shape[0]
    if c is None:
        c = torch.empty(tokens, n, device=a.device, dtype=a.dtype)
    elif c.shape != (tokens, n) or c.dtype != torch.bfloat16 or not c.is_contiguous() or c.device != a.device:
        raise RuntimeError("gmm_swiglu: c must be contiguous bf16 [T, n] on a's device")
    lib = _capi.load()
    z = batch_sizes.shape[0]
    with torch.cuda.device(a.device):
        ws_bytes = _capi.workspace_bytes(z)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device)
        bs = _host_or_device_sizes(batch_sizes)
        rc = lib.b200gmm_run_swiglu(
            a.data_ptr(), b_gate.data_ptr(), b_up.data_ptr(), c.data_ptr(), None, None, 0, bs.data_ptr(),
            1 if bs.is_cuda else 0, z, tokens, k, n, 1 if trans_b else 0, ws.data_ptr(), ws_bytes,
            backend.device_status(a.device).data_ptr(), torch.cuda.current_stream(a.device).cuda_stream)
    _capi.check(rc, "b200gmm_run_swiglu")
    return c


def gmm_swiglu_backward(a, b_gate, b_up, grad_out, batch_sizes, trans_b=False):
    """Gradients of ``gmm_swiglu`` with respect to its two products, in one kernel
    (no counterpart in the reference).  The gate and up products are recomputed in
    the accumulator; returns ``(d_gate, d_up)``, bf16 [T, n] each (two halves of one
    [2, T, n] tensor), with ``d_gate = grad_out * up * silu'(gate)`` and
    ``d_up = grad_out * silu(gate)``.  Rows past ``sum(batch_sizes)`` are zeros."""
    assert a.ndim == 2 and b_gate.ndim == 3 and b_up.ndim == 3 and batch_sizes.ndim == 1 and grad_out.ndim == 2
    n = b_gate.shape[1] if trans_b else b_gate.shape[2]
    k = b_gate.shape[2] if trans_b else b_gate.shape[1]
    if not (a.is_cuda and b_gate.device == b_up.device == grad_out.device == a.device) or \
            (batch_sizes.is_cuda and batch_sizes.device != a.device):
        raise RuntimeError("gmm_swiglu_backward: a, b_gate, b_up, grad_out (and a CUDA batch_sizes) must be on one CUDA device")
    if not (a.dtype == b_gate.dtype == b_up.dtype == grad_out.dtype == torch.bfloat16) or batch_sizes.dtype != torch.int64:
        raise RuntimeError("gmm_swiglu_backward: a, b_gate, b_up, grad_out must be bfloat16, batch_sizes int64")
    tokens = a.shape[0]
    if b_gate.shape != b_up.shape or a.shape[1] != k or batch_sizes.shape[0] != b_gate.shape[0] \
            or grad_out.shape != (tokens, n):
        raise RuntimeError("gmm_swiglu_backward: shapes of a, b_gate, b_up, grad_out and batch_sizes do not fit together")
    if not (a.is_contiguous() and b_gate.is_contiguous() and b_up.is_contiguous() and grad_out.is_contiguous()):
        raise RuntimeError("gmm_swiglu_backward: a, b_gate, b_up and grad_out must be contiguous")
    out = torch.zeros(2, tokens, n, device=a.device, dtype=a.dtype)
    lib = _capi.load()
    z = batch_sizes.shape[0]
    with torch.cuda.device(a.device):
        ws_bytes = _capi.workspace_bytes(z)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device)
        bs = _host_or_device_sizes(batch_sizes)
        rc = lib.b200gmm_run_swiglu_backward(
            a.data_ptr(), b_gate.data_ptr(), b_up.data_ptr(), grad_out.data_ptr(), out.data_ptr(), bs.data_ptr(),
            1 if bs.is_cuda else 0, z, tokens, k, n, 1 if trans_b else 0, ws.data_ptr(), ws_bytes,
            backend.device_status(a.device).data_ptr(), torch.cuda.current_stream(a.device).cuda_stream)
    _capi.check(rc, "b200gmm_run_swiglu_backward")
    return out[0], out[1]


def device_status(device="cuda"):
    """Status bits raised by the kernels on ``device`` since the process began
    (0 = none; see B200GMM_STATUS_* in include/b200gmm.h).  Synchronises."""
    return int(backend.device_status(device).item())
