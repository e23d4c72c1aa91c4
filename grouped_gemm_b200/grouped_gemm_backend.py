"""Stand-in for the compiled module ``grouped_gemm_backend`` of the reference.

The reference binds ``gmm(a, b, c, batch_sizes, trans_a, trans_b)`` with
pybind11 (csrc/ops.cu:7-9) onto ``grouped_gemm::GroupedGemm``
(csrc/grouped_gemm.cu:470-564).  This module has the same one function with the
same argument order, performs the same argument checks (raising RuntimeError as
TORCH_CHECK does) and then hands raw pointers to the C ABI ``b200gmm_run``.
"""
import torch

from grouped_gemm_b200 import _capi

_status_words = {}


def device_status(device):
    """The per-device status word the kernels OR their B200GMM_STATUS_* bits
    into.  Reading it (``int(device_status(dev))``) synchronises; 0 = clean."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    word = _status_words.get(device)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[device] = word
    return word


def _check(cond, msg):
    if not cond:
        raise RuntimeError("grouped_gemm_backend.gmm: " + msg)


def gmm(a, b, c, batch_sizes, trans_a, trans_b):
    """Grouped GEMM into caller-provided ``c``; returns None like the reference."""
    # Checks in the order of csrc/grouped_gemm.cu:476-540.
    _check(not (trans_a and trans_b), "only one of trans_a / trans_b may be set")
    _check(batch_sizes.is_cuda or batch_sizes.device.type == "cpu",
           "batch_sizes must be a CPU or CUDA tensor")
    _check(batch_sizes.ndim == 1, "batch_sizes must be 1-D")
    _check(batch_sizes.dtype == torch.int64, "batch_sizes must be int64")
    _check(a.is_cuda, "a must be a CUDA tensor")
    _check(a.ndim == 2, "a must be 2-D")
    _check(a.dtype == torch.bfloat16, "a must be bfloat16")
    _check(b.is_cuda and c.is_cuda, "b and c must be CUDA tensors")
    _check(b.dtype == torch.bfloat16 and c.dtype == torch.bfloat16, "b and c must be bfloat16")
    z = batch_sizes.shape[0]
    if trans_a:
        _check(b.ndim == 2, "b must be 2-D when trans_a is set")
        _check(c.ndim == 3, "c must be 3-D when trans_a is set")
        _check(b.shape[0] == a.shape[0], "a and b must have the same number of rows")
        _check(c.shape[0] == z and c.shape[1] == a.shape[1] and c.shape[2] == b.shape[1],
               "c must be [num_experts, a.shape[1], b.shape[1]]")
        n = b.shape[1]
    else:
        _check(b.ndim == 3, "b must be 3-D")
        _check(c.ndim == 2, "c must be 2-D")
        hidden_in = b.shape[2] if trans_b else b.shape[1]
        n = b.shape[1] if trans_b else b.shape[2]
        _check(hidden_in == a.shape[1], "contraction dimensions of a and b differ")
        _check(z == b.shape[0], "need one batch size per expert")
        # The reference leaves c's 2-D shape unchecked; a short c would be
        # written out of bounds, so it is checked here.
        _check(c.shape[0] == a.shape[0] and c.shape[1] == n, "c must be [a.shape[0], hidden_out]")
    _check(a.is_contiguous() and b.is_contiguous() and c.is_contiguous(),
           "a, b and c must be contiguous")
    _check(a.device == b.device == c.device, "a, b and c must be on one device")
    if batch_sizes.is_cuda:
        _check(batch_sizes.device == a.device, "batch_sizes must be on a's device or on the CPU")
        _check(batch_sizes.is_contiguous(), "batch_sizes must be contiguous")
    else:
        batch_sizes = batch_sizes.contiguous()

    lib = _capi.load()
    with torch.cuda.device(a.device):
        ws_bytes = _capi.workspace_bytes(z)
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device)
        status = device_status(a.device)
        stream = torch.cuda.current_stream(a.device).cuda_stream
        rc = lib.b200gmm_run(
            a.data_ptr(), b.data_ptr(), c.data_ptr(), batch_sizes.data_ptr(),
            1 if batch_sizes.is_cuda else 0, z, a.shape[0], a.shape[1], n,
            1 if trans_a else 0, 1 if trans_b else 0,
            workspace.data_ptr(), ws_bytes, status.data_ptr(), stream)
    _capi.check(rc, "b200gmm_run")
    return None
