"""The compiled module ``grouped_gemm_backend`` of the reference, B200 edition.

The reference binds ``gmm(a, b, c, batch_sizes, trans_a, trans_b)`` with
pybind11 (csrc/ops.cu:7-9) onto ``grouped_gemm::GroupedGemm``
(csrc/grouped_gemm.cu:470-564).  Here the same one function lives in a torch
extension module (csrc/torch_ext/binding.cpp, built in-tree) that repeats the
reference's argument checks as TORCH_CHECKs (RuntimeError in Python), takes the
current CUDA stream and a workspace from torch, and calls the C ABI
``b200gmm_run`` of libb200gmm.so.  This file only loads that module; if it has
not been built the import fails: there is no other implementation.
"""
import importlib.util
import os

import torch  # noqa: F401  (libc10 / libtorch must be loaded first)

from grouped_gemm_b200 import _capi

_HERE = os.path.dirname(os.path.abspath(__file__))
EXT_PATH = os.path.join(_HERE, "csrc", "torch_ext", "build", "b200gmm_torch_binding.so")


def _load_extension():
    _capi.load()  # libb200gmm.so first: the extension links against it
    if not os.path.exists(EXT_PATH):
        raise ImportError(
            f"{EXT_PATH} is missing: build it with `python grouped_gemm_b200/csrc/build.py` "
            "(needs nvcc and a C++ compiler; there is no fallback binding)")
    spec = importlib.util.spec_from_file_location("b200gmm_torch_binding", EXT_PATH)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


_ext = _load_extension()

#: ``gmm(a, b, c, batch_sizes, trans_a, trans_b) -> None`` -- writes into ``c``.
gmm = _ext.gmm


def device_status(device):
    """The per-device status word the kernels OR their B200GMM_STATUS_* bits
    into (int32[1] tensor).  Reading it (``int(device_status(dev))``)
    synchronises; 0 = clean."""
    device = torch.device(device)
    index = device.index if device.index is not None else torch.cuda.current_device()
    return _ext.device_status(index)
