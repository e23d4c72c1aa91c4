"""Loader of the compiled module ``grouped_gemm_backend``, B200 edition.

The reference binds ``gmm(a, b, c, batch_sizes, trans_a, trans_b)`` with
pybind11 (csrc/ops.cu:7-9) onto ``grouped_gemm::GroupedGemm``
(csrc/grouped_gemm.cu:470-564) in a top-level extension module named
``grouped_gemm_backend`` (setup.py:35).  Here a torch extension of the same name
(csrc/torch_ext/binding.cpp, built in-tree beside the packages) repeats the
reference's argument checks as TORCH_CHECKs (RuntimeError in Python), takes the
current CUDA stream and a workspace from torch, and calls the C ABI
``b200gmm_run`` of libb200gmm.so.  This file only finds and loads that module; if
it has not been built the import fails: there is no other implementation.
"""
import importlib
import importlib.util
import os
import sys

import torch  # noqa: F401  (libc10 / libtorch must be loaded first)

from grouped_gemm_b200 import _capi

_HERE = os.path.dirname(os.path.abspath(__file__))
EXT_NAME = "grouped_gemm_backend"
EXT_PATH = os.path.join(os.path.dirname(_HERE), EXT_NAME + ".so")


def _load_extension():
    _capi.load()  # libb200gmm.so first: the extension links against it
    if EXT_NAME in sys.modules:
        return sys.modules[EXT_NAME]
    if os.path.exists(EXT_PATH):
        # beside this package, whatever sys.path says
        spec = importlib.util.spec_from_file_location(EXT_NAME, EXT_PATH)
        module = importlib.util.module_from_spec(spec)
        sys.modules[EXT_NAME] = module
        try:
            spec.loader.exec_module(module)
        except BaseException:
            del sys.modules[EXT_NAME]
            raise
        return module
    try:
        return importlib.import_module(EXT_NAME)
    except ImportError as exc:
        raise ImportError(
            f"{EXT_PATH} is missing: build it with `python grouped_gemm_b200/csrc/build.py` "
            "(needs nvcc and a C++ compiler; there is no fallback binding)") from exc


_ext = _load_extension()
if not hasattr(_ext, "device_status"):
    raise ImportError(f"the module {EXT_NAME} that is already imported ({getattr(_ext, '__file__', '?')}) is not "
                      "this library's binding")

#: ``gmm(a, b, c, batch_sizes, trans_a, trans_b) -> None`` -- writes into ``c``.
gmm = _ext.gmm


def device_status(device):
    """The per-device status word the kernels OR their B200GMM_STATUS_* bits
    into (int32[1] tensor).  Reading it (``int(device_status(dev))``)
    synchronises; 0 = clean."""
    device = torch.device(device)
    index = device.index if device.index is not None else torch.cuda.current_device()
    return _ext.device_status(index)
