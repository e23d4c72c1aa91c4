"""Helpers shared by the tests: the reference test-suite's input recipe restated,
bf16 bit views, tolerance checks and the golden fixture."""
import ctypes
import hashlib
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden", "ops_test_golden.npz")

# Required tolerance for bf16 results against an fp32-accumulated reference.
RTOL = 1e-2
ATOL = 1e-2


def reference_inputs(bs, x, y):
    """Input recipe of the reference tests (grouped_gemm/ops_test.py:39-41): by
    operator precedence ``(rand - 0.5 * 2) / (y * x)``, i.e. (U[0,1) - 1) / (x*y),
    rounded to bf16.  Stays on CPU here."""
    out = (torch.rand(bs, x, y) - 1.0) / (y * x)
    return out.to(torch.bfloat16)


def variable_batch_sizes(z, m):
    """ops_test.py:87-92."""
    dist = torch.rand(z)
    dist /= dist.sum()
    batch_sizes = (dist * m).to(torch.long)
    batch_sizes[-1] += m * z - batch_sizes.sum()
    return batch_sizes


def bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def from_bits(arr):
    return torch.from_numpy(np.ascontiguousarray(arr).view(np.int16)).view(torch.bfloat16)


def input_digest(a, b):
    return hashlib.sha256(bits(a).tobytes() + bits(b).tobytes()).hexdigest()


def golden_cases():
    data = np.load(GOLDEN)
    keys = sorted({k.split("/")[0] for k in data.files})
    return data, keys


def golden_pair(data, key, name, tensor):
    """(golden values, the same elements of ``tensor``): large results are stored
    as a regular sample of the tensor seen as 2-D (steps in ``<name>_step``)."""
    sr, sc = (int(v) for v in data[key + "/" + name + "_step"])
    gold = from_bits(data[key + "/" + name])
    got = tensor.detach().reshape(-1, tensor.shape[-1])[::sr, ::sc]
    assert tuple(got.shape) == tuple(gold.shape), f"{name}: sample shape {tuple(got.shape)} != {tuple(gold.shape)}"
    return gold, got


def parse_key(key):
    parts = dict((p[0] if p[0] in "zmkn" else p[:-1], p) for p in key.split("_"))
    z = int(parts["z"][1:]); m = int(parts["m"][1:]); k = int(parts["k"][1:]); n = int(parts["n"][1:])
    trans_b = key.split("_tb")[1][0] == "1"
    variable = key.endswith("var1")
    return z, m, k, n, trans_b, variable


def assert_close(actual, expected, rtol=RTOL, atol=ATOL, what=""):
    a, e = actual.float().cpu(), expected.float().cpu()
    assert a.shape == e.shape, f"{what}: shape {tuple(a.shape)} != {tuple(e.shape)}"
    err = (a - e).abs()
    bad = err > (atol + rtol * e.abs())
    assert not bool(bad.any()), (
        f"{what}: {int(bad.sum())}/{bad.numel()} elements outside rtol={rtol} atol={atol}; "
        f"max abs err {float(err.max()):.4g}")


def load_c_oracle():
    from oracle import build as build_oracle
    lib = ctypes.CDLL(build_oracle.build())
    lib.oracle_fill_offsets.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int64,
                                        ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.oracle_fill_offsets.restype = None
    lib.oracle_gmm_bf16.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                    ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int]
    lib.oracle_gmm_bf16.restype = None
    return lib
