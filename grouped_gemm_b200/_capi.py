"""ctypes binding of libb200gmm.so (C ABI declared in include/b200gmm.h).

The library is the only compute path: if it cannot be loaded the import of
``grouped_gemm_b200.backend`` fails; there is no fallback implementation.
"""
import ctypes
import os

# torch first, so that its CUDA runtime is the one the library binds to
# (same reason as grouped_gemm/backend.py:1-3 in the reference).
import torch  # noqa: F401

_HERE = os.path.dirname(os.path.abspath(__file__))
# B200GMM_LIBRARY: path of the built library, for installs that keep it elsewhere.
LIB_PATH = os.environ.get("B200GMM_LIBRARY") or os.path.join(_HERE, "csrc", "libb200gmm.so")

OK = 0
MAX_EXPERTS = 1024
FILL_FIELDS = 9
SCHEDULE_FIELDS = 6
STATIC_MAX_EXPERTS = 256
STATUS_TIMEOUT = 0x1
STATUS_NEGATIVE_SIZE = 0x2
STATUS_ROWS_OVERFLOW = 0x4
STATUS_BAD_ROW_INDEX = 0x8
STATUS_BAD_ROW_DEST = 0x10
STATUS_HANDOFF = 0x20

# name -> (restype, argtypes); exactly the symbols include/b200gmm.h declares.
_c = ctypes
SIGNATURES = {
    "b200gmm_workspace_bytes": (_c.c_int, [_c.c_int, _c.POINTER(_c.c_size_t)]),
    "b200gmm_run": (_c.c_int, [
        _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int,
        _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int, _c.c_int,
        _c.c_void_p, _c.c_size_t, _c.c_void_p, _c.c_void_p]),
    "b200gmm_run_static": (_c.c_int, [
        _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int,
        _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int, _c.c_int,
        _c.c_void_p, _c.c_void_p]),
    "b200gmm_run_scatter": (_c.c_int, [
        _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_int, _c.c_int,
        _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int,
        _c.c_void_p, _c.c_size_t, _c.c_void_p, _c.c_void_p]),
    "b200gmm_run_scatter_push": (_c.c_int, [
        _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_int, _c.c_int,
        _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int,
        _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
        _c.c_void_p, _c.c_size_t, _c.c_void_p, _c.c_void_p]),
    "b200gmm_sum_slots": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int, _c.c_int64, _c.c_void_p]),
    "b200gmm_run_combine": (_c.c_int, [
        _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_int, _c.c_void_p,
        _c.c_int, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int,
        _c.c_void_p, _c.c_size_t, _c.c_void_p, _c.c_void_p]),
    "b200gmm_run_gather": (_c.c_int, [
        _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64,
        _c.c_void_p,
        _c.c_int, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int,
        _c.c_void_p, _c.c_size_t, _c.c_void_p, _c.c_void_p]),
    "b200gmm_run_gather_wgrad": (_c.c_int, [
        _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
        _c.c_int, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int64,
        _c.c_void_p, _c.c_size_t, _c.c_void_p, _c.c_void_p]),
    "b200gmm_run_swiglu": (_c.c_int, [
        _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_void_p,
        _c.c_int, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int,
        _c.c_void_p, _c.c_size_t, _c.c_void_p, _c.c_void_p]),
    "b200gmm_run_swiglu_backward": (_c.c_int, [
        _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
        _c.c_int, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int,
        _c.c_void_p, _c.c_size_t, _c.c_void_p, _c.c_void_p]),
    "b200gmm_push_rows": (_c.c_int, [
        _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
        _c.c_int, _c.c_void_p]),
    "b200gmm_fill_offsets": (_c.c_int, [
        _c.c_void_p, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int, _c.c_int,
        _c.c_void_p, _c.c_void_p]),
    "b200gmm_schedule_host": (_c.c_int, [
        _c.c_void_p, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int, _c.c_int, _c.c_int,
        _c.c_void_p, _c.c_int64, _c.POINTER(_c.c_int64)]),
    "b200gmm_schedule_device": (_c.c_int, [
        _c.c_void_p, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int, _c.c_int, _c.c_int,
        _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_void_p]),
    "b200gmm_selftest_wait_timeout": (_c.c_int, [_c.c_int64, _c.c_void_p, _c.c_void_p]),
    "b200gmm_tile_shape": (_c.c_int, [_c.c_int, _c.POINTER(_c.c_int)]),
    "b200gmm_launch_count": (_c.c_int64, []),
    "b200gmm_strerror": (_c.c_char_p, [_c.c_int]),
}

_lib = None


def load():
    """Load the shared library once and attach prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python grouped_gemm_b200/csrc/build.py` "
            "(needs nvcc; there is no non-CUDA fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        if not hasattr(lib, name):
            raise ImportError(f"{LIB_PATH} lacks {name}: it is older than its sources, rebuild it with "
                              "`python grouped_gemm_b200/csrc/build.py --force`")
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def strerror(code):
    return load().b200gmm_strerror(int(code)).decode()


def check(code, what):
    """Map a non-zero return code to RuntimeError, the exception type the
    reference's TORCH_CHECK failures surface as (csrc/grouped_gemm.cu:21-32)."""
    if code != OK:
        raise RuntimeError(f"{what}: {strerror(code)} (code {code})")


def workspace_bytes(z):
    out = ctypes.c_size_t(0)
    check(load().b200gmm_workspace_bytes(int(z), ctypes.byref(out)), "b200gmm_workspace_bytes")
    return out.value


def launch_count():
    return int(load().b200gmm_launch_count())


def tile_shape(cluster_ctas=1):
    out = (ctypes.c_int * 3)()
    check(load().b200gmm_tile_shape(int(cluster_ctas), out), "b200gmm_tile_shape")
    return tuple(out)
