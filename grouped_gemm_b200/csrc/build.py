"""Build libb200gmm.so (nvcc, sm_100a) and the torch extension module in-tree.

Usage: ``python grouped_gemm_b200/csrc/build.py [--force] [--verbose]`` (run it
as a script: importing the package first would try to load the library).
The library has no torch dependency; it links the shared CUDA runtime so that a
process that already loaded torch's libcudart shares one runtime with it.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
SOURCES = ["b200gmm.cu"]
HEADERS = ["gmm_kernel.cuh", "ptx.cuh", "schedule.cuh", "ep_exchange.cuh", os.path.join(ROOT, "include", "b200gmm.h")]
LIB = os.path.join(HERE, "libb200gmm.so")


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def is_stale():
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    deps = [os.path.join(HERE, s) for s in SOURCES] + [
        h if os.path.isabs(h) else os.path.join(HERE, h) for h in HEADERS
    ]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force=False, verbose=False):
    """Compile the library if it is missing or older than its sources."""
    if not force and not is_stale():
        return LIB
    nvcc = _nvcc()
    cuda_lib = os.path.join(os.path.dirname(os.path.dirname(nvcc)), "lib64")
    cmd = [
        nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-shared", "-cudart", "shared", "-Xcompiler", "-fPIC",
        "-Xlinker", "-rpath," + cuda_lib,
        "-o", LIB,
    ] + [os.path.join(HERE, s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libb200gmm.so")
    return LIB


# The torch extension carries the name of the reference's compiled module
# (setup.py:35 and grouped_gemm/backend.py:8 there) and is put beside the packages,
# so that ``import grouped_gemm_backend`` finds it the way it finds the reference's.
EXT_NAME = "grouped_gemm_backend"
EXT_DIR = os.path.join(HERE, "torch_ext")
EXT_SRC = os.path.join(EXT_DIR, "binding.cpp")
EXT_BUILD = os.path.join(EXT_DIR, "build")
EXT_BUILT = os.path.join(EXT_BUILD, EXT_NAME + ".so")
EXT_LIB = os.path.join(ROOT, EXT_NAME + ".so")


def binding_is_stale():
    if not os.path.exists(EXT_LIB):
        return True
    built = os.path.getmtime(EXT_LIB)
    return any(os.path.getmtime(d) > built for d in (EXT_SRC, os.path.join(ROOT, "include", "b200gmm.h")))


def build_torch_binding(force=False, verbose=False):
    """Compile the torch extension module (torch_ext/binding.cpp) in-tree.  It is
    plain C++ (no device code): argument checks, stream and workspace from torch,
    then the C ABI of libb200gmm.so, which it finds through its rpath (relative
    to its own place beside the ``grouped_gemm_b200`` package)."""
    if not force and not binding_is_stale():
        return EXT_LIB
    build(force=False, verbose=verbose)  # the extension links against the library
    from torch.utils.cpp_extension import load
    os.makedirs(EXT_BUILD, exist_ok=True)
    load(name=EXT_NAME, sources=[EXT_SRC], extra_include_paths=[os.path.join(ROOT, "include")],
         extra_cflags=["-O2", "-std=c++17"],
         extra_ldflags=["-L" + HERE, "-lb200gmm", "-Wl,-rpath,\\$$ORIGIN/grouped_gemm_b200/csrc", "-Wl,-rpath," + HERE],
         build_directory=EXT_BUILD, with_cuda=True, verbose=verbose, is_python_module=False)
    if not os.path.exists(EXT_BUILT):
        raise RuntimeError("torch extension build did not produce " + EXT_BUILT)
    shutil.copy2(EXT_BUILT, EXT_LIB)
    os.utime(EXT_LIB, None)
    return EXT_LIB


def build_all(force=False, verbose=False):
    return build(force=force, verbose=verbose), build_torch_binding(force=force, verbose=verbose)


if __name__ == "__main__":
    for path in build_all(force="--force" in sys.argv, verbose="--verbose" in sys.argv):
        print(path)
