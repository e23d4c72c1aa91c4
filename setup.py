"""pip-installable build (the role of the reference's setup.py:33-76: compile the
native op for the GPU at hand and ship the Python wrappers).  Installs

* ``grouped_gemm``: the reference's import name (``grouped_gemm.ops``, ``grouped_gemm.backend``);
* ``grouped_gemm_backend``: the compiled module the reference's backend.py:8 imports;
* ``grouped_gemm_b200``: the implementation, with libb200gmm.so (the C-ABI library) inside.

The native parts are built in-tree by grouped_gemm_b200/csrc/build.py (nvcc,
-gencode arch=compute_100a,code=sm_100a, and a C++ torch extension) and copied
into the build as they are.

    pip install --no-build-isolation .
"""
import importlib.util
import os
import shutil

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildNative(build_py):
    def run(self):
        spec = importlib.util.spec_from_file_location(
            "b200gmm_build", os.path.join(HERE, "grouped_gemm_b200", "csrc", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _, ext = mod.build_all()
        super().run()
        # the compiled module sits beside the packages, as the reference's does
        os.makedirs(self.build_lib, exist_ok=True)
        shutil.copy2(ext, os.path.join(self.build_lib, os.path.basename(ext)))


setup(
    name="grouped_gemm_b200",
    version="0.2.0",
    description="B200-native grouped GEMM with the Python API of tgale96/grouped_gemm",
    packages=find_packages(include=["grouped_gemm", "grouped_gemm_b200", "grouped_gemm_b200.*"]),
    package_data={"grouped_gemm_b200": ["csrc/libb200gmm.so", "csrc/*.cu", "csrc/*.cuh", "csrc/*.py",
                                        "csrc/torch_ext/*.cpp"]},
    cmdclass={"build_py": BuildNative},
    python_requires=">=3.9",
    install_requires=["torch>=2.4"],
)
