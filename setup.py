"""pip-installable build of grouped_gemm_b200 (the role of the reference's
setup.py: compile the native op for the GPU at hand and ship the Python
wrappers).  The native parts are built in-tree by grouped_gemm_b200/csrc/build.py:
libb200gmm.so (nvcc, -gencode arch=compute_100a,code=sm_100a) and the torch
extension module that binds it; both are then packaged as data files.

    pip install --no-build-isolation .
"""
import importlib.util
import os

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildNative(build_py):
    def run(self):
        spec = importlib.util.spec_from_file_location(
            "b200gmm_build", os.path.join(HERE, "grouped_gemm_b200", "csrc", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build_all()
        super().run()


setup(
    name="grouped_gemm_b200",
    version="0.1.0",
    description="B200-native grouped GEMM with the Python API of tgale96/grouped_gemm",
    packages=find_packages(include=["grouped_gemm_b200", "grouped_gemm_b200.*"]),
    package_data={"grouped_gemm_b200": ["csrc/libb200gmm.so", "csrc/torch_ext/build/*.so", "csrc/*.cu",
                                        "csrc/*.cuh", "csrc/*.py", "csrc/torch_ext/*.cpp"]},
    cmdclass={"build_py": BuildNative},
    python_requires=">=3.9",
    install_requires=["torch>=2.4"],
)
