"""Compile oracle/fill_oracle.c into oracle/libgmm_oracle.so (gcc): the C
restatement of the argument fill that the tests check the CUDA path against.

There is no oracle/_ref target: the reference's own native code cannot be
compiled without its CUTLASS submodule (both of its sources include CUTLASS
headers, and the submodule is empty in a plain checkout), and it has no CPU path.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libgmm_oracle.so")


def build(force=False):
    src = os.path.join(HERE, "fill_oracle.c")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.run(["gcc", "-O2", "-fPIC", "-shared", "-o", LIB, src], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
