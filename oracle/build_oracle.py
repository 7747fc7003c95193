"""Compiles the CPU oracle (gemmrc_oracle.c) into oracle/liboracle.so with gcc + OpenMP.

Test infrastructure: only tests/, the smoke check and the benchmark's CPU legs load the result.
The reference itself has no CPU implementation of this path and its CUDA sources need CUTLASS,
libtorch and pybind11, so there is nothing to compile into oracle/_ref.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "gemmrc_oracle.c")
LIB = os.path.join(HERE, "liboracle.so")


def build(force=False):
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = ["gcc", "-O3", "-mavx2", "-mfma", "-mf16c", "-fopenmp", "-shared", "-fPIC", "-std=c11",
           "-o", LIB, SRC, "-lm"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("oracle build failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
