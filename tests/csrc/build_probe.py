"""Builds tests/csrc/libwait_probe.so, the test-only kernel that makes a bounded device wait run out
(tests/test_bounded_wait.py).  nvcc cross-compiles it for sm_100a without a GPU."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "wait_probe.cu")
LIB = os.path.join(HERE, "libwait_probe.so")


def build(force=False):
    deps = [SRC, os.path.join(HERE, "..", "..", "general-nvgpu-testing_b200", "csrc", "umma_common.cuh"),
            os.path.join(HERE, "..", "..", "general-nvgpu-testing_b200", "csrc", "sm100_ptx.cuh")]
    if not force and os.path.exists(LIB) and all(os.path.getmtime(d) <= os.path.getmtime(LIB) for d in deps):
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler",
           "-fPIC,-fvisibility=hidden", "-cudart", "static", "-shared", "-o", LIB, SRC, "-lpthread", "-ldl", "-lrt"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed on wait_probe.cu:\n" + r.stdout)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
