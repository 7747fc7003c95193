"""Builds libbeam_b200.so (the C-ABI library with the sm_100a kernels) in-tree with nvcc.

Run as a script (`python build.py`) or call `build()`.  Cross-compiles without a GPU.  The library
links the CUDA runtime statically and resolves the one driver symbol it needs at run time, so it
loads (and exports its symbols) on a machine without a GPU or libcuda.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libbeam_b200.so")
DRIVER = os.path.join(HERE, "beam_bench")
SOURCES = ["gemmrc_launch.cu", "splitk_static.cu", "host_entry.cu", "host_common.cc", "beam_api.cc"]
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-cudart", "static",
]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(HERE, "..", "include", "beam_b200.h"))
    objs = []
    procs = []
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(CSRC, os.path.splitext(src)[0] + ".o")
        objs.append(obj)
        if force or _stale(obj, [path] + headers):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-x", "cu", "-c", path, "-o", obj]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError("nvcc failed on %s" % src)
    if force or procs or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-cudart", "static", "-o", LIB] + objs + ["-lpthread", "-ldl", "-lrt"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout)
            raise RuntimeError("link failed")
    build_driver(force=force or bool(procs))
    return LIB


def build_driver(force=False):
    """beam_bench: the C++ timing driver (csrc/bench_main.cc), linked against libbeam_b200.so beside it."""
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    src = os.path.join(CSRC, "bench_main.cc")
    if not force and not _stale(DRIVER, [src, LIB]):
        return DRIVER
    cmd = [nvcc, "-std=c++17", "-O2", "-cudart", "static", "-o", DRIVER, src, "-L" + HERE, "-lbeam_b200",
           "-Xlinker", "-rpath=$ORIGIN", "-lpthread", "-ldl", "-lrt"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("beam_bench link failed")
    return DRIVER


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
