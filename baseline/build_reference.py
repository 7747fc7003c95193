"""Builds the reference's own CUDA extension (`beam_C`: its CuTe / CUTLASS sm80-era kernels and cuBLAS wrappers),
unmodified, for sm_100a, as a timed comparison baseline and a second parity witness on the GPU box.

Sources are compiled where they lie (the reference checkout, read-only); nothing is copied into this
repository.  Objects and the module go to baseline/_ref/ (git-ignored; shipped to the GPU box with the other
built artefacts).  The reference's CMake build needs ccache and a populated CUTLASS submodule, neither of which
exists here; this recipe compiles the same translation units directly against the CUTLASS/CuTe headers vendored
in the image's site-packages, libtorch and pybind11.

    python baseline/build_reference.py /path/to/reference

If a needed header tree is missing the script says so and exits 1; bench.py then reports the reference kernels
as "not built".
"""
import glob
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def main():
    if len(sys.argv) != 2:
        print("usage: python baseline/build_reference.py /path/to/the/reference/checkout")
        return 2
    ref = sys.argv[1]
    cuda_dir = os.path.join(ref, "cuda")
    if not os.path.isdir(cuda_dir):
        print("reference checkout not found at", ref)
        return 1
    site = sysconfig.get_paths()["purelib"]
    cutlass = None
    for cand in (os.path.join(site, "flashinfer", "data", "cutlass"),
                 os.path.join(site, "tilelang", "3rdparty", "cutlass")):
        if os.path.isdir(os.path.join(cand, "include", "cute")):
            cutlass = cand
            break
    if cutlass is None:
        print("no CUTLASS/CuTe header tree found in site-packages")
        return 1
    import pybind11
    import torch
    torch_dir = os.path.dirname(torch.__file__)
    os.makedirs(OUT, exist_ok=True)
    inc = ["-I" + os.path.join(cuda_dir, "include"), "-I" + os.path.join(cutlass, "include"),
           "-I" + os.path.join(cutlass, "tools", "util", "include"), "-I" + pybind11.get_include(),
           "-I" + sysconfig.get_paths()["include"]]
    torch_inc = ["-I" + os.path.join(torch_dir, "include"),
                 "-I" + os.path.join(torch_dir, "include", "torch", "csrc", "api", "include"),
                 "-I/usr/local/cuda/include"]
    cu = sorted(glob.glob(os.path.join(cuda_dir, "*", "*.cu")))
    cc = sorted(glob.glob(os.path.join(cuda_dir, "*.cc")) + glob.glob(os.path.join(cuda_dir, "*", "*.cc")))
    jobs = []
    for src in cu:
        obj = os.path.join(OUT, os.path.basename(os.path.dirname(src)) + "_" + os.path.basename(src) + ".o")
        jobs.append((obj, ["nvcc", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "--use_fast_math",
                           "--expt-relaxed-constexpr", "-O3", "-Xcompiler", "-fPIC"] + inc + ["-c", src, "-o", obj]))
    for src in cc:
        obj = os.path.join(OUT, os.path.basename(os.path.dirname(src)) + "_" + os.path.basename(src) + ".o")
        jobs.append((obj, ["g++", "-std=c++20", "-O2", "-fPIC", "-D_GLIBCXX_USE_CXX11_ABI=1",
                           "-DINTERFACE_NAME=beam_C"] + inc + torch_inc + ["-c", src, "-o", obj]))

    def run(job):
        obj, cmd = job
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        return obj, r.returncode, r.stdout[-2000:]

    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        results = list(ex.map(run, jobs))
    for obj, rc, out in results:
        if rc != 0:
            print("FAILED", obj)
            print(out)
            return 1
    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    so = os.path.join(OUT, "beam_C" + suffix)
    link = ["g++", "-shared", "-o", so] + [o for o, _, _ in results] + [
        "-L" + os.path.join(torch_dir, "lib"), "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
        "-ltorch_python", "-L/usr/local/cuda/lib64", "-lcudart", "-lcublas",
        "-Wl,-rpath," + os.path.join(torch_dir, "lib"), "-Wl,-rpath,/usr/local/cuda/lib64"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        print(r.stdout[-3000:])
        return 1
    for o, _, _ in results:
        os.remove(o)
    print("built", so)
    return 0


if __name__ == "__main__":
    sys.exit(main())
