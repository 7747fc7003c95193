"""Generates tests/golden/gemmrc_golden.npz.

The reference's only correctness check compares each kernel with `torch.matmul(a, b.t(), out=c)`
(python/gemm_test.py:114-115,139-140,164-165).  This script evaluates that same call on the CPU, on small
seeded fp16 inputs, and stores inputs and outputs; the CPU oracle must reproduce the outputs and the
CUDA kernels must match them within the stated tolerance.  It also stores an fp64 evaluation, and, for
the fused GEMM+LayerNorm path (which the reference does not implement), torch's layer_norm applied in
fp64 to the fp64 GEMM result.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = [
    # name, M, N, K, distribution
    ("tiny", 8, 16, 64, "uniform"),
    ("ragged", 72, 40, 136, "uniform"),
    ("tile", 128, 128, 256, "uniform"),
    ("wide", 96, 264, 320, "normal01"),
    ("deepk", 16, 24, 4096, "uniform"),
]


def draw(rng, shape, dist):
    if dist == "uniform":
        return rng.uniform(-1.0, 1.0, shape).astype(np.float16)
    return (rng.standard_normal(shape) * 0.1).astype(np.float16)


def main():
    out = {}
    for idx, (name, m, n, k, dist) in enumerate(CASES):
        rng = np.random.Generator(np.random.PCG64(1234 + idx))
        a = draw(rng, (m, k), dist)
        b = draw(rng, (n, k), dist)
        ta, tb = torch.from_numpy(a), torch.from_numpy(b)
        c = torch.empty(m, n, dtype=torch.float16)
        torch.matmul(ta, tb.t(), out=c)  # the reference's ansfunc, on the CPU
        c64 = torch.matmul(ta.double(), tb.double().t())
        gamma = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float16)
        beta = (0.1 * rng.standard_normal(n)).astype(np.float16)
        ln64 = torch.nn.functional.layer_norm(c64, (n,), torch.from_numpy(gamma).double(),
                                              torch.from_numpy(beta).double(), 1e-5)
        out[name + "_a"] = a
        out[name + "_b"] = b
        out[name + "_c"] = c.numpy()
        out[name + "_c64"] = c64.numpy().astype(np.float32)  # fp64 result, stored in fp32 to stay small
        out[name + "_gamma"] = gamma
        out[name + "_beta"] = beta
        out[name + "_ln64"] = ln64.numpy().astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "gemmrc_golden.npz"), **out)
    print("wrote", os.path.join(HERE, "gemmrc_golden.npz"), "torch", torch.__version__)


if __name__ == "__main__":
    main()
