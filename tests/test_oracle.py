"""CPU tests of the oracle: pinned to the golden vectors (torch.matmul, the reference's own answer
function, evaluated on the CPU) and to fp64; fp16 conversion bit-exactness; split-K and LayerNorm
restatements; the error metric."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gemmrc_golden.npz")
CASES = ["tiny", "ragged", "tile", "wide", "deepk"]


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


@pytest.mark.parametrize("name", CASES)
def test_oracle_reproduces_reference_answer_function(oracle_mod, golden, name):
    a, b, c = golden[name + "_a"], golden[name + "_b"], golden[name + "_c"]
    got = oracle_mod.gemmrc(a, b)
    assert got.dtype == np.float16 and got.shape == c.shape
    # torch's CPU half matmul accumulates in fp32 like the oracle, but may order k differently:
    # equal within one fp16 rounding of the fp64 value, and within the parity tolerance of each other.
    assert oracle_mod.floored_max_rel(got, c) <= 2e-3
    assert oracle_mod.floored_max_rel(got, golden[name + "_c64"]) <= 1e-3


@pytest.mark.parametrize("name", CASES)
def test_oracle_fp64_rows(oracle_mod, golden, name):
    a, b = golden[name + "_a"], golden[name + "_b"]
    rows = np.arange(0, a.shape[0], 3)
    got = oracle_mod.gemmrc_rows_f64(a, b, rows)
    np.testing.assert_allclose(got, golden[name + "_c64"][rows], rtol=1e-5, atol=1e-5)


def test_fp16_conversions_bit_exact(oracle_mod):
    L = oracle_mod.lib()
    every_half = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    as_float = every_half.view(np.float16).astype(np.float32)
    for h in range(0, 65536, 7):
        f = L.oracle_half_to_float(h)
        if np.isnan(as_float[h]):
            assert np.isnan(f)
        else:
            assert f == as_float[h]
    rng = np.random.Generator(np.random.PCG64(7))
    x = (rng.standard_normal(20000) * np.exp(rng.uniform(-22, 12, 20000))).astype(np.float32)
    # ties and boundaries: halfway points between consecutive halves, overflow edge, subnormal edge
    halves = np.arange(0, 0x7C00, 37, dtype=np.uint16).view(np.float16).astype(np.float64)
    nxt = (np.arange(0, 0x7C00, 37, dtype=np.uint16) + 1).view(np.float16).astype(np.float64)
    ties = ((halves + nxt) / 2).astype(np.float32)
    x = np.concatenate([x, ties, -ties, np.float32([65504, 65519.99, 65520, 1e9, 2.0 ** -24, 2.0 ** -25,
                                                    2.0 ** -25 * 1.0001, 0.0, -0.0])])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    got = np.array([L.oracle_float_to_half(float(v)) for v in x], dtype=np.uint16)
    assert (got == want).all()


def test_empty_and_bad_arguments(oracle_mod):
    L = oracle_mod.lib()
    assert L.oracle_gemmrc_f16(None, None, None, 0, 4, 4) != 0
    a = np.zeros((4, 8), np.float16)
    b = np.zeros((4, 8), np.float16)
    with pytest.raises(RuntimeError):
        oracle_mod.gemmrc_splitk(a, b, 5)  # more slices than 64-wide k-blocks
    with pytest.raises(TypeError):
        oracle_mod.gemmrc(a.astype(np.float32), b)


def test_splitk_restatement_matches_plain(oracle_mod):
    rng = np.random.Generator(np.random.PCG64(11))
    a = rng.uniform(-1, 1, (40, 1024)).astype(np.float16)
    b = rng.uniform(-1, 1, (24, 1024)).astype(np.float16)
    plain = oracle_mod.gemmrc(a, b)
    assert (oracle_mod.gemmrc_splitk(a, b, 1) == plain).all()  # one slice is the plain loop, bit for bit
    for s in (2, 5, 16):
        sk = oracle_mod.gemmrc_splitk(a, b, s)
        assert oracle_mod.floored_max_rel(sk, plain) <= 2e-3
    # linearity in the slices: with K made of two halves where the second half of A is zero, slices see it
    a2 = a.copy()
    a2[:, 512:] = 0
    assert (oracle_mod.gemmrc_splitk(a2, b, 2) == oracle_mod.gemmrc(a2[:, :512], b[:, :512])).all()


@pytest.mark.parametrize("name", CASES)
def test_layernorm_restatement(oracle_mod, golden, name):
    a, b = golden[name + "_a"], golden[name + "_b"]
    gamma, beta = golden[name + "_gamma"], golden[name + "_beta"]
    got = oracle_mod.gemm_layernorm(a, b, gamma, beta, 1e-5)
    assert oracle_mod.floored_max_rel(got, golden[name + "_ln64"]) <= 2e-3
    rows = np.arange(0, a.shape[0], 5)
    t64 = oracle_mod.gemm_layernorm_rows_f64(a, b, gamma, beta, rows, 1e-5)
    np.testing.assert_allclose(t64, golden[name + "_ln64"][rows], rtol=2e-5, atol=2e-5)


def test_error_metric():
    import oracle
    ref = np.array([100.0, 1.0, 0.0, -50.0])
    assert oracle.floored_max_rel(ref, ref) == 0.0
    rms = np.sqrt(np.mean(ref * ref))
    got = ref.copy()
    got[2] = 0.5  # an entry whose reference is zero is judged against 1 % of the rms
    assert abs(oracle.floored_max_rel(got, ref) - 0.5 / (1e-2 * rms)) < 1e-12
    got = ref.copy()
    got[0] = 101.0
    assert abs(oracle.floored_max_rel(got, ref) - 0.01) < 1e-12
    assert oracle.floored_max_rel(np.zeros(0), np.zeros(0)) == 0.0
