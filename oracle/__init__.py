"""CPU oracle for the fp16 rc GEMM path (test infrastructure, never a product dependency).

Thin numpy front end over oracle/liboracle.so (built from gemmrc_oracle.c by build_oracle.py).
Matrices are numpy float16 arrays, C-contiguous:  A [M,K], B [N,K]  ->  C [M,N].
Also holds the error metric the parity tests use.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            from . import build_oracle
            build_oracle.build()
        L = ctypes.CDLL(path)
        vp, i, f, d = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_double
        L.oracle_gemmrc_f16.argtypes = [vp, vp, vp, i, i, i]
        L.oracle_gemmrc_f32.argtypes = [vp, vp, vp, i, i, i]
        L.oracle_gemmrc_splitk_f16.argtypes = [vp, vp, vp, i, i, i, i]
        L.oracle_gemmrc_rows_f64.argtypes = [vp, vp, vp, i, vp, i, i, i]
        L.oracle_gemm_layernorm_f16.argtypes = [vp, vp, vp, vp, f, vp, i, i, i]
        L.oracle_gemm_layernorm_rows_f64.argtypes = [vp, vp, vp, vp, d, vp, i, vp, i, i, i]
        L.oracle_float_to_half.argtypes = [f]
        L.oracle_float_to_half.restype = ctypes.c_uint16
        L.oracle_half_to_float.argtypes = [ctypes.c_uint16]
        L.oracle_half_to_float.restype = f
        L.oracle_num_threads.restype = i
        L.oracle_set_num_threads.argtypes = [i]
        _LIB = L
    return _LIB


def _h(x):
    x = np.ascontiguousarray(x)
    if x.dtype != np.float16:
        raise TypeError("expected float16, got %s" % x.dtype)
    return x


def _p(x):
    return ctypes.c_void_p(x.ctypes.data)


def _check(st, what):
    if st != 0:
        raise RuntimeError("%s failed with status %d" % (what, st))


def num_threads():
    return int(lib().oracle_num_threads())


def use_all_cores():
    """Use every core this process may run on, whatever OMP_NUM_THREADS says; returns the thread count."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().oracle_set_num_threads(n)
    return num_threads()


def gemmrc(a, b):
    """fp16( fp32-accumulated a @ b.T ), k ascending, one accumulator per output."""
    a, b = _h(a), _h(b)
    m, k = a.shape
    n, k2 = b.shape
    assert k == k2
    c = np.empty((m, n), dtype=np.float16)
    _check(lib().oracle_gemmrc_f16(_p(a), _p(b), _p(c), m, n, k), "oracle_gemmrc_f16")
    return c


def gemmrc_f32(a, b):
    a, b = _h(a), _h(b)
    m, k = a.shape
    n, _ = b.shape
    c = np.empty((m, n), dtype=np.float32)
    _check(lib().oracle_gemmrc_f32(_p(a), _p(b), _p(c), m, n, k), "oracle_gemmrc_f32")
    return c


def gemmrc_splitk(a, b, slices):
    a, b = _h(a), _h(b)
    m, k = a.shape
    n, _ = b.shape
    c = np.empty((m, n), dtype=np.float16)
    _check(lib().oracle_gemmrc_splitk_f16(_p(a), _p(b), _p(c), m, n, k, int(slices)), "oracle_gemmrc_splitk_f16")
    return c


def gemmrc_rows_f64(a, b, rows):
    """float64 truth for the given row indices: shape [len(rows), N]."""
    a, b = _h(a), _h(b)
    m, k = a.shape
    n, _ = b.shape
    rows = np.ascontiguousarray(rows, dtype=np.int32)
    out = np.empty((len(rows), n), dtype=np.float64)
    _check(lib().oracle_gemmrc_rows_f64(_p(a), _p(b), _p(rows), len(rows), _p(out), m, n, k), "oracle_gemmrc_rows_f64")
    return out


def gemm_layernorm(x, w, gamma, beta, eps=1e-5):
    x, w, gamma, beta = _h(x), _h(w), _h(gamma), _h(beta)
    m, k = x.shape
    n, _ = w.shape
    assert gamma.shape == (n,) and beta.shape == (n,)
    out = np.empty((m, n), dtype=np.float16)
    _check(lib().oracle_gemm_layernorm_f16(_p(x), _p(w), _p(gamma), _p(beta), float(eps), _p(out), m, n, k),
           "oracle_gemm_layernorm_f16")
    return out


def gemm_layernorm_rows_f64(x, w, gamma, beta, rows, eps=1e-5):
    x, w, gamma, beta = _h(x), _h(w), _h(gamma), _h(beta)
    m, k = x.shape
    n, _ = w.shape
    rows = np.ascontiguousarray(rows, dtype=np.int32)
    out = np.empty((len(rows), n), dtype=np.float64)
    _check(lib().oracle_gemm_layernorm_rows_f64(_p(x), _p(w), _p(gamma), _p(beta), float(eps), _p(rows), len(rows),
                                                _p(out), m, n, k), "oracle_gemm_layernorm_rows_f64")
    return out


# ---------------------------------------------------------------------------------- error metric
REL_TOL = 1e-2  # bound on floored_max_rel for fp16 outputs


def floored_max_rel(got, ref, rms=None):
    """max |got - ref| / max(|ref|, 1e-2 * rms(ref)).

    Plain relative error is ill-posed for GEMM outputs (entries near zero make it arbitrarily large for a
    perfectly rounded result), so the denominator is floored at 1 % of the root-mean-square of the
    reference.  A correctly rounded fp16 result scores about 4.9e-4 (half an fp16 ulp).
    """
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    if rms is None:
        rms = float(np.sqrt(np.mean(ref * ref))) if ref.size else 0.0
    den = np.maximum(np.abs(ref), 1e-2 * rms)
    den = np.where(den == 0, 1.0, den)
    return float(np.max(np.abs(got - ref) / den)) if ref.size else 0.0


def max_abs_over_max(got, ref):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.max(np.abs(got - ref)) / max(np.max(np.abs(ref)), 1e-30))
