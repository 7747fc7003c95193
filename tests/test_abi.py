"""CPU tests of the C-ABI library: it loads without a GPU, exports every symbol the header declares,
and rejects bad arguments with status codes (no compute is attempted here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "beam_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"BEAM_API\s+[\w\s\*]+?\b(beam_\w+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib(built_library):
    return ctypes.CDLL(built_library)


def test_header_declares_the_registry():
    names = declared_symbols()
    for required in ("beam_custom_gemmrc_128x128", "beam_custom_gemmrc_128x256", "beam_cutlass_gemmrc",
                     "beam_cutlass_gemmrc_spec", "beam_cutlass_gemmrc_splitk", "beam_cutlass_gemmrc_splitk_spec",
                     "beam_gemmrc_layernorm", "beam_gemmrc_fp16", "beam_gemmrc_fp16_host", "beam_status_string"):
        assert required in names


def test_library_exports_every_declared_symbol(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), "libbeam_b200.so does not export %s" % name


def test_status_strings(lib):
    lib.beam_status_string.restype = ctypes.c_char_p
    seen = set()
    for code in range(0, 9):
        s = lib.beam_status_string(code).decode()
        assert s and s != "unknown status"
        seen.add(s)
    assert len(seen) == 9
    assert lib.beam_status_string(99).decode() == "unknown status"
    lib.beam_version.restype = ctypes.c_char_p
    assert b"sm_100a" in lib.beam_version()


def _aligned_buffer(nbytes):
    raw = ctypes.create_string_buffer(nbytes + 64)
    addr = (ctypes.addressof(raw) + 63) & ~63
    return raw, addr


def test_argument_validation_needs_no_gpu(lib):
    vp, i = ctypes.c_void_p, ctypes.c_int
    f = lib.beam_cutlass_gemmrc
    f.argtypes = [vp, vp, vp, i, i, i, vp]
    keep, p = _aligned_buffer(1 << 16)
    assert f(None, p, p, 64, 64, 64, None) == 1       # null pointer
    assert f(p, p, p, 0, 64, 64, None) == 1           # empty problem
    assert f(p, p, p, 64, 64, -8, None) == 1
    assert f(p + 2, p, p, 64, 64, 64, None) == 3      # misaligned A
    assert f(p, p, p, 64, 60, 64, None) == 3          # N not a multiple of 8
    assert f(p, p, p, 64, 64, 60, None) == 3          # K not a multiple of 8
    # a well-formed call on a machine without a GPU reports "no device", never crashes or falls back
    import torch
    if not torch.cuda.is_available():
        assert f(p, p, p, 64, 64, 64, None) == 8
    g = lib.beam_cutlass_gemmrc_spec
    g.argtypes = [vp, vp, vp, i, i, i, i, i, i, i, vp]
    assert g(p, p, p, 64, 64, 64, 192, 128, 64, 64, None) == 2   # unknown tile family
    assert g(p, p, p, 64, 64, 64, 128, 96, 64, 64, None) == 2


def test_allgather_entry_validates_without_gpu(lib):
    vp, i = ctypes.c_void_p, ctypes.c_int
    f = lib.beam_gemmrc_fp16_allgather
    f.argtypes = [vp, vp, ctypes.POINTER(vp), i, i, i, i, i, vp, vp]
    keep, p = _aligned_buffer(1 << 16)
    ptrs = (vp * 2)(vp(p), vp(p))
    assert f(p, p, None, 2, 0, 64, 64, 64, None, None) == 1          # no destination list
    assert f(p, p, ptrs, 9, 0, 64, 64, 64, None, None) == 1          # more than 8 ranks
    assert f(p, p, ptrs, 2, 2, 64, 64, 64, None, None) == 1          # rank out of range
    assert f(p, p, ptrs, 2, 0, 0, 64, 64, None, None) == 1           # empty block
    holes = (vp * 2)(vp(p), vp(None))
    assert f(p, p, holes, 2, 0, 64, 64, 64, None, None) == 1         # a missing peer pointer
    assert f(p, p, ptrs, 2, 1, 64, 60, 64, None, None) == 3          # N not a multiple of 8


def test_splitk_sizing_functions(lib):
    i = ctypes.c_int
    ws = lib.beam_gemmrc_splitk_workspace_bytes
    ws.restype = ctypes.c_size_t
    ws.argtypes = [i, i, i, i, i]
    assert ws(128, 256, 65536, 128, 64) == 64 * 128 * 256 * 4
    # problems with M, N <= 64 run folded (two k-blocks per UMMA): every slice leaves two partial planes
    assert ws(64, 64, 131072, 64, 16) == 2 * 16 * 64 * 64 * 4
    assert ws(64, 64, 131072, 128, 16) == 16 * 64 * 64 * 4        # an explicit 128-wide tile does not fold
    assert ws(0, 64, 64, 0, 0) == 0
    h = lib.beam_gemmrc_splitk_heuristic
    h.argtypes = [i, i, i, i]
    s = h(128, 256, 65536, 128)
    assert 1 <= s <= 256 and s * 2 <= 148 + 2            # two 128-wide tiles share the SMs
    assert h(8192, 8192, 8192, 0) == 1                    # a large-MN problem is not split
    assert h(64, 64, 256, 64) == 1                        # too little K to split
    # a split factor beyond K/64 falls back to the heuristic
    assert ws(64, 64, 128, 64, 50) == 2 * h(64, 64, 128, 64) * 64 * 64 * 4
    # medium M, N with more arithmetic than memory time (M N / (M + N) >= 200): the 256-wide tile, a slice per SM,
    # at least 8 k-blocks per slice (148 SMs assumed without a device)
    assert h(512, 512, 8192, 0) == 16                     # 8 tiles of 128 x 256: 148 / 8 = 18, capped by 128 k-blocks / 8
    assert h(1024, 1024, 8192, 0) == 4                    # 32 tiles: 148 / 32
    assert ws(512, 512, 8192, 0, 0) == 16 * 512 * 512 * 4
    assert h(128, 256, 65536, 0) == h(128, 256, 65536, 128)   # the HBM-bound shapes keep the 128-wide tile
    ln = lib.beam_gemmrc_layernorm_workspace_bytes
    ln.restype = ctypes.c_size_t
    ln.argtypes = [i, i, i]
    # N tiles <= CTA pairs: tiles wait in TMEM, the workspace holds statistics (8 bytes per row per 256-wide tile)
    # and tickets only; with more N tiles than pairs an fp32 panel is parked as well
    assert 16384 * 16 * 8 <= ln(16384, 4096, 4096) < 16384 * 16 * 8 + (1 << 20)
    assert ln(512, 256 * 80, 64) >= 512 * 256 * 80 * 4
    assert ln(0, 64, 64) == 0


def test_splitk_and_layernorm_reject_missing_workspace(lib):
    vp, i, sz, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_float
    keep, p = _aligned_buffer(1 << 16)
    sk = lib.beam_cutlass_gemmrc_splitk
    sk.argtypes = [vp, vp, vp, i, i, i, i, vp, sz, vp]
    import torch
    if torch.cuda.is_available():
        pytest.skip("device-pointer checks below use host memory as stand-ins")
    assert sk(p, p, p, 64, 64, 4096, -1, p, 1 << 16, None) == 1
    ln = lib.beam_gemmrc_layernorm
    ln.argtypes = [vp, vp, vp, vp, vp, f32, i, i, i, vp, sz, vp]
    assert ln(p, p, p, None, p, 1e-5, 64, 64, 64, p, 1 << 16, None) == 1
    assert ln(p, p, p, p, p, 1e-5, 64, 64, 64, None, 0, None) == 4
    assert ln(p, p, p, p, p, 1e-5, 64, 64, 64, p, 16, None) == 4


def test_cpp_driver_is_built_and_explains_itself(lib):
    """build.py links the C++ timing driver next to the library; without arguments that parse it prints its usage."""
    import subprocess
    exe = os.path.join(os.path.dirname(lib._name), "beam_bench")
    assert os.path.exists(exe)
    r = subprocess.run([exe, "--bogus"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    assert r.returncode == 1 and "usage: beam_bench" in r.stderr
