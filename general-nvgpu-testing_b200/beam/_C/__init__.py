"""`beam._C` — the kernel registry of BEAM, bound to the B200 C-ABI library.

The reference builds a pybind11 module `beam_C` whose functions take torch tensors
(cuda/main.cc:51-60; signatures in python/beam/_C/beam_C.pyi:3-23) and re-exports it from
python/beam/_C/__init__.py.  Here the same names, argument names, defaults and in-place `c` are kept,
but each function is a thin ctypes call into libbeam_b200.so: tensors are checked, reduced to raw device
pointers and sizes, and launched on torch's current CUDA stream.  Errors become Python exceptions
(the reference exits the process or silently does nothing), which is what `Operator.check_callable`
needs to reject a candidate.

There is no CPU path: importing works anywhere (so the API can be inspected), but every kernel call
raises unless libbeam_b200.so is built and the tensors live on an sm_100 device.
"""
import ctypes
import os

import torch

__all__ = [
    "cublas_gemmexrc",
    "cublas_hgemmrc",
    "cutlass_gemmrc",
    "cutlass_gemmrc_spec",
    "cutlass_gemmrc_splitk",
    "cutlass_gemmrc_splitk_spec",
    "custom_gemmrc_128x128",
    "custom_gemmrc_128x256",
    "cutlass_parallel_gemmrc_lnr",
    "cutlass_parallel_gemmrc_silu",
    "gemmrc",
    "gemmrc_host",
    "gemmrc_host_rows",
    "gemmrc_allgather",
    "splitk_describe",
    "release_workspaces",
    "BeamError",
    "library_path",
]

_PKG = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
_LIB_PATH = os.path.join(_PKG, "libbeam_b200.so")
_lib = None

BEAM_OK = 0
_VALUE_ERRORS = (1, 2, 3, 4)  # invalid argument, unsupported, alignment, workspace


class BeamError(RuntimeError):
    """A kernel could not be launched or reported a device fault."""


class beam_gemm_cfg(ctypes.Structure):
    _fields_ = [
        ("tile_n", ctypes.c_int),
        ("cta_pair", ctypes.c_int),
        ("stages", ctypes.c_int),
        ("group_m", ctypes.c_int),
        ("split_k_slices", ctypes.c_int),
        ("max_ctas", ctypes.c_int),
        ("l2_hints", ctypes.c_int),
        ("flags", ctypes.c_int),
        ("tile_m", ctypes.c_int),
        ("tiles_in_flight", ctypes.c_int),
    ]


def library_path():
    return _LIB_PATH


def _load():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise BeamError(
            "libbeam_b200.so is not built (%s); run `python %s` — there is no fallback path"
            % (_LIB_PATH, os.path.join(_PKG, "build.py")))
    L = ctypes.CDLL(_LIB_PATH)
    vp, i, f, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
    L.beam_status_string.restype = ctypes.c_char_p
    L.beam_status_string.argtypes = [i]
    L.beam_last_cuda_error.restype = ctypes.c_char_p
    L.beam_version.restype = ctypes.c_char_p
    L.beam_device_status.argtypes = [i, ctypes.POINTER(i)]
    L.beam_gemmrc_fp16.argtypes = [vp, vp, vp, i, i, i, ctypes.POINTER(beam_gemm_cfg), vp]
    for name in ("beam_custom_gemmrc_128x128", "beam_custom_gemmrc_128x256", "beam_cutlass_gemmrc"):
        getattr(L, name).argtypes = [vp, vp, vp, i, i, i, vp]
    L.beam_cutlass_gemmrc_spec.argtypes = [vp, vp, vp, i, i, i, i, i, i, i, vp]
    L.beam_gemmrc_splitk_workspace_bytes.restype = sz
    L.beam_gemmrc_splitk_workspace_bytes.argtypes = [i, i, i, i, i]
    L.beam_gemmrc_splitk_heuristic.argtypes = [i, i, i, i]
    L.beam_gemmrc_splitk_describe.argtypes = [i, i, i, i, i, i, ctypes.POINTER(i)]
    L.beam_cutlass_gemmrc_splitk.argtypes = [vp, vp, vp, i, i, i, i, vp, sz, vp]
    L.beam_gemmrc_splitk_fp16.argtypes = [vp, vp, vp, i, i, i, ctypes.POINTER(beam_gemm_cfg), vp, sz, vp]
    L.beam_cutlass_gemmrc_splitk_spec.argtypes = [vp, vp, vp, i, i, i, i, i, i, i, i, vp, sz, vp]
    L.beam_gemmrc_layernorm_workspace_bytes.restype = sz
    L.beam_gemmrc_layernorm_workspace_bytes.argtypes = [i, i, i]
    L.beam_gemmrc_layernorm.argtypes = [vp, vp, vp, vp, vp, f, i, i, i, vp, sz, vp]
    L.beam_gemmrc_fp16_host.argtypes = [vp, vp, vp, i, i, i]
    L.beam_gemmrc_fp16_host_rows.argtypes = [vp, vp, vp, i, i, i]
    L.beam_gemmrc_silu.argtypes = [vp, vp, vp, i, i, i, vp, vp, ctypes.c_longlong, vp]
    L.beam_gemmrc_fp16_allgather.argtypes = [vp, vp, ctypes.POINTER(vp), i, i, i, i, i, ctypes.POINTER(beam_gemm_cfg), vp]
    _lib = L
    return L


def _raise(status, what):
    L = _load()
    msg = "%s: %s" % (what, L.beam_status_string(status).decode())
    if status in (5, 6, 8):
        detail = L.beam_last_cuda_error().decode()
        if detail:
            msg += " [%s]" % detail
    if status in _VALUE_ERRORS:
        raise ValueError(msg)
    raise BeamError(msg)


def _check_abc(a, b, c, allow_bf16=False):
    """Same preconditions as the reference's checkTensor / checkIntEqual / fp16 dispatch
    (cuda/include/torch_utils.h:7-47, cuda/cutlass_kernels/main.cc:25-45), reported as exceptions."""
    for name, t in (("a", a), ("b", b), ("c", c)):
        if not isinstance(t, torch.Tensor):
            raise TypeError("%s must be a torch.Tensor" % name)
        if t.dtype != torch.float16 and not (allow_bf16 and t.dtype == torch.bfloat16 and t.dtype == a.dtype):
            raise TypeError("%s must be float16, got %s" % (name, t.dtype))
        if not t.is_cuda:
            raise ValueError("%s must be a CUDA tensor (there is no CPU path)" % name)
        if not t.is_contiguous():
            raise ValueError("%s must be contiguous" % name)
        if t.dim() != 2:
            raise ValueError("%s must be 2-D" % name)
    if not (a.device == b.device == c.device):
        raise ValueError("a, b, c must be on the same device")
    m, k = a.shape
    n, kb = b.shape
    if k != kb:
        raise ValueError("a is [M,K]=%s but b is [N,K]=%s" % (tuple(a.shape), tuple(b.shape)))
    if tuple(c.shape) != (m, n):
        raise ValueError("c must be [M,N]=(%d,%d), got %s" % (m, n, tuple(c.shape)))
    return int(m), int(n), int(k)


def _stream(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


_workspaces = {}


def _workspace(device, nbytes):
    """Grow-only scratch tensor per device and stream, owned by the binding (the reference hides a cudaMalloc'd
    buffer inside the extension instead: cutlass_gemmrc_splitk.cu:31-42).  Per stream, because calls on different
    streams may run at the same time and must not share partial sums or statistics."""
    key = (device.type, device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(int(nbytes), 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def release_workspaces():
    """Drops the scratch tensors the binding keeps per device and stream (they are grow-only otherwise).  The
    caller makes sure that no split-K or LayerNorm call is still running."""
    _workspaces.clear()


def _run(fn_name, a, b, c, *extra):
    m, n, k = _check_abc(a, b, c)
    L = _load()
    with torch.cuda.device(a.device):
        st = getattr(L, fn_name)(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, *extra, _stream(a))
    if st != BEAM_OK:
        _raise(st, fn_name)


def custom_gemmrc_128x128(a, b, c):
    """c[M,N] = a[M,K] @ b[N,K].T with 128x128 tiles (registry slot of cute_gemm_128x128.cu)."""
    _run("beam_custom_gemmrc_128x128", a, b, c)


def custom_gemmrc_128x256(a, b, c):
    """c = a @ b.T with 128x256 tiles (registry slot of cute_gemm_128x256.cu)."""
    _run("beam_custom_gemmrc_128x256", a, b, c)


def cutlass_gemmrc(a, b, c):
    """c = a @ b.T, library default: 256x256 tile on a CTA pair (slot of cutlass_gemmrc.cu:21-40)."""
    _run("beam_cutlass_gemmrc", a, b, c)


def _pair(v, name):
    v = list(v)
    if len(v) != 2:
        raise ValueError("%s must have two entries" % name)
    return int(v[0]), int(v[1])


def cutlass_gemmrc_spec(a, b, c, shape_threadblock=[128, 128], shape_warp=[64, 64]):
    """c = a @ b.T with the tile family named by shape_threadblock: [128,128], [128,256] (one CTA per
    tile) or [256,128], [256,256] (CTA pair).  shape_warp is kept for signature compatibility
    (cuda/cutlass_kernels/main.cc:129-132) and ignored."""
    tbm, tbn = _pair(shape_threadblock, "shape_threadblock")
    wm, wn = _pair(shape_warp, "shape_warp")
    _run("beam_cutlass_gemmrc_spec", a, b, c, tbm, tbn, wm, wn)


def gemmrc(a, b, c, tile_n=0, cta_pair=0, stages=0, group_m=0, max_ctas=0, l2_hints=0, tile_m=0, tiles_in_flight=0,
           whole_tiles=False):
    """c = a @ b.T with explicit Blackwell knobs (0 = default); what the tuner searches over.  The three tensors may
    be bfloat16 instead of float16 (all three alike).  whole_tiles=True keeps the last wave's 256 x 256 tiles whole
    instead of cutting them into 128-column halves (a cut tile sums K in a different, equally fixed order)."""
    m, n, k = _check_abc(a, b, c, allow_bf16=True)
    if not (a.dtype == b.dtype == c.dtype):
        raise TypeError("a, b, c must share one dtype")
    flags = (2 if a.dtype == torch.bfloat16 else 0) | (FLAG_WHOLE_TILES if whole_tiles else 0)
    cfg = beam_gemm_cfg(int(tile_n), int(cta_pair), int(stages), int(group_m), 0, int(max_ctas), int(l2_hints), flags,
                        int(tile_m), int(tiles_in_flight))
    L = _load()
    with torch.cuda.device(a.device):
        st = L.beam_gemmrc_fp16(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, ctypes.byref(cfg), _stream(a))
    if st != BEAM_OK:
        _raise(st, "beam_gemmrc_fp16")


FLAG_INPUTS_STABLE = 1
FLAG_SPLITK_TWO_KERNELS = 4
FLAG_SPLITK_ONE_KERNEL = 8
FLAG_WHOLE_TILES = 16


def _splitk_flags(inputs_stable, two_kernels):
    """two_kernels: None = the library decides, True = partials + reduction kernels, False = one kernel where it applies."""
    flags = FLAG_INPUTS_STABLE if inputs_stable else 0
    if two_kernels is True:
        flags |= FLAG_SPLITK_TWO_KERNELS
    elif two_kernels is False:
        flags |= FLAG_SPLITK_ONE_KERNEL
    return flags


def splitk_describe(m, n, k, tile_n=0, split_k_slices=0, inputs_stable=False, two_kernels=None):
    """How a split-K call with these arguments runs on the current device: a dict with the tile N, the number of K
    slices, whether the problem runs folded, the kernels per call (1 or 2) and whether the first kernel is a
    programmatic dependent launch."""
    info = (ctypes.c_int * 5)()
    flags = _splitk_flags(inputs_stable, two_kernels)
    st = _load().beam_gemmrc_splitk_describe(int(m), int(n), int(k), int(tile_n), int(split_k_slices), flags, info)
    if st != BEAM_OK:
        _raise(st, "beam_gemmrc_splitk_describe")
    return {"tile_n": info[0], "slices": info[1], "folded": bool(info[2]), "kernels_per_call": info[3],
            "programmatic_dependent_launch": bool(info[4])}


def _splitk(a, b, c, tile_n, split_k_slices, inputs_stable, two_kernels=None):
    m, n, k = _check_abc(a, b, c)
    L = _load()
    flags = _splitk_flags(inputs_stable, two_kernels)
    cfg = beam_gemm_cfg(int(tile_n), 0, 0, 0, int(split_k_slices), 0, 0, flags)
    with torch.cuda.device(a.device):
        nbytes = L.beam_gemmrc_splitk_workspace_bytes(m, n, k, int(tile_n), int(split_k_slices))
        if nbytes > (4 << 30):
            raise ValueError("split-K scratch of %d bytes: split-K is meant for small M*N" % nbytes)
        ws = _workspace(a.device, nbytes)
        st = L.beam_gemmrc_splitk_fp16(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, ctypes.byref(cfg),
                                       ws.data_ptr(), ws.numel(), _stream(a))
    if st != BEAM_OK:
        _raise(st, "beam_gemmrc_splitk_fp16")


def cutlass_gemmrc_splitk(a, b, c, split_k_slices=0, inputs_stable=False, two_kernels=None):
    """Split-K c = a @ b.T for small M, N and huge K; fp32 partials summed in a fixed order (bitwise
    reproducible).  split_k_slices = 0 lets the library choose (slot of cutlass_gemmrc_splitk.cu:59-105).
    inputs_stable=True promises that a and b are not outputs of the kernel just before this call on the
    stream, which lets back-to-back calls overlap (BEAM_FLAG_INPUTS_STABLE).  two_kernels=True forces the
    partials-then-reduction pair of kernels where the library would run the call as one kernel, False the one-kernel
    form where the library would launch two (same bits either way); None leaves the choice to the library."""
    _splitk(a, b, c, 0, split_k_slices, inputs_stable, two_kernels)


def cutlass_gemmrc_splitk_spec(a, b, c, shape_threadblock=[128, 128], shape_warp=[64, 64], split_k_slices=0,
                               inputs_stable=False, two_kernels=None):
    """Split-K with the tile's N taken from shape_threadblock[1] (64, 128 or 256); shape_warp is accepted for
    signature compatibility (cuda/cutlass_kernels/main.cc:137-141) and ignored."""
    tbm, tbn = _pair(shape_threadblock, "shape_threadblock")
    _pair(shape_warp, "shape_warp")
    if tbn not in (64, 128, 256):
        raise ValueError("shape_threadblock[1] must be 64, 128 or 256")
    _splitk(a, b, c, tbn, split_k_slices, inputs_stable, two_kernels)


def cutlass_parallel_gemmrc_lnr(a, b, c, gamma, beta, eps=1e-5):
    """Fused GEMM + LayerNorm: c[M,N] = LayerNorm_rows(a[M,K] @ b[N,K].T) * gamma[N] + beta[N].

    Keeps the reference's registry slot and five-tensor arity (cuda/cute_kernels/main.cc:55-76,87), but
    the last two tensors are LayerNorm's gamma and beta rather than the input/output of the unrelated
    SiLU that the reference kernel runs beside its GEMM (cute_gemm_ln.cu:127-198)."""
    m, n, k = _check_abc(a, b, c)
    for name, t in (("gamma", gamma), ("beta", beta)):
        if not (isinstance(t, torch.Tensor) and t.is_cuda and t.is_contiguous() and t.dtype == torch.float16):
            raise TypeError("%s must be a contiguous CUDA float16 tensor" % name)
        if t.numel() != n:
            raise ValueError("%s must have N=%d elements" % (name, n))
    L = _load()
    with torch.cuda.device(a.device):
        nbytes = L.beam_gemmrc_layernorm_workspace_bytes(m, n, k)
        ws = _workspace(a.device, nbytes)
        st = L.beam_gemmrc_layernorm(a.data_ptr(), b.data_ptr(), c.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
                                     float(eps), m, n, k, ws.data_ptr(), ws.numel(), _stream(a))
    if st != BEAM_OK:
        _raise(st, "beam_gemmrc_layernorm")


def cutlass_parallel_gemmrc_silu(a, b, c, x, y):
    """c = a @ b.T and, in the same kernel, y = silu(x) element-wise over a second fp16 tensor: the semantics of the
    reference kernel registered as `cutlass_parallel_gemmrc_lnr` (cuda/cute_kernels/main.cc:55-76, cute_gemm_ln.cu),
    which co-schedules a memory-bound element-wise op with a compute-bound GEMM."""
    m, n, k = _check_abc(a, b, c)
    for name, t in (("x", x), ("y", y)):
        if not (isinstance(t, torch.Tensor) and t.is_cuda and t.is_contiguous() and t.dtype == torch.float16):
            raise TypeError("%s must be a contiguous CUDA float16 tensor" % name)
    if x.numel() != y.numel():
        raise ValueError("x and y must have the same number of elements")
    L = _load()
    with torch.cuda.device(a.device):
        st = L.beam_gemmrc_silu(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, x.data_ptr(), y.data_ptr(),
                                x.numel(), _stream(a))
    if st != BEAM_OK:
        _raise(st, "beam_gemmrc_silu")


def gemmrc_allgather(a_local, b, gathered_ptrs, rank, n, tile_n=0, cta_pair=0, stages=0, group_m=0):
    """Fused row-sharded GEMM + all-gather: this rank's a_local[M_local,K] @ b[N,K].T is written into row block `rank`
    of every rank's gathered C[world * M_local, N]; gathered_ptrs[d] is rank d's buffer as a device pointer valid in
    this process (see beam.sharded.GatheredC).  Asynchronous; complete once all ranks' kernels have finished."""
    for name, t in (("a_local", a_local), ("b", b)):
        if not (isinstance(t, torch.Tensor) and t.is_cuda and t.is_contiguous() and t.dtype == torch.float16
                and t.dim() == 2):
            raise TypeError("%s must be a contiguous 2-D CUDA float16 tensor" % name)
    m, k = a_local.shape
    if b.shape != (n, k):
        raise ValueError("b must be [N,K]=(%d,%d), got %s" % (n, k, tuple(b.shape)))
    world = len(gathered_ptrs)
    arr = (ctypes.c_void_p * world)(*[ctypes.c_void_p(int(x)) for x in gathered_ptrs])
    cfg = None
    if tile_n or cta_pair or stages or group_m:
        cfg = ctypes.byref(beam_gemm_cfg(int(tile_n), int(cta_pair), int(stages), int(group_m)))
    L = _load()
    with torch.cuda.device(a_local.device):
        st = L.beam_gemmrc_fp16_allgather(a_local.data_ptr(), b.data_ptr(), arr, world, int(rank), int(m), int(n), int(k),
                                          cfg, _stream(a_local))
    if st != BEAM_OK:
        _raise(st, "beam_gemmrc_fp16_allgather")


def gemmrc_host(a, b, c):
    """a, b, c are CPU float16 tensors (ideally pinned): copies in, multiplies on the current CUDA device,
    copies c back; returns when c is complete."""
    for name, t in (("a", a), ("b", b), ("c", c)):
        if not (isinstance(t, torch.Tensor) and not t.is_cuda and t.is_contiguous() and t.dtype == torch.float16):
            raise TypeError("%s must be a contiguous CPU float16 tensor" % name)
    m, k = a.shape
    n, kb = b.shape
    if k != kb or tuple(c.shape) != (m, n):
        raise ValueError("shape mismatch")
    st = _load().beam_gemmrc_fp16_host(a.data_ptr(), b.data_ptr(), c.data_ptr(), int(m), int(n), int(k))
    if st != BEAM_OK:
        _raise(st, "beam_gemmrc_fp16_host")


def gemmrc_host_rows(a, b_dev, c):
    """a and c are CPU float16 tensors (ideally pinned), b_dev is a CUDA float16 tensor [N,K] on the current device:
    copies a in, multiplies, copies c back; returns when c is complete.  What a rank of a row-sharded job calls
    once B is on its GPU (see beam.sharded.ShardedHostGemm)."""
    for name, t in (("a", a), ("c", c)):
        if not (isinstance(t, torch.Tensor) and not t.is_cuda and t.is_contiguous() and t.dtype == torch.float16):
            raise TypeError("%s must be a contiguous CPU float16 tensor" % name)
    if not (isinstance(b_dev, torch.Tensor) and b_dev.is_cuda and b_dev.is_contiguous() and b_dev.dtype == torch.float16
            and b_dev.dim() == 2):
        raise TypeError("b_dev must be a contiguous 2-D CUDA float16 tensor")
    m, k = a.shape
    n, kb = b_dev.shape
    if k != kb or tuple(c.shape) != (m, n):
        raise ValueError("shape mismatch")
    with torch.cuda.device(b_dev.device):
        torch.cuda.current_stream().synchronize()  # b_dev must be complete: the entry works on its own streams
        st = _load().beam_gemmrc_fp16_host_rows(a.data_ptr(), b_dev.data_ptr(), c.data_ptr(), int(m), int(n), int(k))
    if st != BEAM_OK:
        _raise(st, "beam_gemmrc_fp16_host_rows")


def device_status(clear=False):
    """(status, fault_word) of the current device; synchronises it."""
    word = ctypes.c_int(0)
    st = _load().beam_device_status(1 if clear else 0, ctypes.byref(word))
    return st, word.value


# ---- cuBLAS comparators (baselines only; kept because the tuner and the driver list them) ---------
def cublas_gemmexrc(a, b, c):
    """cuBLAS GemmEx with fp32 compute via torch (reference: cuda/cublas.cc:93-122). Comparison baseline."""
    _check_abc(a, b, c)
    torch.matmul(a, b.t(), out=c)


def cublas_hgemmrc(a, b, c):
    """cuBLAS Hgemm slot (reference: cuda/cublas.cc:44-71, fp16 compute type).  Comparison baseline: torch's
    fp16 matmul with fp16 accumulation switched on for the duration of the call
    (torch.backends.cuda.matmul.allow_fp16_accumulation), which is what selects cuBLAS's fp16-compute kernels.
    On a torch build without that switch this is the same call as cublas_gemmexrc."""
    _check_abc(a, b, c)
    mm = torch.backends.cuda.matmul
    if not hasattr(mm, "allow_fp16_accumulation"):
        torch.matmul(a, b.t(), out=c)
        return
    saved = mm.allow_fp16_accumulation
    mm.allow_fp16_accumulation = True
    try:
        torch.matmul(a, b.t(), out=c)
    finally:
        mm.allow_fp16_accumulation = saved
