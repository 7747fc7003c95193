"""GPU parity tests (pytest -m gpu): the sm_100a kernels, called through the C-ABI library, against the CPU
oracle, the golden vectors and size-independent properties.

Tolerance: the reference accepts rtol = atol = 2e-2 against torch.matmul (python/gemm_test.py:46); the bar here
is tighter: max |got - ref| / max(|ref|, 1e-2 * rms(ref)) <= 1e-2 for fp16 outputs (oracle.REL_TOL), which a
correctly rounded result meets at about 5e-4.  Split-K must in addition be bitwise reproducible.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gemmrc_golden.npz")


def _inputs(m, n, k, dist, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    if dist == "uniform":
        a = rng.uniform(-1, 1, (m, k)).astype(np.float16)
        b = rng.uniform(-1, 1, (n, k)).astype(np.float16)
    else:
        a = (rng.standard_normal((m, k), dtype=np.float32) * dist).astype(np.float16)
        b = (rng.standard_normal((n, k), dtype=np.float32) * dist).astype(np.float16)
    return a, b


def _dev(x):
    return torch.from_numpy(x).cuda()


def _healthy(beam):
    st, word = beam.device_status()
    assert (st, word) == (0, 0), "device fault word %#x" % word


@pytest.fixture(scope="module")
def beam(built_library):
    import beam as beam_pkg
    assert os.path.exists(beam_pkg.library_path())
    return beam_pkg


REGISTRY = ["custom_gemmrc_128x128", "custom_gemmrc_128x256", "cutlass_gemmrc"]


@pytest.mark.parametrize("name", REGISTRY)
def test_config1_plumbing_512_cubed(beam, oracle_mod, name):
    """BASELINE config 1: M=N=K=512, uniform [-1,1], checked against the fp32 CPU loop."""
    a, b = _inputs(512, 512, 512, "uniform", 1234 + 1)
    want = oracle_mod.gemmrc(a, b)
    c = torch.zeros(512, 512, dtype=torch.float16, device="cuda")
    getattr(beam, name)(_dev(a), _dev(b), c)
    torch.cuda.synchronize()
    _healthy(beam)
    assert oracle_mod.floored_max_rel(c.cpu().numpy(), want) <= oracle_mod.REL_TOL
    assert oracle_mod.max_abs_over_max(c.cpu().numpy(), want) <= 2e-3


@pytest.mark.parametrize("tb", [[128, 128], [128, 256], [256, 128], [256, 256], [256, 512], [512, 256]])
def test_spec_tile_families(beam, oracle_mod, tb):
    a, b = _inputs(768, 512, 320, "uniform", 21)
    want = oracle_mod.gemmrc(a, b)
    c = torch.zeros(768, 512, dtype=torch.float16, device="cuda")
    beam.cutlass_gemmrc_spec(a=_dev(a), b=_dev(b), c=c, shape_threadblock=tb, shape_warp=[64, 64])
    torch.cuda.synchronize()
    _healthy(beam)
    assert oracle_mod.floored_max_rel(c.cpu().numpy(), want) <= oracle_mod.REL_TOL


def test_two_accumulator_tiles_without_persistence(beam):
    """max_ctas = -1 launches one 256 x 512 (or 512 x 256) tile per CTA pair; the result is the persistent grid's, bit for bit."""
    a, b = _inputs(1100, 1544, 712, 0.1, 4242)
    da, db = _dev(a), _dev(b)
    for kw in (dict(tile_n=512), dict(tile_n=256, tile_m=512)):
        c0 = torch.zeros(1100, 1544, dtype=torch.float16, device="cuda")
        c1 = torch.ones(1100, 1544, dtype=torch.float16, device="cuda")
        beam.gemmrc(da, db, c0, cta_pair=2, **kw)
        beam.gemmrc(da, db, c1, cta_pair=2, max_ctas=-1, **kw)
        torch.cuda.synchronize()
        assert torch.equal(c0, c1), kw
    _healthy(beam)


@pytest.mark.parametrize("case", ["tiny", "ragged", "tile", "wide", "deepk"])
def test_golden_vectors(beam, oracle_mod, case):
    g = np.load(GOLDEN)
    a, b, want = g[case + "_a"], g[case + "_b"], g[case + "_c"]
    for name in REGISTRY:
        c = torch.full(want.shape, 7.0, dtype=torch.float16, device="cuda")
        getattr(beam, name)(_dev(a), _dev(b), c)
        torch.cuda.synchronize()
        assert oracle_mod.floored_max_rel(c.cpu().numpy(), want) <= oracle_mod.REL_TOL, name
        assert oracle_mod.floored_max_rel(c.cpu().numpy(), g[case + "_c64"]) <= oracle_mod.REL_TOL, name
    _healthy(beam)


@pytest.mark.parametrize("m,n,k", [(1, 8, 8), (8, 8, 8), (127, 136, 72), (129, 264, 200), (300, 1000, 1096),
                                    (257, 520, 64), (1000, 24, 4104)])
@pytest.mark.parametrize("tile_n,cta_pair", [(64, 1), (128, 1), (256, 1), (128, 2), (256, 2), (512, 2), (256, -2)])
def test_ragged_shapes(beam, oracle_mod, m, n, k, tile_n, cta_pair):
    """Edge tiles in M, N and K: out-of-range parts are zero-filled on load and masked on store, and nothing
    outside C[M,N] is written."""
    a, b = _inputs(m, n, k, "uniform", m * 31 + n * 7 + k)
    want = oracle_mod.gemmrc(a, b)
    guard = torch.full((m + 2, n), 3.0, dtype=torch.float16, device="cuda")
    c = guard[1:m + 1]
    tile_m = 512 if cta_pair < 0 else 0  # cta_pair -2 stands for the 512 x 256 tile of a CTA pair
    beam.gemmrc(_dev(a), _dev(b), c, tile_n=tile_n, cta_pair=abs(cta_pair), tile_m=tile_m)
    torch.cuda.synchronize()
    assert oracle_mod.floored_max_rel(c.cpu().numpy(), want) <= oracle_mod.REL_TOL
    assert (guard[0] == 3.0).all() and (guard[m + 1] == 3.0).all()
    if tile_n == 128:
        # 128-wide tiles run two tiles in flight by default (an odd tile count leaves a phantom second tile);
        # the one-tile-at-a-time kernel must give the same bits
        c1 = torch.full((m, n), 4.0, dtype=torch.float16, device="cuda")
        beam.gemmrc(_dev(a), _dev(b), c1, tile_n=tile_n, cta_pair=cta_pair, tiles_in_flight=1)
        torch.cuda.synchronize()
        assert torch.equal(c1, c)
    _healthy(beam)


@pytest.mark.parametrize("knobs", [dict(tile_n=256, cta_pair=2), dict(tile_n=512, cta_pair=2), dict(tile_n=128, cta_pair=1),
                                   dict(tile_n=128, cta_pair=2), dict(tile_n=256, cta_pair=1)])
def test_dependent_launches_see_their_predecessors_output(beam, knobs):
    """Every large-GEMM kernel is a programmatic dependent launch: it sets itself up while the kernel before it on the
    stream drains and waits for that kernel's completion before its first load.  A chain in which each GEMM multiplies
    the previous GEMM's output (written with bulk stores that the writing kernel does not wait out) must give the bits
    of the same chain run with a device-wide synchronisation after every launch."""
    torch.manual_seed(5)
    m, n = 1536, 1536
    x0 = (torch.randn(m, n, device="cuda") * 0.05).half()
    ws = [(torch.randn(n, n, device="cuda") * n ** -0.5).half() for _ in range(3)]  # keeps the chain's magnitude

    def chain(sync):
        bufs = [torch.zeros(m, n, dtype=torch.float16, device="cuda") for _ in range(2)]
        src = x0
        for i in range(24):
            dst = bufs[i % 2]
            beam.gemmrc(src, ws[i % 3], dst, **knobs)
            if sync:
                torch.cuda.synchronize()
            src = dst
        torch.cuda.synchronize()
        return src.clone()

    want = chain(True)
    for _ in range(3):
        assert torch.equal(chain(False), want)
    assert torch.isfinite(want.float()).all() and want.float().abs().max() > 0
    _healthy(beam)


def test_cut_tiles_of_the_last_wave(beam, oracle_mod):
    """256 x 256 tiles on CTA pairs: when the last wave of the persistent grid would occupy at most half of the pairs,
    its tiles are computed as 128-column halves on two UMMA chains (even and odd k-blocks summed separately).  A
    4096 x 4096 problem has 256 tiles, three waves of 74 pairs and 34 tiles over: whole and cut tiles in one launch.
    The result must match the oracle, repeat bit for bit, and stay within rounding of the all-whole-tiles result;
    with one k-block, or a ring depth that does not support cutting, the two forms are the same bits."""
    m, n, k = 4096, 4096, 192
    a, b = _inputs(m, n, k, 0.1, 4242)
    da, db = _dev(a), _dev(b)
    want = oracle_mod.gemmrc(a, b)
    cut = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    beam.gemmrc(da, db, cut, tile_n=256, cta_pair=2)
    assert oracle_mod.floored_max_rel(cut.cpu().numpy(), want) <= oracle_mod.REL_TOL
    again = torch.zeros_like(cut)
    beam.gemmrc(da, db, again, tile_n=256, cta_pair=2)
    assert torch.equal(cut, again)
    whole = torch.zeros_like(cut)
    beam.gemmrc(da, db, whole, tile_n=256, cta_pair=2, whole_tiles=True)
    assert oracle_mod.floored_max_rel(whole.cpu().numpy(), want) <= oracle_mod.REL_TOL
    assert oracle_mod.floored_max_rel(cut.cpu().numpy(), whole.cpu().numpy()) <= 2e-3
    odd_ring = torch.zeros_like(cut)
    beam.gemmrc(da, db, odd_ring, tile_n=256, cta_pair=2, stages=5)  # no cutting with an odd ring depth
    assert torch.equal(odd_ring, whole)
    one_kb = torch.zeros(512, 512, dtype=torch.float16, device="cuda")
    one_kb_whole = torch.zeros_like(one_kb)
    beam.gemmrc(da[:512, :64].contiguous(), db[:512, :64].contiguous(), one_kb, tile_n=256, cta_pair=2)
    beam.gemmrc(da[:512, :64].contiguous(), db[:512, :64].contiguous(), one_kb_whole, tile_n=256, cta_pair=2,
                whole_tiles=True)
    assert torch.equal(one_kb, one_kb_whole)
    _healthy(beam)


def test_random_shapes_all_paths(beam, oracle_mod):
    """Seeded sweep of awkward shapes through the large-GEMM tile families, split-K and the fused LayerNorm."""
    rng = np.random.Generator(np.random.PCG64(2024))
    for trial in range(16):
        m = int(rng.integers(1, 700))
        n = int(rng.integers(1, 90)) * 8
        k = int(rng.integers(1, 160)) * 8
        a, b = _inputs(m, n, k, "uniform", 9000 + trial)
        want = oracle_mod.gemmrc(a, b)
        da, db = _dev(a), _dev(b)
        tile_n, cta_pair = [(64, 1), (128, 1), (256, 1), (128, 2), (256, 2), (512, 2)][trial % 6]
        c = torch.full((m, n), -3.0, dtype=torch.float16, device="cuda")
        beam.gemmrc(da, db, c, tile_n=tile_n, cta_pair=cta_pair)
        assert oracle_mod.floored_max_rel(c.cpu().numpy(), want) <= oracle_mod.REL_TOL, (m, n, k, tile_n, cta_pair)
        c.fill_(-3.0)
        beam.cutlass_gemmrc_splitk(da, db, c, split_k_slices=int(rng.integers(0, 6)))
        assert oracle_mod.floored_max_rel(c.cpu().numpy(), want) <= oracle_mod.REL_TOL, ("splitk", m, n, k)
        gamma = (1 + 0.1 * rng.standard_normal(n)).astype(np.float16)
        beta = (0.1 * rng.standard_normal(n)).astype(np.float16)
        if n >= 16:  # LayerNorm over a handful of columns is dominated by fp16 rounding of gamma/beta, not by the kernel
            beam.cutlass_parallel_gemmrc_lnr(da, db, c, _dev(gamma), _dev(beta), 1e-5)
            ln = oracle_mod.gemm_layernorm(a, b, gamma, beta, 1e-5)
            assert oracle_mod.floored_max_rel(c.cpu().numpy(), ln) <= oracle_mod.REL_TOL, ("layernorm", m, n, k)
    _healthy(beam)


def test_two_streams_reentrant(beam, oracle_mod):
    """Calls on different streams do not share state: each gets its own result (device-pointer entry points take the
    caller's stream and keep nothing between calls)."""
    cases = []
    for i in range(4):
        a, b = _inputs(512 + 64 * i, 768, 1024, 0.1, 600 + i)
        cases.append((_dev(a), _dev(b), oracle_mod.gemmrc(a, b),
                      torch.zeros(512 + 64 * i, 768, dtype=torch.float16, device="cuda")))
    streams = [torch.cuda.Stream() for _ in range(2)]
    torch.cuda.synchronize()
    for rep in range(3):
        for i, (da, db, _, c) in enumerate(cases):
            with torch.cuda.stream(streams[i % 2]):
                beam.cutlass_gemmrc(da, db, c)
    torch.cuda.synchronize()
    for _, _, want, c in cases:
        assert oracle_mod.floored_max_rel(c.cpu().numpy(), want) <= oracle_mod.REL_TOL
    _healthy(beam)


def test_zero_and_identity_inputs(beam):
    n = 384
    eye = torch.eye(n, dtype=torch.float16, device="cuda")
    b = ((torch.arange(n * n, device="cuda").reshape(n, n) % 2048) - 1024).half()
    c = torch.empty(n, n, dtype=torch.float16, device="cuda")
    beam.cutlass_gemmrc(eye, b, c)  # I * B^T = B^T exactly
    assert torch.equal(c, b.t())
    beam.cutlass_gemmrc(torch.zeros_like(eye), b, c)
    assert (c == 0).all()


def test_permutation_and_scaling_properties(beam, oracle_mod):
    """Size-independent properties: permuting the rows of A (columns of C come from rows of B) permutes C bit
    for bit, because every output is the same dot product wherever its tile lands (all six tiles of this problem are
    computed the same way); and (2A) B^T equals
    2 (A B^T) to rounding (not bitwise: the tensor cores need not treat subnormal fp16 inputs like normals)."""
    a, b = _inputs(640, 512, 1024, 0.1, 77)
    da, db = _dev(a), _dev(b)
    c1 = torch.empty(640, 512, dtype=torch.float16, device="cuda")
    beam.cutlass_gemmrc(da, db, c1)
    gen = torch.Generator(device="cuda").manual_seed(3)
    pa = torch.randperm(640, device="cuda", generator=gen)
    pb = torch.randperm(512, device="cuda", generator=gen)
    c2 = torch.empty_like(c1)
    beam.cutlass_gemmrc(da[pa].contiguous(), db[pb].contiguous(), c2)
    assert torch.equal(c2, c1[pa][:, pb])
    c3 = torch.empty_like(c1)
    beam.cutlass_gemmrc(da * 2, db, c3)
    assert oracle_mod.floored_max_rel(c3.cpu().numpy(), (c1 * 2).cpu().numpy()) <= 1e-3


def test_config2_8192_cubed(beam, oracle_mod):
    """BASELINE config 2 at full size: every tile family against cuBLAS (fp32 accumulate) on all elements,
    and 24 sampled rows against the fp64 CPU oracle."""
    m = n = k = 8192
    gen = torch.Generator(device="cuda").manual_seed(1234 + 2)
    a = (torch.randn(m, k, device="cuda", generator=gen) * 0.1).half()
    b = (torch.randn(n, k, device="cuda", generator=gen) * 0.1).half()
    ref = torch.matmul(a, b.t())
    rows = np.linspace(0, m - 1, 24).astype(np.int32)
    truth = oracle_mod.gemmrc_rows_f64(a.cpu().numpy(), b.cpu().numpy(), rows)
    rms = float(np.sqrt(np.mean(truth * truth)))
    for tb in ([128, 128], [128, 256], [256, 128], [256, 256], [256, 512]):
        c = torch.zeros(m, n, dtype=torch.float16, device="cuda")
        beam.cutlass_gemmrc_spec(a, b, c, shape_threadblock=tb)
        torch.cuda.synchronize()
        _healthy(beam)
        got_rows = c[torch.from_numpy(rows).long().cuda()].cpu().numpy()
        assert oracle_mod.floored_max_rel(got_rows, truth, rms) <= oracle_mod.REL_TOL, tb
        d = (c.float() - ref.float()).abs()
        den = torch.clamp(ref.float().abs(), min=1e-2 * rms)
        assert float((d / den).max()) <= oracle_mod.REL_TOL, tb


SPLITK_CASES = [
    # m, n, k, tile_n, slices
    (128, 256, 65536, 128, 0), (128, 256, 65536, 128, 4), (128, 256, 65536, 128, 64), (128, 256, 65536, 256, 32),
    (128, 256, 65536, 64, 16), (64, 64, 131072, 64, 0), (64, 64, 131072, 64, 8), (64, 64, 131072, 64, 64),
    (40, 72, 1096, 64, 3), (200, 136, 2048, 128, 5),
    (128, 256, 65536, 64, 64),  # 4 tiles x 64 slices = 256 work items: more than the SMs, so two kernels
]


@pytest.mark.parametrize("m,n,k,tile_n,slices", SPLITK_CASES)
def test_config3_splitk(beam, oracle_mod, m, n, k, tile_n, slices):
    """BASELINE config 3 (both shapes) and ragged cases: parity with the fp32 CPU loop and with the slice-ordered
    restatement, and bitwise identical results on a second run."""
    a, b = _inputs(m, n, k, "uniform", 1234 + 3 + slices)
    want = oracle_mod.gemmrc(a, b)
    da, db = _dev(a), _dev(b)
    c = torch.full((m, n), 5.0, dtype=torch.float16, device="cuda")
    beam.cutlass_gemmrc_splitk_spec(da, db, c, shape_threadblock=[128, tile_n], split_k_slices=slices)
    torch.cuda.synchronize()
    _healthy(beam)
    got = c.cpu().numpy()
    assert oracle_mod.floored_max_rel(got, want) <= oracle_mod.REL_TOL
    if slices > 0:
        assert oracle_mod.floored_max_rel(got, oracle_mod.gemmrc_splitk(a, b, slices)) <= oracle_mod.REL_TOL
    c2 = torch.zeros_like(c)
    beam.cutlass_gemmrc_splitk_spec(da, db, c2, shape_threadblock=[128, tile_n], split_k_slices=slices)
    assert torch.equal(c, c2), "split-K must be bitwise reproducible"
    # A call can run as one cooperative kernel when its (tile, slice) items fit on the device at once (tiles of at
    # most 128 columns, at most 256 partial planes); the library picks that form for folded problems and two kernels
    # otherwise.  Forced either way, the bits must be those of the default: the sum is associated identically.
    plan = beam.splitk_describe(m, n, k, tile_n, slices)
    items = -(-m // 128) * -(-n // plan["tile_n"]) * plan["slices"]
    planes = plan["slices"] * (2 if plan["folded"] else 1)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    can_fuse = items <= sms and plan["tile_n"] <= 128 and planes <= 256
    assert plan["kernels_per_call"] == (1 if can_fuse and plan["folded"] else 2), plan
    assert beam.splitk_describe(m, n, k, tile_n, slices, two_kernels=True)["kernels_per_call"] == 2
    assert beam.splitk_describe(m, n, k, tile_n, slices, two_kernels=False)["kernels_per_call"] == (1 if can_fuse else 2)
    for forced in (True, False):
        c3 = torch.zeros_like(c)
        beam.cutlass_gemmrc_splitk_spec(da, db, c3, shape_threadblock=[128, tile_n], split_k_slices=slices,
                                        two_kernels=forced)
        torch.cuda.synchronize()
        _healthy(beam)
        assert torch.equal(c, c3), "one-kernel and two-kernel split-K must agree bit for bit (two_kernels=%s)" % forced


@pytest.mark.parametrize("m,n,k,tile_n,slices", [(128, 256, 16384, 128, 32), (64, 64, 32768, 64, 0),
                                                 (72, 200, 4096, 64, 7), (512, 512, 4096, 256, 0),
                                                 (520, 264, 2048, 128, 5)])
def test_splitk_exact_on_integer_inputs(beam, oracle_mod, m, n, k, tile_n, slices):
    """With small integer inputs every product and every partial sum is exact in fp32, so the order of the
    additions does not matter and the kernel must reproduce the slice-ordered CPU restatement bit for bit."""
    rng = np.random.Generator(np.random.PCG64(77 + slices))
    a = rng.integers(-2, 3, (m, k)).astype(np.float16)
    b = rng.integers(-2, 3, (n, k)).astype(np.float16)
    s = beam.splitk_describe(m, n, k, tile_n, slices)["slices"]
    want = oracle_mod.gemmrc_splitk(a, b, s)
    assert np.array_equal(want, oracle_mod.gemmrc(a, b))
    c = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    for forced in (None, True, False):
        c.zero_()
        beam.cutlass_gemmrc_splitk_spec(_dev(a), _dev(b), c, shape_threadblock=[128, tile_n], split_k_slices=slices,
                                        two_kernels=forced)
        torch.cuda.synchronize()
        _healthy(beam)
        assert np.array_equal(c.cpu().numpy(), want), forced


def test_splitk_default_entry(beam, oracle_mod):
    a, b = _inputs(128, 256, 8192, "uniform", 99)
    want = oracle_mod.gemmrc(a, b)
    c = torch.zeros(128, 256, dtype=torch.float16, device="cuda")
    for s in (0, 7, 100000):  # heuristic, explicit, out of range (falls back to the heuristic)
        c.zero_()
        beam.cutlass_gemmrc_splitk(a=_dev(a), b=_dev(b), c=c, split_k_slices=s)
        assert oracle_mod.floored_max_rel(c.cpu().numpy(), want) <= oracle_mod.REL_TOL


@pytest.mark.parametrize("m,n,k", [(512, 512, 8192), (1024, 1024, 2048), (520, 264, 4104), (300, 1000, 1096)])
def test_splitk_medium_shapes(beam, oracle_mod, m, n, k):
    """Split-K beyond the small-M-N shapes (512 x 512 x 8192 is the reference's own split-K test call,
    python/gemm_test.py:201): problems with more arithmetic than memory time take the 256-wide tile and a slice per SM,
    and outputs of 64 Ki elements and more are summed by the one-thread-per-four-columns reduction.  Against the
    oracle, and twice for the same bits."""
    a, b = _inputs(m, n, k, "uniform", 7 * m + n + k)
    want = oracle_mod.gemmrc(a, b)
    plan = beam.splitk_describe(m, n, k)
    if m * n >= 200 * (m + n) and n >= 256:
        assert plan["tile_n"] == 256 and plan["slices"] >= 1
    c = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    beam.cutlass_gemmrc_splitk(_dev(a), _dev(b), c)
    assert oracle_mod.floored_max_rel(c.cpu().numpy(), want) <= oracle_mod.REL_TOL
    again = torch.full_like(c, 5.0)
    beam.cutlass_gemmrc_splitk(_dev(a), _dev(b), again)
    assert torch.equal(c, again)
    _healthy(beam)


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (300, 1000, 264), (512, 4096, 512), (96, 264, 320)])
def test_config4_layernorm_small(beam, oracle_mod, m, n, k):
    rng = np.random.Generator(np.random.PCG64(1234 + 4))
    x = (rng.standard_normal((m, k)) * 0.02).astype(np.float16)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float16)
    gamma = (1 + 0.1 * rng.standard_normal(n)).astype(np.float16)
    beta = (0.1 * rng.standard_normal(n)).astype(np.float16)
    want = oracle_mod.gemm_layernorm(x, w, gamma, beta, 1e-5)
    out = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    beam.cutlass_parallel_gemmrc_lnr(_dev(x), _dev(w), out, _dev(gamma), _dev(beta), 1e-5)
    torch.cuda.synchronize()
    _healthy(beam)
    assert oracle_mod.floored_max_rel(out.cpu().numpy(), want) <= oracle_mod.REL_TOL
    out2 = torch.zeros_like(out)
    beam.cutlass_parallel_gemmrc_lnr(_dev(x), _dev(w), out2, _dev(gamma), _dev(beta), 1e-5)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("m,n,k,offset", [(2321, 2056, 200, 0.0), (4100, 1288, 72, 0.0), (2560, 2048, 512, 0.3),
                                          (512, 19208, 64, 0.0)])
def test_layernorm_tmem_resident_and_parked_paths(beam, oracle_mod, m, n, k, offset):
    """Shapes with at least as many 256 x 256 tiles as CTA pairs and no more N tiles than pairs run the kernel that
    keeps tiles in TMEM until their rows' statistics are complete (ragged M, N, K; a row mean several times the row's
    spread -- much larger offsets make the fp32 accumulation order itself visible at this tolerance, for any
    implementation); the last shape has more N tiles than pairs and takes the kernel that parks an fp32 panel."""
    rng = np.random.Generator(np.random.PCG64(77 + m))
    x = (rng.standard_normal((m, k)) * 0.05).astype(np.float16)
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float16)
    if offset:
        x[:, 0] = np.float16(offset)
        w[:, 0] = np.float16(1.0)       # every output gets +offset: mean = 5 x standard deviation
    gamma = (1 + 0.1 * rng.standard_normal(n)).astype(np.float16)
    beta = (0.1 * rng.standard_normal(n)).astype(np.float16)
    want = oracle_mod.gemm_layernorm(x, w, gamma, beta, 1e-5)
    out = torch.full((m, n), 9.0, dtype=torch.float16, device="cuda")
    beam.cutlass_parallel_gemmrc_lnr(_dev(x), _dev(w), out, _dev(gamma), _dev(beta), 1e-5)
    torch.cuda.synchronize()
    _healthy(beam)
    assert oracle_mod.floored_max_rel(out.cpu().numpy(), want) <= oracle_mod.REL_TOL
    out2 = torch.zeros_like(out)
    beam.cutlass_parallel_gemmrc_lnr(_dev(x), _dev(w), out2, _dev(gamma), _dev(beta), 1e-5)
    assert torch.equal(out, out2)


def test_layernorm_on_two_streams_at_once(beam):
    """Two fused GEMM+LayerNorm grids in flight on different streams: the grids wait on their own CTAs, so each must be
    placed as a whole (cooperative launch); results equal the one-stream results and no wait runs out."""
    m, n, k = 4096, 2048, 1024
    gen = torch.Generator(device="cuda").manual_seed(31)
    xs = [(torch.randn(m, k, device="cuda", generator=gen) * 0.05).half() for _ in range(2)]
    w = (torch.randn(n, k, device="cuda", generator=gen) * 0.05).half()
    gamma = (1 + 0.1 * torch.randn(n, device="cuda", generator=gen)).half()
    beta = (0.1 * torch.randn(n, device="cuda", generator=gen)).half()
    want = []
    for x in xs:
        o = torch.empty(m, n, dtype=torch.float16, device="cuda")
        beam.cutlass_parallel_gemmrc_lnr(x, w, o, gamma, beta, 1e-5)
        want.append(o)
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs = [torch.zeros(m, n, dtype=torch.float16, device="cuda") for _ in range(2)]
    for rep in range(10):
        for i, st in enumerate(streams):
            with torch.cuda.stream(st):
                beam.cutlass_parallel_gemmrc_lnr(xs[i], w, outs[i], gamma, beta, 1e-5)
    torch.cuda.synchronize()
    _healthy(beam)
    for i in range(2):
        assert torch.equal(outs[i], want[i])


def test_golden_layernorm(beam, oracle_mod):
    g = np.load(GOLDEN)
    for case in ("ragged", "tile", "wide"):
        a, b = g[case + "_a"], g[case + "_b"]
        out = torch.zeros(a.shape[0], b.shape[0], dtype=torch.float16, device="cuda")
        beam.cutlass_parallel_gemmrc_lnr(_dev(a), _dev(b), out, _dev(g[case + "_gamma"]), _dev(g[case + "_beta"]),
                                         1e-5)
        assert oracle_mod.floored_max_rel(out.cpu().numpy(), g[case + "_ln64"]) <= oracle_mod.REL_TOL, case


def test_config4_layernorm_full_size(beam, oracle_mod):
    """BASELINE config 4: X[16384,4096] x W[4096,4096]^T + LayerNorm; 16 sampled rows against the fp64 oracle,
    and the row statistics of the whole output: mean of (out - beta) / gamma ~ 0 and variance ~ 1."""
    m, n, k = 16384, 4096, 4096
    gen = torch.Generator(device="cuda").manual_seed(1234 + 4)
    x = (torch.randn(m, k, device="cuda", generator=gen) * 0.02).half()
    w = (torch.randn(n, k, device="cuda", generator=gen) * 0.02).half()
    gamma = (1 + 0.1 * torch.randn(n, device="cuda", generator=gen)).half()
    beta = (0.1 * torch.randn(n, device="cuda", generator=gen)).half()
    out = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    beam.cutlass_parallel_gemmrc_lnr(x, w, out, gamma, beta, 1e-5)
    torch.cuda.synchronize()
    _healthy(beam)
    rows = np.linspace(0, m - 1, 16).astype(np.int32)
    truth = oracle_mod.gemm_layernorm_rows_f64(x.cpu().numpy(), w.cpu().numpy(), gamma.cpu().numpy(),
                                               beta.cpu().numpy(), rows, 1e-5)
    got = out[torch.from_numpy(rows).long().cuda()].cpu().numpy()
    assert oracle_mod.floored_max_rel(got, truth) <= oracle_mod.REL_TOL
    z = (out.float() - beta.float()) / gamma.float()
    assert float(z.mean(dim=1).abs().max()) < 5e-3
    assert float((z.var(dim=1, unbiased=False) - 1).abs().max()) < 2e-2


def test_error_paths_on_device(beam):
    a = torch.zeros(64, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        beam.cutlass_gemmrc(a, a[:, :32].contiguous(), a)          # K mismatch
    with pytest.raises(ValueError):
        beam.cutlass_gemmrc(a, a, torch.zeros(64, 32, dtype=torch.float16, device="cuda"))
    with pytest.raises(ValueError):
        beam.cutlass_gemmrc(a.t(), a, a)                            # not contiguous
    with pytest.raises(TypeError):
        beam.cutlass_gemmrc(a.float(), a, a)
    with pytest.raises(ValueError):
        beam.cutlass_gemmrc_spec(a, a, a, shape_threadblock=[64, 64])
    a60 = torch.zeros(64, 60, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        beam.cutlass_gemmrc(a60, a60, a)                            # K % 8 != 0
    lib = ctypes.CDLL(beam.library_path())
    sk = lib.beam_cutlass_gemmrc_splitk
    vp, i = ctypes.c_void_p, ctypes.c_int
    sk.argtypes = [vp, vp, vp, i, i, i, i, vp, ctypes.c_size_t, vp]
    ws = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    big = torch.zeros(64, 4096, dtype=torch.float16, device="cuda")
    assert sk(big.data_ptr(), big.data_ptr(), a.data_ptr(), 64, 64, 4096, 8, ws.data_ptr(), 1024, None) == 4
    assert sk(big.data_ptr(), big.data_ptr(), a.data_ptr(), 64, 64, 4096, 8, None, 0, None) == 4
    _healthy(beam)


def test_host_buffer_entry(beam, oracle_mod):
    a, b = _inputs(1000, 520, 264, 0.1, 5)
    want = oracle_mod.gemmrc(a, b)
    c = torch.zeros(1000, 520, dtype=torch.float16)
    beam.gemmrc_host(torch.from_numpy(a), torch.from_numpy(b), c)
    assert oracle_mod.floored_max_rel(c.numpy(), want) <= oracle_mod.REL_TOL
    pa, pb = torch.from_numpy(a).pin_memory(), torch.from_numpy(b).pin_memory()
    pc = torch.zeros(1000, 520, dtype=torch.float16).pin_memory()
    beam.gemmrc_host(pa, pb, pc)
    assert torch.equal(pc, c)


@pytest.mark.parametrize("m,n,k", [(1000, 520, 264), (2304, 1800, 512), (300, 4104, 128), (4096, 264, 1024)])
def test_host_buffer_entry_strips(beam, oracle_mod, m, n, k):
    """The host entry multiplies strip by strip as row blocks of A and B arrive (several blocks per dimension here,
    ragged last blocks included) and writes each strip into C with a row pitch: every element must be there, and the
    form with B already on the device must give the same bits."""
    a, b = _inputs(m, n, k, 0.1, m + n + k)
    want = oracle_mod.gemmrc(a, b)
    pa, pb = torch.from_numpy(a).pin_memory(), torch.from_numpy(b).pin_memory()
    pc = torch.full((m, n), 9.0, dtype=torch.float16).pin_memory()
    beam.gemmrc_host(pa, pb, pc)
    assert oracle_mod.floored_max_rel(pc.numpy(), want) <= oracle_mod.REL_TOL
    dc = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    beam.gemmrc(pa.cuda(), pb.cuda(), dc, whole_tiles=True)  # the host entry multiplies whole tiles only
    assert torch.equal(dc.cpu(), pc), "host-buffer path and device path must agree bit for bit"
    pc2 = torch.full((m, n), 7.0, dtype=torch.float16).pin_memory()
    beam.gemmrc_host_rows(pa, pb.cuda(), pc2)
    assert torch.equal(pc2, pc)
    _healthy(beam)


def test_reference_kernels_agree_with_oracle_and_ours(beam, oracle_mod):
    """Second parity witness: the reference's own kernels (built unmodified for sm_100a by
    baseline/build_reference.py; skipped when that build is absent) against the CPU oracle and against the new
    kernels on the same seeded inputs."""
    import sys
    ref_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
    if not (os.path.isdir(ref_dir) and any(f.startswith("beam_C") for f in os.listdir(ref_dir))):
        pytest.skip("reference kernels not built")
    sys.path.insert(0, ref_dir)
    import beam_C
    a, b = _inputs(512, 512, 512, "uniform", 1234 + 1)
    want = oracle_mod.gemmrc(a, b)
    da, db = _dev(a), _dev(b)
    ours = torch.zeros(512, 512, dtype=torch.float16, device="cuda")
    beam.cutlass_gemmrc(da, db, ours)
    for name in ("custom_gemmrc_128x128", "custom_gemmrc_128x256", "cutlass_gemmrc"):
        c = torch.zeros(512, 512, dtype=torch.float16, device="cuda")
        getattr(beam_C, name)(da, db, c)
        torch.cuda.synchronize()
        assert oracle_mod.floored_max_rel(c.cpu().numpy(), want) <= oracle_mod.REL_TOL, name
        assert oracle_mod.floored_max_rel(ours.cpu().numpy(), c.cpu().numpy()) <= oracle_mod.REL_TOL, name
    a2, b2 = _inputs(128, 256, 8192, "uniform", 1234 + 3)
    c2 = torch.zeros(128, 256, dtype=torch.float16, device="cuda")
    beam_C.cutlass_gemmrc_splitk(_dev(a2), _dev(b2), c2, 8)
    torch.cuda.synchronize()
    assert oracle_mod.floored_max_rel(c2.cpu().numpy(), oracle_mod.gemmrc(a2, b2)) <= oracle_mod.REL_TOL


def test_overlapped_splitk_calls(beam, oracle_mod):
    """BEAM_FLAG_INPUTS_STABLE: back-to-back calls that are allowed to overlap still give each call's own result."""
    cases = []
    for i in range(6):
        a, b = _inputs(128, 256, 16384, "uniform", 500 + i)
        cases.append((_dev(a), _dev(b), oracle_mod.gemmrc(a, b), torch.zeros(128, 256, dtype=torch.float16, device="cuda")))
    for rep in range(3):
        for da, db, _, c in cases:
            beam.cutlass_gemmrc_splitk(da, db, c, split_k_slices=0, inputs_stable=True)
    torch.cuda.synchronize()
    _healthy(beam)
    for _, _, want, c in cases:
        assert oracle_mod.floored_max_rel(c.cpu().numpy(), want) <= oracle_mod.REL_TOL


def test_one_kernel_splitk_overlapped_and_on_two_streams(beam, oracle_mod):
    """The one-kernel split-K is a cooperative grid launched as a programmatic dependent.  Trains of such calls that
    may overlap (BEAM_FLAG_INPUTS_STABLE), and two trains on two streams at once (each with its own scratch: the
    binding keeps one per stream), must still give every call its own result."""
    cases = []
    for i in range(4):
        a, b = _inputs(64, 64, 32768, "uniform", 700 + i)
        cases.append((_dev(a), _dev(b), oracle_mod.gemmrc(a, b), torch.zeros(64, 64, dtype=torch.float16, device="cuda")))
    for da, db, _, c in cases * 3:
        beam.cutlass_gemmrc_splitk(da, db, c, inputs_stable=True, two_kernels=False)
    torch.cuda.synchronize()
    _healthy(beam)
    for _, _, want, c in cases:
        assert oracle_mod.floored_max_rel(c.cpu().numpy(), want) <= oracle_mod.REL_TOL
        c.zero_()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for rep in range(5):
        for idx, (da, db, _, c) in enumerate(cases):
            with torch.cuda.stream(streams[idx % 2]):
                beam.cutlass_gemmrc_splitk(da, db, c, two_kernels=False)
    torch.cuda.synchronize()
    _healthy(beam)
    for _, _, want, c in cases:
        assert oracle_mod.floored_max_rel(c.cpu().numpy(), want) <= oracle_mod.REL_TOL


@pytest.mark.parametrize("m,n,k,count", [(1024, 1024, 1024, 256 * 1024), (300, 264, 200, 12345), (8192, 4096, 512, 1 << 22),
                                         (128, 128, 64, 0)])
def test_gemm_with_coscheduled_silu(beam, oracle_mod, m, n, k, count):
    """C = A B^T with y = silu(x) worked in by the epilogue warps: both results against CPU references, and against the
    reference's own co-scheduling kernel where that one can run (tile-multiple shapes, built baseline)."""
    a, b = _inputs(m, n, k, 0.1, 4242)
    rng = np.random.Generator(np.random.PCG64(17))
    x = (rng.standard_normal(count) * 2).astype(np.float16)
    da, db, dx = _dev(a), _dev(b), _dev(x) if count else torch.zeros(0, dtype=torch.float16, device="cuda")
    c = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    y = torch.full((count,), 9.0, dtype=torch.float16, device="cuda")
    beam.cutlass_parallel_gemmrc_silu(da, db, c, dx, y)
    torch.cuda.synchronize()
    _healthy(beam)
    assert oracle_mod.floored_max_rel(c.cpu().numpy(), oracle_mod.gemmrc(a, b)) <= oracle_mod.REL_TOL
    if count:
        xf = x.astype(np.float64)
        want = xf / (1.0 + np.exp(-xf))
        assert oracle_mod.floored_max_rel(y.cpu().numpy(), want) <= 2e-3
    ref_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
    if count and m % 128 == 0 and n % 128 == 0 and k % 32 == 0 and count % 1024 == 0 and os.path.isdir(ref_dir) \
            and any(f.startswith("beam_C") for f in os.listdir(ref_dir)):
        import sys
        sys.path.insert(0, ref_dir)
        import beam_C
        c_ref = torch.zeros_like(c)
        y_ref = torch.zeros(count // 1024, 1024, dtype=torch.float16, device="cuda")
        beam_C.cutlass_parallel_gemmrc_lnr(da, db, c_ref, dx.view(count // 1024, 1024), y_ref)
        torch.cuda.synchronize()
        assert oracle_mod.floored_max_rel(c.cpu().numpy(), c_ref.cpu().numpy()) <= oracle_mod.REL_TOL
        assert oracle_mod.floored_max_rel(y.cpu().numpy(), y_ref.view(-1).cpu().numpy()) <= 2e-3


@pytest.mark.parametrize("tile_n,cta_pair", [(128, 1), (256, 2), (512, 2)])
def test_bf16_gemm(beam, tile_n, cta_pair):
    """bf16 operands through the same kernels (descriptor bits + final rounding): against an fp32 matmul of the same
    bf16 values.  Half an ulp of bf16 is 2^-9 = 2e-3, so the fp16 bound of 1e-2 still holds."""
    import oracle
    g = torch.Generator(device="cuda").manual_seed(31)
    a = (torch.randn(520, 1096, device="cuda", generator=g) * 0.1).bfloat16()
    b = (torch.randn(776, 1096, device="cuda", generator=g) * 0.1).bfloat16()
    c = torch.zeros(520, 776, dtype=torch.bfloat16, device="cuda")
    beam.gemmrc(a, b, c, tile_n=tile_n, cta_pair=cta_pair)
    want = (a.float() @ b.float().t())
    assert oracle.floored_max_rel(c.float().cpu().numpy(), want.cpu().numpy()) <= oracle.REL_TOL
    assert torch.equal(c, torch.matmul(a, b.t())) or \
        oracle.floored_max_rel(c.float().cpu().numpy(), torch.matmul(a, b.t()).float().cpu().numpy()) <= 8e-3
    with pytest.raises(TypeError):
        beam.gemmrc(a, b.half(), c)
    with pytest.raises(TypeError):
        beam.cutlass_gemmrc(a, b, c)            # the registry names stay fp16-only, like the reference's


def test_reference_style_driver(beam):
    """The driver with the reference's interface (gemm_test.py): every kernel it lists passes its check."""
    import gemm_test
    r = gemm_test.test_gemm(1024, 1024, 1024, "fp16")
    assert r["verdicts"] == ["success"] * 3 and all(t > 1.0 for t in r["custom"])
    r = gemm_test.test_gemm_splitk(128, 256, 8192, "fp16")
    assert all(v == "success" for v in r["verdicts"])


def test_tuner_picks_a_kernel(beam):
    tuner = beam.OperatorTuner()
    tuner.gemm_ops = tuner.gemm_ops[:5] + tuner.gemm_ops[5:8]   # a short list keeps the test fast
    op, tflops = tuner.tune([2048, 2048, 2048])
    assert op is not None and 1.0 < tflops < 2500.0
    assert tuner.tune([2048, 2048, 2048]) == (op, tflops)


def test_cpp_timing_driver(beam):
    """beam_bench (csrc/bench_main.cc) times registry kernels from C++ through the C ABI with the reference's
    test_pipeline scheme (cuda/cublas.cc:12-40): it must run the kernels it names and report a healthy device."""
    import json
    import subprocess
    exe = os.path.join(os.path.dirname(beam.library_path()), "beam_bench")
    assert os.path.exists(exe), "beam_bench is built next to libbeam_b200.so by build.py"
    for extra in (["--kernel", "cutlass_gemmrc", "--m", "1024", "--n", "1024", "--k", "1024", "--nrep", "3"],
                  ["--kernel", "cutlass_gemmrc_spec", "--tb_m", "256", "--tb_n", "128", "--m", "768", "--n", "520", "--k", "264"],
                  ["--kernel", "cutlass_gemmrc_splitk", "--m", "128", "--n", "256", "--k", "8192", "--nrep", "4"],
                  ["--kernel", "cutlass_gemmrc_splitk", "--m", "64", "--n", "64", "--k", "16384", "--stable", "1", "--sets", "2"]):
        r = subprocess.run([exe] + extra, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
        assert r.returncode == 0, r.stderr
        line = json.loads(r.stdout.strip().splitlines()[-1])
        assert line["device_status"] == 0 and line["fault_word"] == 0 and line["us_per_call"] > 0
    r = subprocess.run([exe, "--kernel", "no_such_kernel", "--m", "64", "--n", "64", "--k", "64"], stdout=subprocess.PIPE,
                       stderr=subprocess.PIPE, text=True, timeout=120)
    assert r.returncode == 3 and "invalid argument" in r.stderr
