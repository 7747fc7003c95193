"""CPU tests of the Python host side: the registry mirrors the reference's names and signatures, calls
without a GPU fail loudly (no fallback), the tuner keeps the reference's interface, and the row-sharding
helpers work across two gloo ranks."""
import inspect
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def test_registry_names_and_signatures():
    import beam
    # python/beam/_C/beam_C.pyi:3-23 in the reference
    expected = {
        "cublas_gemmexrc": ["a", "b", "c"],
        "cublas_hgemmrc": ["a", "b", "c"],
        "custom_gemmrc_128x128": ["a", "b", "c"],
        "custom_gemmrc_128x256": ["a", "b", "c"],
        "cutlass_gemmrc": ["a", "b", "c"],
        "cutlass_gemmrc_spec": ["a", "b", "c", "shape_threadblock", "shape_warp"],
        "cutlass_gemmrc_splitk": ["a", "b", "c", "split_k_slices"],
        "cutlass_gemmrc_splitk_spec": ["a", "b", "c", "shape_threadblock", "shape_warp", "split_k_slices"],
    }
    for name, params in expected.items():
        fn = getattr(beam, name)
        got = inspect.signature(fn).parameters
        # the reference's parameters come first and in order; anything after them is additive and optional
        assert list(got)[:len(params)] == params, name
        for extra in list(got)[len(params):]:
            assert got[extra].default is not inspect.Parameter.empty, (name, extra)
    sig = inspect.signature(beam.cutlass_gemmrc_spec)
    assert sig.parameters["shape_threadblock"].default == [128, 128]
    assert sig.parameters["shape_warp"].default == [64, 64]
    assert inspect.signature(beam.cutlass_gemmrc_splitk).parameters["split_k_slices"].default == 0
    assert len(inspect.signature(beam.cutlass_parallel_gemmrc_lnr).parameters) >= 5
    assert hasattr(beam, "Operator") and hasattr(beam, "OperatorTuner")


def test_no_cpu_fallback(built_library):
    import beam
    a = torch.zeros(64, 64, dtype=torch.float16)
    b = torch.zeros(64, 64, dtype=torch.float16)
    c = torch.zeros(64, 64, dtype=torch.float16)
    for fn in (beam.cutlass_gemmrc, beam.custom_gemmrc_128x128, beam.custom_gemmrc_128x256,
               beam.cutlass_gemmrc_splitk, beam.cutlass_gemmrc_spec, beam.cutlass_gemmrc_splitk_spec):
        with pytest.raises(ValueError, match="CUDA tensor"):
            fn(a, b, c)
    with pytest.raises(ValueError):
        beam.cutlass_parallel_gemmrc_lnr(a, b, c, torch.zeros(64, dtype=torch.float16),
                                         torch.zeros(64, dtype=torch.float16))
    if not torch.cuda.is_available():
        # the host-buffer entry needs a device too: it must say so, not compute on the CPU
        with pytest.raises(beam.BeamError):
            beam.gemmrc_host(a, b, c)
    assert (c == 0).all()


def test_shape_and_dtype_checks():
    from beam import _C
    a = torch.zeros(8, 16, dtype=torch.float16)
    with pytest.raises(TypeError):
        _C._check_abc(a.float(), a, a)
    with pytest.raises(TypeError):
        _C._check_abc("a", a, a)


def test_operator_and_tuner_interface():
    from functools import partial
    import beam
    calls = []

    def fake(a, b, c):
        calls.append((a.shape, b.shape, c.shape))

    op = beam.Operator(fake)
    assert str(op) == "fake"
    assert "tile_n=256" in str(beam.Operator(partial(beam.gemmrc, tile_n=256)))

    def broken(a, b, c):
        raise ValueError("unsupported")

    t = torch.zeros(2, 2)
    # check_callable synchronises the device after the call; without one it must still report failures
    assert beam.Operator(broken).check_callable(t, t, t) is False
    tuner = beam.OperatorTuner()
    assert tuner.get_hash("gemm", [1, 2, 3]) == "gemm(1,2,3,)"          # reference: tuner.py:109-114
    names = [str(o) for o in tuner.gemm_ops]
    for required in ("cublas_gemmexrc", "cutlass_gemmrc", "cutlass_gemmrc_splitk", "custom_gemmrc_128x128",
                     "custom_gemmrc_128x256"):
        assert required in names
    splits = {o.func.keywords["split_k_slices"] for o in tuner.gemm_ops
              if hasattr(o.func, "keywords") and "split_k_slices" in o.func.keywords}
    assert {4, 8, 16, 32, 64} <= splits                                  # the stated split-factor search space
    tuner.cache["gemm(4,4,4,)"] = ("op", 1.0)
    assert tuner.tune([4, 4, 4]) == ("op", 1.0)                          # cache hit needs no GPU


def test_driver_check_verdicts():
    """gemm_test.check keeps the reference's rule: rtol = atol = 2e-2, fewer than 0.12 % mismatches only warn."""
    import gemm_test
    want = torch.ones(100, 100, dtype=torch.float16)
    got = want.clone()
    assert gemm_test.check(lambda: None, [want], [got]) == "success"
    got[0, 0] = 2.0                                   # 1 of 10000 = 0.01 %
    assert gemm_test.check(lambda: None, [want], [got]) == "warning"
    got[:1, :20] = 2.0                                # 0.2 %
    assert gemm_test.check(lambda: None, [want], [got]) == "failure"
    got = want + 0.03                                 # inside atol + rtol * |c| = 0.04
    assert gemm_test.check(lambda: None, [want], [got]) == "success"


def test_tuner_cache_persistence(tmp_path):
    import beam
    path = str(tmp_path / "tuned.json")
    t1 = beam.OperatorTuner()
    op = t1.gemm_ops[3]
    t1.cache["gemm(8192,8192,8192,)"] = (op, 1234.5)
    t1.cache["gemm(64,64,131072,)"] = (t1.gemm_ops[-1], 7.25)
    t1.save(path)
    t1.save(path)  # idempotent, keeps the file valid
    t2 = beam.OperatorTuner()
    assert t2.load(path) == 2
    got_op, got_tf = t2.tune([8192, 8192, 8192])          # served from the loaded cache, no GPU needed
    assert str(got_op) == str(op) and got_tf == 1234.5
    assert str(t2.cache["gemm(64,64,131072,)"][0]) == str(t1.gemm_ops[-1])
    assert beam.OperatorTuner().load(str(tmp_path / "missing.json")) == 0


def test_row_block_partition():
    from beam.sharded import row_block
    for m, world in ((65536, 8), (65536, 4), (10, 4), (3, 8), (0, 2), (8192, 1)):
        blocks = [row_block(m, world, r) for r in range(world)]
        assert blocks[0][0] == 0 and blocks[-1][1] == m
        for (s0, e0), (s1, e1) in zip(blocks, blocks[1:]):
            assert e0 == s1 and e0 >= s0
        sizes = [e - s for s, e in blocks]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        row_block(8, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _gloo_worker(rank, world, port, m, ragged_m, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(here, "general-nvgpu-testing_b200"))
    from beam.sharded import all_gather_rows, row_block, sharded_gemmrc
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        for mm in (m, ragged_m):
            g = torch.Generator().manual_seed(5)
            a = torch.randn(mm, 32, generator=g).half()
            b = torch.randn(24, 32, generator=g).half()
            s, e = row_block(mm, world, rank)
            c_local = torch.empty(e - s, 24, dtype=torch.float16)
            # the CUDA kernel is stood in for by an fp32 matmul: this test covers the sharding, not the kernel
            sharded_gemmrc(a[s:e], b, c_local, kernel=lambda x, y, z: z.copy_((x.float() @ y.float().t()).half()))
            full = all_gather_rows(c_local, mm)
            want = (a.float() @ b.float().t()).half()
            assert torch.equal(full, want), "rank %d m=%d" % (rank, mm)
        open(os.path.join(result_dir, "ok%d" % rank), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_row_sharded_gemm_two_gloo_ranks(tmp_path):
    world = 2
    mp.spawn(_gloo_worker, args=(world, _free_port(), 64, 37, str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]


def test_b_shards_cover_b_exactly():
    """ShardedHostGemm uploads disjoint, equal shards of B that together are all of B; uneven splits are refused."""
    from beam.sharded import b_shard_rows
    for n, world in ((8192, 8), (1024, 2), (520, 1), (4096, 4)):
        spans = [b_shard_rows(n, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
        assert len({e - s for s, e in spans}) == 1
    with pytest.raises(ValueError):
        b_shard_rows(1000, 3, 0)
    with pytest.raises(ValueError):
        b_shard_rows(1024, 2, 2)


def test_numa_binding_is_harmless_without_a_gpu():
    """bind_to_gpu_numa_node only ever narrows this process's own CPU affinity and reports False when it cannot ask
    NVML (no driver in this container): the affinity must be unchanged then."""
    from beam.sharded import bind_to_gpu_numa_node
    before = os.sched_getaffinity(0)
    ok = bind_to_gpu_numa_node(0)
    after = os.sched_getaffinity(0)
    assert after <= before and (ok or after == before)
    os.sched_setaffinity(0, before)
