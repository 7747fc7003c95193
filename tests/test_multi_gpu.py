"""Two-GPU test of the fused GEMM + all-gather and of the row-sharded GEMM + LayerNorm (pytest -m gpu on a box with at least two GPUs; skipped otherwise).
Each rank multiplies its row block and the kernel's epilogue stores every tile into both ranks' gathered buffers
through peer-mapped (symmetric) memory; the result must equal the plain sharded GEMM followed by an NCCL all-gather
and, on the small shapes, the CPU oracle's GEMM of every rank's rows."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(here, "general-nvgpu-testing_b200"))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import numpy as np
        sys.path.insert(0, here)
        import oracle  # the CPU checker (built by the parent process before the ranks start)
        import beam
        from beam.sharded import GatheredC, all_gather_rows, gemmrc_allgather
        for (m_local, n, k, knobs) in ((512, 1024, 512, {}), (300, 776, 264, {"tile_n": 256, "cta_pair": 2}),
                                       (2048, 4096, 1024, {"tile_n": 512, "cta_pair": 2})):
            g = torch.Generator(device="cuda").manual_seed(100 + rank)
            a = (torch.randn(m_local, k, device="cuda", generator=g) * 0.1).half()
            gb = torch.Generator(device="cuda").manual_seed(7)
            b = (torch.randn(n, k, device="cuda", generator=gb) * 0.1).half()
            c_local = torch.empty(m_local, n, dtype=torch.float16, device="cuda")
            beam.gemmrc(a, b, c_local, **knobs)
            want = all_gather_rows(c_local, m_local * world)
            gathered = GatheredC(m_local, n)
            gathered.tensor.fill_(3.0)
            got = gemmrc_allgather(a, b, gathered, **knobs)
            torch.cuda.synchronize()
            assert torch.equal(got, want), "rank %d shape %s" % (rank, (m_local, n, k))
            if m_local <= 512:
                # against the CPU oracle too: every rank's block of the gathered result, the peers' blocks included
                a_all = [(torch.randn(m_local, k, device="cuda", generator=torch.Generator(device="cuda").manual_seed(
                    100 + r)) * 0.1).half().cpu().numpy() for r in range(world)]
                ref = np.concatenate([oracle.gemmrc(ar, b.cpu().numpy()) for ar in a_all], axis=0)
                assert oracle.floored_max_rel(got.cpu().numpy(), ref) <= oracle.REL_TOL, "oracle, rank %d" % rank
        # Row-sharded GEMM + LayerNorm: the statistics are per row, so the gathered result of the two ranks must be
        # what one GPU computes for all rows.
        from beam.sharded import sharded_gemm_layernorm
        m_local, n, k = 2560, 2048, 256
        xs = [(torch.randn(m_local, k, device="cuda", generator=torch.Generator(device="cuda").manual_seed(500 + r))
               * 0.05).half() for r in range(world)]
        gw = torch.Generator(device="cuda").manual_seed(9)
        w = (torch.randn(n, k, device="cuda", generator=gw) * 0.05).half()
        gamma = (1 + 0.1 * torch.randn(n, device="cuda", generator=gw)).half()
        beta = (0.1 * torch.randn(n, device="cuda", generator=gw)).half()
        out_local = torch.empty(m_local, n, dtype=torch.float16, device="cuda")
        sharded_gemm_layernorm(xs[rank], w, out_local, gamma, beta, 1e-5)
        got = all_gather_rows(out_local, m_local * world)
        full = torch.empty(m_local * world, n, dtype=torch.float16, device="cuda")
        beam.cutlass_parallel_gemmrc_lnr(torch.cat(xs), w, full, gamma, beta, 1e-5)
        torch.cuda.synchronize()
        assert torch.equal(got, full), "sharded LayerNorm, rank %d" % rank
        # Host-resident operands: each rank uploads 1/world of B, the ranks all-gather it over NVLink, and only the
        # rank's own rows of A and C cross PCIe.
        from beam.sharded import ShardedHostGemm
        m_local, n, k = 1280, 1024, 512
        gb = torch.Generator().manual_seed(31)
        b_host = (torch.randn(n, k, generator=gb) * 0.1).half().pin_memory()
        a_host = (torch.randn(m_local, k, generator=torch.Generator().manual_seed(40 + rank)) * 0.1).half().pin_memory()
        c_host = torch.zeros(m_local, n, dtype=torch.float16).pin_memory()
        ShardedHostGemm(n, k)(a_host, b_host, c_host)
        c_dev = torch.empty(m_local, n, dtype=torch.float16, device="cuda")
        beam.gemmrc(a_host.cuda(), b_host.cuda(), c_dev, whole_tiles=True)  # the host entry multiplies whole tiles only
        torch.cuda.synchronize()
        assert torch.equal(c_dev.cpu(), c_host), "sharded host GEMM, rank %d" % rank
        assert oracle.floored_max_rel(c_host.numpy(), oracle.gemmrc(a_host.numpy(), b_host.numpy())) <= oracle.REL_TOL
        st, word = beam.device_status()
        assert (st, word) == (0, 0)
        open(os.path.join(out_dir, "ok%d" % rank), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_fused_gemm_allgather_two_gpus(tmp_path, built_library, oracle_mod):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]
