"""The safety net under every kernel: a device-side wait that nothing satisfies gives up after its time limit,
records a fault code, lets the common teardown run and returns, and the GPU context stays usable.

The product kernels' limit is two seconds and is never reached in a healthy run, so this test drives the same
wait functions (csrc/umma_common.cuh) from a test-only kernel (tests/csrc/wait_probe.cu) with a limit of one
millisecond on mbarriers that are initialised and never arrived on.  Nothing here faults, traps or hangs: the
wait is bounded by construction and the kernel ends by itself within a few milliseconds.
"""
import ctypes
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def probe():
    sys.path.insert(0, os.path.join(HERE, "csrc"))
    import build_probe
    L = ctypes.CDLL(build_probe.build())
    L.wait_probe_launch.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_ulonglong, ctypes.c_void_p]
    return L


@pytest.mark.parametrize("ctas", [1, 8])
def test_wait_gives_up_and_the_context_stays_usable(probe, built_library, oracle_mod, ctas):
    import beam
    torch.cuda.set_device(0)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.zeros(4, dtype=torch.int32, device="cuda")
    limit_ns = 1_000_000
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert probe.wait_probe_launch(status.data_ptr(), out.data_ptr(), ctas, limit_ns, stream) == 0
    torch.cuda.synchronize()           # returns: the kernel ended by itself
    producer_ok, warp_ok, finished, waited_us = (int(v) for v in out.cpu())
    assert producer_ok == 0 and warp_ok == 0, "both waits must report that they gave up"
    assert finished == ctas, "every CTA must reach the end of the teardown"
    assert int(status.item()) in (0x101, 0x104), hex(int(status.item()))   # kFaultProducerWait / kFaultEpilogueWait
    assert limit_ns / 1000 <= waited_us < 100_000, waited_us
    # the library's own fault word is untouched and a normal GEMM right after still passes
    rng = np.random.Generator(np.random.PCG64(5))
    a = rng.uniform(-1, 1, (256, 512)).astype(np.float16)
    b = rng.uniform(-1, 1, (384, 512)).astype(np.float16)
    c = torch.zeros(256, 384, dtype=torch.float16, device="cuda")
    beam.cutlass_gemmrc(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), c)
    torch.cuda.synchronize()
    assert beam.device_status() == (0, 0)
    assert oracle_mod.floored_max_rel(c.cpu().numpy(), oracle_mod.gemmrc(a, b)) <= oracle_mod.REL_TOL
