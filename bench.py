#!/usr/bin/env python
"""Benchmark of the fp16 rc GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (per GPU): C[8192,8192] = A[8192,8192] x B[8192,8192]^T, fp16 in, fp32 accumulate, fp16 out, inputs
0.1 * normal(0,1) from a fixed seed.  At N GPUs every rank owns an 8192-row block of A and C and a copy of B
(weak scaling); at N = 8 this is the row-sharded 65536 x 8192 x 8192 problem.  No collective is on the timed
path (the all-gather of C is optional and reported separately under "extras").

A step is one launch of the default kernel (`cutlass_gemmrc`: 256x512 tiles on CTA pairs).  `value` is
whole-job TFLOP/s with inputs resident in HBM, timed with CUDA events, max over ranks.  `e2e` is the same
metric through the host-buffer entry (pinned host A, B -> device -> kernel -> pinned host C) with the copies
inside the timed region.  One JSON line on stdout (rank 0).

`--impl reference` times the reference's CPU-side statement of the same GEMM (the fp32 CPU loop of oracle/,
all host threads) on a bounded sample of rows of the same workload; rank 0 only.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "general-nvgpu-testing_b200"))
sys.path.insert(0, ROOT)

M_PER_GPU, N, K = 8192, 8192, 8192
SEED = 1234 + 2
METRIC = "fp16 gemmrc TFLOP/s (M=8192 per GPU, N=K=8192, fp32 accumulate)"
UNIT = "TFLOP/s"
# DRAM bytes per launch of the default kernel (256x512 pair tile) at 8192^3, from the committed ncu
# capture of that kernel: dram__bytes_read.sum + dram__bytes_write.sum.
NCU_DRAM_BYTES_PER_LAUNCH = 8.49817e8 + 1.26315e8

REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
           0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x100: "display_clock_setting"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            return {"burst": float(d["bf16_tflops"]), "sustained": float(d.get("bf16_tflops_sustained", 0.0)),
                    "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
        except Exception:
            pass
    return {"burst": 1590.0, "sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Polls SM clock and clock-event reasons through NVML while a timed region runs (reads only)."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                for bit, name in REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def physical_index(local_index):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:
            return local_index
    return local_index


def cpu_sample(oracle, a_rows, b, seconds_target):
    """Times the CPU fp32 loop on the first rows of the workload; returns (TFLOP/s, rows used)."""
    import numpy as np
    probe = min(256, a_rows.shape[0])  # large enough to amortise the one-off widening of B
    t0 = time.perf_counter()
    oracle.gemmrc(a_rows[:probe], b)
    dt = max(time.perf_counter() - t0, 1e-4)
    rows = int(min(a_rows.shape[0], max(probe, (seconds_target / dt) * probe)))
    rows = max(16, rows // 16 * 16)
    t0 = time.perf_counter()
    oracle.gemmrc(a_rows[:rows], b)
    dt = time.perf_counter() - t0
    return 2.0 * rows * b.shape[0] * b.shape[1] / dt * 1e-12, rows, dt


def host_gemm_mkl(a_rows, b, seconds_target=4.0):
    """The host GEMM a user of the reference would have at hand: torch-CPU fp32 `a.float() @ b.float().T` (MKL, all
    threads) on the first rows of the workload, sized to a few seconds.  Returns a dict for the JSON line."""
    import torch
    try:
        torch.set_num_threads(os.cpu_count() or 1)
    except Exception:
        pass
    bf = torch.from_numpy(b).float()
    probe = min(512, a_rows.shape[0])
    af = torch.from_numpy(a_rows[:probe]).float()
    torch.matmul(af, bf.t())  # first call: thread pool start-up
    t0 = time.perf_counter()
    torch.matmul(af, bf.t())
    dt = max(time.perf_counter() - t0, 1e-4)
    rows = int(min(a_rows.shape[0], max(probe, seconds_target / dt * probe)))
    af = torch.from_numpy(a_rows[:rows]).float()
    t0 = time.perf_counter()
    torch.matmul(af, bf.t())
    dt = time.perf_counter() - t0
    return {"value": 2.0 * rows * b.shape[0] * b.shape[1] / dt * 1e-12, "unit": UNIT, "cores": torch.get_num_threads(),
            "kind": "torch-CPU fp32 matmul (MKL), operands widened outside the timer",
            "sample": "first %d rows of A x all of B (%d x %d x %d), %.2f s" % (rows, rows, b.shape[0], b.shape[1], dt)}


def run_reference(args):
    """The reference has no CPU implementation of this path and its CUDA sources cannot be timed on host cores;
    its CPU-side statement (fp32 loop, oracle/gemmrc_oracle.c) is timed instead, all threads, bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    from oracle import build_oracle
    build_oracle.build()
    import oracle
    oracle.use_all_cores()
    rng = np.random.Generator(np.random.PCG64(SEED))
    budget = min(2.0, 150.0 / max(args.steps + args.warmup, 1))
    b = (rng.standard_normal((N, K), dtype=np.float32) * 0.1).astype(np.float16)
    a = (rng.standard_normal((1024, K), dtype=np.float32) * 0.1).astype(np.float16)
    tf, rows, dt = cpu_sample(oracle, a, b, budget)
    for _ in range(max(args.warmup - 1, 0)):
        oracle.gemmrc(a[:rows], b)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.gemmrc(a[:rows], b)
    dt = (time.perf_counter() - t0) / args.steps
    value = 2.0 * rows * N * K / dt * 1e-12
    sample = "first %d rows of A x all of B (%d x %d x %d) per step" % (rows, rows, N, K)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 accumulate of f16 (CPU)", "data": "synthetic",
        "config": {"workload": "fp16 gemmrc 8192x8192x8192 (BASELINE configs[1]), sampled rows", "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
                         "sample": sample, "host_gemm_mkl": host_gemm_mkl(a, b)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def load_reference_module():
    """The reference's own extension (its CuTe / CUTLASS sm80-era kernels, built unmodified for sm_100a by
    baseline/build_reference.py into the git-ignored baseline/_ref): comparison only.  None if it is not built."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not any(f.startswith("beam_C") and f.endswith(".so") for f in (os.listdir(ref_dir) if os.path.isdir(ref_dir) else [])):
        return None
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    import beam_C  # prints its cuBLAS / CUTLASS versions to stderr
    return beam_C


def reference_kernels(torch, beam_C, a, b, c, ev_time, do_bench_ms):
    """The reference's large-GEMM kernels on the bench inputs: its two CuTe kernels, the CUTLASS default and the five
    tile / warp instances of cutlass_gemmrc_spec (cuda/cutlass_kernels/cutlass_gemmrc.cu:105-110)."""
    res = {}
    want = torch.matmul(a, b.t()).float()
    flop = 2.0 * M_PER_GPU * N * K
    cases = [("custom_gemmrc_128x128", lambda: beam_C.custom_gemmrc_128x128(a, b, c)),
             ("custom_gemmrc_128x256", lambda: beam_C.custom_gemmrc_128x256(a, b, c)),
             ("cutlass_gemmrc", lambda: beam_C.cutlass_gemmrc(a, b, c))]
    for tb, wp in (([128, 128], [64, 64]), ([128, 256], [64, 64]), ([256, 128], [64, 64]), ([256, 128], [128, 32]),
                   ([256, 128], [32, 128])):
        cases.append(("cutlass_gemmrc_spec_%dx%d_warp_%dx%d" % (tb[0], tb[1], wp[0], wp[1]),
                      lambda tb=tb, wp=wp: beam_C.cutlass_gemmrc_spec(a, b, c, tb, wp)))
    for name, fn in cases:
        try:
            c.zero_()
            ms = ev_time(fn, 5)
            err = float((c.float() - want).abs().max() / want.abs().max())
            res[name] = {"tflops": flop / ms * 1e-9, "max_abs_err_over_max": err}
            if name in ("custom_gemmrc_128x256", "cutlass_gemmrc"):
                res[name]["do_bench_tflops"] = flop / do_bench_ms(fn) * 1e-9
        except Exception as ex:
            res[name] = "failed: %r" % (ex,)
    return res


def extras(beam, torch, a, b, c, peaks, clock_sampler):
    """Side measurements on rank 0 at N = 1 (bounded to well under a minute of GPU time): cuBLAS on the same inputs,
    every tile family, a sustained ours / cuBLAS comparison, the reference's own kernels, the split-K shapes against
    the HBM roofline (CUDA-graph batches over rotating input sets larger than L2), GEMM + SiLU and GEMM + LayerNorm.
    Every leg carries the SM clock and throttle reasons sampled while it ran."""
    out = {}
    flop = 2.0 * M_PER_GPU * N * K

    def ev_time(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / iters

    def do_bench_ms(fn):
        """The reference's timer (python/gemm_test.py:73-75, python/beam/tuner.py:38-39): L2 flushed before every
        repetition, 100 ms of warm-up, 100 ms of repetitions, mean."""
        from triton.testing import do_bench
        return float(do_bench(fn, warmup=100, rep=100))

    t_start = time.perf_counter()

    def leg(name, fn):
        """Runs one leg under its own clock sampler; a failing leg is reported, not raised.  Legs that would start
        after four minutes of side measurements are skipped, so that the whole command stays within minutes."""
        if time.perf_counter() - t_start > 240.0:
            out[name] = "skipped: time budget of the side measurements used up"
            return
        t0 = time.perf_counter()
        with clock_sampler() as clk:
            try:
                res = fn()
            except Exception as ex:
                res = {"error": repr(ex)}
        if isinstance(res, dict):
            res["clocks"] = clk.summary()
        out[name] = res
        sys.stderr.write("[bench] %s: %.1f s\n" % (name, time.perf_counter() - t0))
        sys.stderr.flush()

    beam_C = None
    try:
        beam_C = load_reference_module()
    except Exception as ex:
        out["reference_module_error"] = repr(ex)

    def large_gemm_leg():
        # Each kernel is timed as a burst of 20 launches after half a second of idling, like the headline: timed
        # back to back, the later kernels of the list would run at the power-capped clock the earlier ones left behind.
        def burst(fn):
            torch.cuda.synchronize()
            time.sleep(0.5)
            return flop / ev_time(fn, 20) * 1e-9
        r = {"cublas_fp32acc_tflops": burst(lambda: torch.matmul(a, b.t(), out=c))}
        for name, tb in (("128x128", [128, 128]), ("128x256", [128, 256]), ("256x128", [256, 128]),
                         ("256x256", [256, 256]), ("256x512", [256, 512])):
            r["tile_%s_tflops" % name] = burst(lambda: beam.cutlass_gemmrc_spec(a, b, c, shape_threadblock=tb))
        return r

    leg("large_gemm_8192", large_gemm_leg)
    # kept at the top level too: earlier records read these keys there
    if "error" not in out["large_gemm_8192"]:
        for k_, v_ in out["large_gemm_8192"].items():
            if k_ != "clocks":
                out[k_] = v_

    def do_bench_leg():
        r = {"timer": "triton.testing.do_bench(warmup=100, rep=100), the reference's timer: L2 flushed before each call"}
        r["ours_cutlass_gemmrc_tflops"] = flop / do_bench_ms(lambda: beam.cutlass_gemmrc(a, b, c)) * 1e-9
        r["cublas_tflops"] = flop / do_bench_ms(lambda: torch.matmul(a, b.t(), out=c)) * 1e-9
        return r

    leg("do_bench_8192", do_bench_leg)

    def sustained_leg():
        """Ours and cuBLAS in alternating blocks (A B A B), about 2 s of launches each after a common warm-up, so that
        both see the same power-capped clock regime; reported as TFLOP/s and as SM cycles per launch (time x median
        SM clock of that arm's own samples), which separates the kernel from the clock it was given."""
        ours = lambda: beam.cutlass_gemmrc(a, b, c)
        cub = lambda: torch.matmul(a, b.t(), out=c)
        for _ in range(300):
            ours()
        torch.cuda.synchronize()
        per_block, blocks = 700, 4
        arms = {"ours": {"ms": 0.0, "mhz": []}, "cublas": {"ms": 0.0, "mhz": []}}
        for blk in range(2 * blocks):
            name, fn = ("ours", ours) if blk % 2 == 0 else ("cublas", cub)
            with clock_sampler() as clk:
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                for _ in range(per_block):
                    fn()
                e.record()
                torch.cuda.synchronize()
            arms[name]["ms"] += s.elapsed_time(e)
            arms[name]["mhz"] += clk.samples
        r = {"launches_per_arm": per_block * blocks, "pattern": "ABAB blocks of %d launches after 300 warm-up launches" % per_block}
        for name, d in arms.items():
            ms = d["ms"] / (per_block * blocks)
            mhz = sorted(d["mhz"])[len(d["mhz"]) // 2] if d["mhz"] else None
            r[name] = {"tflops": flop / ms * 1e-9, "ms_per_launch": ms, "seconds": d["ms"] * 1e-3, "sm_mhz_median": mhz,
                       "sm_cycles_per_launch": ms * 1e-3 * mhz * 1e6 if mhz else None}
        r["ours_over_cublas"] = r["ours"]["tflops"] / r["cublas"]["tflops"]
        return r

    leg("sustained_8192_ours_vs_cublas", sustained_leg)

    if beam_C is not None:
        leg("reference_kernels_sm80_on_b200", lambda: reference_kernels(torch, beam_C, a, b, c, ev_time, do_bench_ms))
    else:
        out["reference_kernels_sm80_on_b200"] = "not built"

    def graph_us(fns):
        for f in fns:
            f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            with torch.cuda.graph(g, stream=st):
                for f in fns:
                    f()
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(5):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            g.replay()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e) / len(fns) * 1e3)
        return sorted(ts)[len(ts) // 2]

    def splitk_leg(m, n, k):
        # A ~10 us kernel timed straight after a power-saturating GEMM loop measures the throttled clock the
        # GEMMs left behind (both this kernel and cuBLAS read 40 % slower for about a second), so let it settle.
        torch.cuda.synchronize()
        time.sleep(1.5)
        sets = 6  # 6 x (A + B) > 126 MB of L2, walked cyclically: every launch reads from HBM
        As = [(torch.rand(m, k, device="cuda") * 2 - 1).half() for _ in range(sets)]
        Bs = [(torch.rand(n, k, device="cuda") * 2 - 1).half() for _ in range(sets)]
        cc = torch.zeros(m, n, dtype=torch.float16, device="cuda")
        bytes_ = 2.0 * (m * k + n * k + m * n)
        roof = lambda us: bytes_ / (us * 1e-6) * 1e-9 / peaks["hbm_gbs"]
        batch = lambda fn: graph_us([(lambda i=i: fn(As[i % sets], Bs[i % sets])) for i in range(24)])
        # "plain": every call waits for the call before it (a chain of dependent calls, no promise from the caller);
        # "overlapped": BEAM_FLAG_INPUTS_STABLE, consecutive calls may stream side by side.
        r = {"algorithmic_bytes": bytes_, "hbm_peak_GBps": peaks["hbm_gbs"], "peak_source": peaks["source"],
             "plan_plain": beam.splitk_describe(m, n, k), "plan_overlapped": beam.splitk_describe(m, n, k, inputs_stable=True)}
        r["us_plain"] = batch(lambda x, y: beam.cutlass_gemmrc_splitk(x, y, cc))
        r["us_plain_two_kernels"] = batch(lambda x, y: beam.cutlass_gemmrc_splitk(x, y, cc, two_kernels=True))
        r["us_overlapped"] = batch(lambda x, y: beam.cutlass_gemmrc_splitk(x, y, cc, inputs_stable=True))
        r["us_overlapped_two_kernels"] = batch(lambda x, y: beam.cutlass_gemmrc_splitk(x, y, cc, inputs_stable=True,
                                                                                        two_kernels=True))
        r["frac_plain"] = roof(r["us_plain"])
        r["frac_plain_two_kernels"] = roof(r["us_plain_two_kernels"])
        us = min(r["us_overlapped"], r["us_overlapped_two_kernels"])
        r["GBps"] = bytes_ / (us * 1e-6) * 1e-9
        r["frac_of_%s_hbm" % peaks["source"]] = roof(us)
        r["cublas_us"] = batch(lambda x, y: torch.matmul(x, y.t(), out=cc))
        if beam_C is not None:
            # the reference's own split-K (CUTLASS GemmSplitKParallel + ReduceSplitK, two launches on the legacy
            # stream, its own slice heuristic); its default instance and the 64 x 64 one, the only one sized for M = N = 64
            want = torch.matmul(As[0], Bs[0].t()).float()
            for name, fn in (("reference_cutlass_gemmrc_splitk_us", lambda x, y: beam_C.cutlass_gemmrc_splitk(x, y, cc, 0)),
                             ("reference_splitk_spec_64x64_us",
                              lambda x, y: beam_C.cutlass_gemmrc_splitk_spec(x, y, cc, [64, 64], [32, 32], 0))):
                if name == "reference_cutlass_gemmrc_splitk_us" and (m < 128 or n < 128):
                    # Its slice heuristic counts M/128 * N/128 = 0 tiles for this shape and then loops on the host
                    # without end (cuda/cutlass_kernels/cutlass_gemmrc_splitk.cu:44-57,83): not called.
                    r[name] = "not run: the reference's heuristic does not terminate for M or N < 128"
                    continue
                try:
                    cc.zero_()
                    fn(As[0], Bs[0])
                    torch.cuda.synchronize()
                    err = float((cc.float() - want).abs().max() / want.abs().max())
                    if err > 1e-2:
                        r[name] = "did not compute this shape (max abs err / max = %.3g)" % err
                        continue
                    s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    torch.cuda.synchronize()
                    s_.record(torch.cuda.default_stream())
                    for i in range(24):
                        fn(As[i % sets], Bs[i % sets])
                    e_.record(torch.cuda.default_stream())
                    torch.cuda.synchronize()
                    r[name] = s_.elapsed_time(e_) / 24 * 1e3
                except Exception as ex:
                    r[name] = "failed: %r" % (ex,)
        return r

    for (m, n, k) in ((128, 256, 65536), (64, 64, 131072)):
        leg("splitk_%dx%dx%d" % (m, n, k), lambda: splitk_leg(m, n, k))

    def silu_leg():
        # GEMM with a co-scheduled element-wise SiLU over a second tensor (what the reference's cute_gemm_ln.cu does)
        xs = torch.randn(64 << 20, device="cuda", dtype=torch.float16)
        ys = torch.empty_like(xs)
        return {"fused_ms": ev_time(lambda: beam.cutlass_parallel_gemmrc_silu(a, b, c, xs, ys), 10),
                "gemm_ms": ev_time(lambda: beam.cutlass_gemmrc_spec(a, b, c, shape_threadblock=[256, 256]), 10),
                "torch_silu_ms": ev_time(lambda: torch.nn.functional.silu(xs, inplace=False), 10)}

    leg("gemm_8192_plus_silu_64Mi", silu_leg)

    def layernorm_leg():
        m, n, k = 16384, 4096, 4096
        x = (torch.randn(m, k, device="cuda") * 0.02).half()
        w = (torch.randn(n, k, device="cuda") * 0.02).half()
        g = (1 + 0.1 * torch.randn(n, device="cuda")).half()
        bt = (0.1 * torch.randn(n, device="cuda")).half()
        o = torch.empty(m, n, dtype=torch.float16, device="cuda")
        ms = ev_time(lambda: beam.cutlass_parallel_gemmrc_lnr(x, w, o, g, bt, 1e-5), 10)
        return {"ms": ms, "tflops": 2.0 * m * n * k / ms * 1e-9,
                "torch_matmul_plus_layer_norm_ms": ev_time(
                    lambda: torch.nn.functional.layer_norm(torch.matmul(x, w.t()), (n,), g, bt, 1e-5), 10),
                "gemm_alone_ms": ev_time(lambda: beam.cutlass_gemmrc_spec(x, w, o, shape_threadblock=[256, 256]), 10)}

    leg("gemm_layernorm_16384x4096x4096", layernorm_leg)
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import beam
    if not os.path.exists(beam.library_path()):
        raise SystemExit("libbeam_b200.so is missing; run python general-nvgpu-testing_b200/build.py")
    peaks = measured_peaks()

    # Rank r owns rows [r*8192, (r+1)*8192) of the global A; B is replicated (same seed everywhere).
    gen = torch.Generator(device="cuda").manual_seed(SEED)
    b = (torch.randn(N, K, device="cuda", generator=gen) * 0.1).half()
    gen_a = torch.Generator(device="cuda").manual_seed(SEED + 1000 + rank)
    a = (torch.randn(M_PER_GPU, K, device="cuda", generator=gen_a) * 0.1).half()
    c = torch.zeros(M_PER_GPU, N, dtype=torch.float16, device="cuda")

    def step():
        beam.cutlass_gemmrc(a, b, c)

    def barrier():
        if world > 1:
            dist.barrier()

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    st, word = beam.device_status()
    if st != 0:
        raise SystemExit("device fault word %#x after warm-up" % word)

    # ---- value: inputs resident in HBM (3 x 128 MB > the 126 MB L2, so no flush is needed between steps)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    torch.cuda.synchronize()
    with ClockSampler(physical_index(local)) as clk:
        start.record()
        for _ in range(args.steps):
            step()
        end.record()
        torch.cuda.synchronize()
    barrier()
    ms_total = start.elapsed_time(end)
    t = torch.tensor([ms_total], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_step = ms_total / args.steps
    flops_step_all = 2.0 * M_PER_GPU * N * K * world
    value = flops_step_all / (ms_step * 1e-3) * 1e-12
    per_gpu = value / world

    # ---- e2e: host buffers through the host entry, copies inside the timed region
    # (host buffers are allocated after binding the rank to its GPU's NUMA node, so that they are local to its PCIe root)
    from beam.sharded import bind_to_gpu_numa_node
    cpus_before = os.sched_getaffinity(0)
    numa_bound = bind_to_gpu_numa_node(local)
    ha, hb = a.cpu().pin_memory(), b.cpu().pin_memory()
    hc = torch.zeros(M_PER_GPU, N, dtype=torch.float16).pin_memory()  # zeros: the pages are touched here
    os.sched_setaffinity(0, cpus_before)  # only the allocations above needed the binding
    if world > 1:
        # Every rank holds A_local and all of B on the host; rank r uploads 1/world of B and the ranks all-gather it
        # over NVLink, so B crosses PCIe once per step for the whole job instead of once per rank.
        from beam.sharded import ShardedHostGemm
        host_gemm = ShardedHostGemm(N, K)
        e2e_call = lambda: host_gemm(ha, hb, hc)
    else:
        e2e_call = lambda: beam.gemmrc_host(ha, hb, hc)
    for _ in range(2):
        e2e_call()
    e2e_steps = max(3, min(args.steps, 10))
    barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_call()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    barrier()
    t = torch.tensor([dt], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = flops_step_all / (float(t.item()) / e2e_steps) * 1e-12
    e2e_ok = bool(torch.equal(hc.cuda(), c))

    gather = None
    if world > 1:
        # Optional all-gather of C over NCCL / NVLink, outside the headline: every rank ends up with all of C.
        from beam.sharded import all_gather_rows
        for _ in range(2):
            full = all_gather_rows(c, M_PER_GPU * world)
        torch.cuda.synchronize()
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(5):
            full = all_gather_rows(c, M_PER_GPU * world)
        g1.record()
        torch.cuda.synchronize()
        tg = torch.tensor([g0.elapsed_time(g1) / 5], dtype=torch.float64, device="cuda")
        dist.all_reduce(tg, op=dist.ReduceOp.MAX)
        gather_ms = float(tg.item())
        recv_bytes = 2.0 * M_PER_GPU * N * (world - 1)
        gather = {"nccl_all_gather_ms": gather_ms, "bytes_received_per_gpu": recv_bytes,
                  "GBps_in_per_gpu": recv_bytes / (gather_ms * 1e-3) * 1e-9,
                  "tflops_gemm_then_nccl_gather": flops_step_all / ((ms_step + gather_ms) * 1e-3) * 1e-12}
        # The same result from ONE kernel per rank: the GEMM epilogue stores each tile into every rank's gathered
        # buffer (peer-mapped symmetric memory) while the main loop runs on.
        try:
            from beam.sharded import GatheredC, gemmrc_allgather
            gc = GatheredC(M_PER_GPU, N)
            for _ in range(2):
                gemmrc_allgather(a, b, gc)
            torch.cuda.synchronize()
            barrier()
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record()
            for _ in range(5):
                gemmrc_allgather(a, b, gc)
            f1.record()
            torch.cuda.synchronize()
            tf_ = torch.tensor([f0.elapsed_time(f1) / 5], dtype=torch.float64, device="cuda")
            dist.all_reduce(tf_, op=dist.ReduceOp.MAX)
            fused_ms = float(tf_.item())
            mine = gc.tensor[rank * M_PER_GPU:(rank + 1) * M_PER_GPU]
            gather["fused_gemm_gather_ms"] = fused_ms
            gather["tflops_fused"] = flops_step_all / (fused_ms * 1e-3) * 1e-12
            gather["GBps_in_per_gpu_fused"] = recv_bytes / (fused_ms * 1e-3) * 1e-9
            gather["fused_matches"] = bool(torch.equal(mine, c))
            # Every block of this rank's gathered buffer (its own and the world - 1 blocks that the peers' kernels
            # stored over NVLink) against the NCCL all-gather of the same C blocks, on every rank.
            all_ok = torch.tensor([1 if torch.equal(gc.tensor, full) else 0], dtype=torch.int32, device="cuda")
            dist.all_reduce(all_ok, op=dist.ReduceOp.MIN)
            gather["fused_matches_all_blocks"] = bool(int(all_ok.item()) == 1)
        except Exception as ex:
            gather["fused_error"] = repr(ex)
        del full

    if rank == 0:
        burst = ms_total < 500.0  # a short run sits in the burst regime, a long one under the power cap
        peak = peaks["burst"] if burst or not peaks["sustained"] else peaks["sustained"]
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16 in, f32 accumulate, f16 out", "data": "synthetic",
            "config": {"workload": "fp16 gemmrc M=%d N=%d K=%d (BASELINE configs[1] per GPU; row-sharded "
                                   "configs[4] at 8 GPUs)" % (M_PER_GPU * world, N, K),
                       "rows_per_gpu": M_PER_GPU, "kernel": "cutlass_gemmrc: 256x512 tile per CTA pair (cta_group::2, two N=256 "
                       "accumulators), 3-stage TMA ring, 8-warp TMA-store epilogue", "parallelism": "rows of A sharded x%d, B replicated, no collective" % world,
                       "l2": "A, B, C are 3 x 128 MiB per GPU, larger than the 126 MB L2; no flush between steps"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 2 * (M_PER_GPU * K * world + N * K),
                    "d2h_bytes_per_step": 2 * M_PER_GPU * N * world, "steps": e2e_steps, "matches_device_path": e2e_ok,
                    "path": ("beam_gemmrc_fp16_host: A and B up in alternating row blocks, C strips back as they "
                             "become computable" if world == 1 else
                             "beam.sharded.ShardedHostGemm: each rank uploads its rows of A and 1/%d of B, B is "
                             "all-gathered over NVLink (NCCL), C rows come back; per step" % world),
                    "host_buffers_numa_local": bool(numa_bound),
                    "timer": "host clock around the blocking call (copies and kernels on internal streams)"},
            "gpu_launches": args.steps,
            "clocks": clk.summary(),
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": UNIT, "frac": per_gpu / peak,
                         "traffic": NCU_DRAM_BYTES_PER_LAUNCH,
                         "peak_source": "%s cuBLAS bf16 %s of %s" % (peaks["source"], "burst" if burst else "sustained",
                                                                     "MEASURED_PEAKS.json" if peaks["source"] ==
                                                                     "measured" else "the profiling recipe"),
                         "algorithmic_flops_per_launch": 2.0 * M_PER_GPU * N * K,
                         "frac_of_spec_2250": per_gpu / 2250.0},
        }
        if gather is not None:
            line["extras"] = {"all_gather_c": gather}
        if world == 1:
            from oracle import build_oracle
            build_oracle.build()
            import oracle
            oracle.use_all_cores()
            tf, rows, dt = cpu_sample(oracle, ha.numpy(), hb.numpy(), 10.0)
            line["cpu_baseline"] = {"value": tf, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
                                    "sample": "first %d rows of A x all of B (%d x %d x %d), %.1f s" %
                                              (rows, rows, N, K, dt),
                                    "host_gemm_mkl": host_gemm_mkl(ha.numpy(), hb.numpy())}
            if not args.no_extras:
                try:
                    line["extras"] = extras(beam, torch, a, b, c, peaks,
                                            lambda: ClockSampler(physical_index(local)))
                except Exception as ex:  # side measurements never take the headline down
                    line["extras"] = {"error": repr(ex)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_profile_case(args):
    """A handful of launches of one kernel on its BASELINE shape, for `ncu ... python bench.py --profile X`.
    layernorm runs a quarter of config 4's rows so that a full-set capture stays small."""
    import torch
    import beam
    torch.cuda.set_device(0)
    torch.manual_seed(SEED)
    n_launch = max(args.steps, 1)
    if args.profile in ("gemm", "gemm256", "gemm128x128", "gemm256x128", "gemm128x128_single", "gemm256x128_single",
                        "cublas", "gemm_k4096", "gemm256_k4096", "cublas_k4096"):  # cublas: the comparison kernel
        k_dim = 4096 if args.profile.endswith("_k4096") else K  # "_k4096": the same output with half the K
        args.profile = args.profile.replace("_k4096", "")
        a = (torch.randn(M_PER_GPU, k_dim, device="cuda") * 0.1).half()
        b = (torch.randn(N, k_dim, device="cuda") * 0.1).half()
        c = torch.zeros(M_PER_GPU, N, dtype=torch.float16, device="cuda")
        fn = {"cublas": lambda: beam.cublas_gemmexrc(a, b, c),
              "gemm256": lambda: beam.cutlass_gemmrc_spec(a, b, c, shape_threadblock=[256, 256]),  # one accumulator per tile
              # the N = 128 families: two tiles in flight (the default) and one tile at a time
              "gemm128x128": lambda: beam.custom_gemmrc_128x128(a, b, c),
              "gemm256x128": lambda: beam.cutlass_gemmrc_spec(a, b, c, shape_threadblock=[256, 128]),
              "gemm128x128_single": lambda: beam.gemmrc(a, b, c, tile_n=128, cta_pair=1, tiles_in_flight=1),
              "gemm256x128_single": lambda: beam.gemmrc(a, b, c, tile_n=128, cta_pair=2, tiles_in_flight=1),
              "gemm": lambda: beam.cutlass_gemmrc(a, b, c)}[args.profile]
    elif args.profile in ("gemm256_lastwave_4096", "gemm256_lastwave_1024"):
        # 256 x 256 tiles on pairs at a size whose last wave fills at most half of the pairs: launches alternate
        # between whole tiles and the default (last-wave tiles cut into halves), whole first
        m, n, k = (4096, 4096, 4096) if args.profile.endswith("4096") else (1024, 1024, 8192)
        a = (torch.randn(m, k, device="cuda") * 0.1).half()
        b = (torch.randn(n, k, device="cuda") * 0.1).half()
        c = torch.zeros(m, n, dtype=torch.float16, device="cuda")
        turn = [0]

        def fn():
            beam.gemmrc(a, b, c, tile_n=256, cta_pair=2, whole_tiles=(turn[0] % 2 == 0))
            turn[0] += 1
    elif args.profile in ("splitk", "splitk64", "splitk_plain", "splitk64_plain"):
        m, n, k = (128, 256, 65536) if args.profile.startswith("splitk_") or args.profile == "splitk" else (64, 64, 131072)
        a = (torch.rand(m, k, device="cuda") * 2 - 1).half()
        b = (torch.rand(n, k, device="cuda") * 2 - 1).half()
        c = torch.zeros(m, n, dtype=torch.float16, device="cuda")
        stable = not args.profile.endswith("_plain")  # "_plain": every call waits for the one before it
        fn = lambda: beam.cutlass_gemmrc_splitk(a, b, c, inputs_stable=stable)
    else:
        m, n, k = 4096, 4096, 4096
        a = (torch.randn(m, k, device="cuda") * 0.02).half()
        b = (torch.randn(n, k, device="cuda") * 0.02).half()
        g = (1 + 0.1 * torch.randn(n, device="cuda")).half()
        bt = (0.1 * torch.randn(n, device="cuda")).half()
        c = torch.zeros(m, n, dtype=torch.float16, device="cuda")
        fn = lambda: beam.cutlass_parallel_gemmrc_lnr(a, b, c, g, bt, 1e-5)
    for _ in range(n_launch):
        fn()
    torch.cuda.synchronize()
    st, word = beam.device_status()
    print(json.dumps({"profile": args.profile, "launches": n_launch, "status": st, "fault_word": word}))
    if st != 0:
        raise SystemExit(1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the cuBLAS / split-K / LayerNorm side measurements")
    ap.add_argument("--profile", default=None,
                    choices=["gemm", "gemm256", "gemm128x128", "gemm256x128", "gemm128x128_single", "gemm256x128_single",
                             "cublas", "splitk", "splitk64", "splitk_plain", "splitk64_plain", "layernorm",
                             "gemm256_lastwave_4096", "gemm256_lastwave_1024", "gemm_k4096", "gemm256_k4096",
                             "cublas_k4096"],
                    help="run a few launches of one kernel and exit (the command the ncu captures in profiles/ wrap)")
    args = ap.parse_args()
    if args.profile:
        run_profile_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
