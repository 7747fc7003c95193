"""Row-sharded rc GEMM over the GPUs of one node (no counterpart in the reference, which is single-GPU:
python/gemm_test.py:236 only ever calls torch.cuda.set_device(0)).

Rows of C depend only on the same rows of A and on all of B, so the GEMM (and the row-wise LayerNorm
after it) shards by contiguous blocks of M with no exchange: rank g owns rows [g*M/G, (g+1)*M/G) of A and
C and a full copy of B.  The only collective is the optional all-gather of C over NCCL/NVLink.
One process per GPU; torch.distributed carries the plumbing.
"""
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def row_block(m: int, world: int, rank: int) -> Tuple[int, int]:
    """[start, stop) of the rows rank `rank` of `world` owns: contiguous, sizes differ by at most one,
    earlier ranks take the remainder.  Empty blocks are possible when world > m."""
    if m < 0 or world <= 0 or not (0 <= rank < world):
        raise ValueError("bad shard request m=%d world=%d rank=%d" % (m, world, rank))
    base, rem = divmod(m, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def sharded_gemmrc(a_local: torch.Tensor, b: torch.Tensor, c_local: torch.Tensor,
                   kernel: Optional[Callable] = None) -> None:
    """c_local = a_local @ b.T on this rank's rows.  `kernel` defaults to beam.cutlass_gemmrc."""
    if a_local.shape[0] == 0:
        return
    if kernel is None:
        from . import _C
        kernel = _C.cutlass_gemmrc
    kernel(a_local, b, c_local)


def sharded_gemm_layernorm(x_local: torch.Tensor, w: torch.Tensor, out_local: torch.Tensor, gamma: torch.Tensor,
                           beta: torch.Tensor, eps: float = 1e-5) -> None:
    """out_local = LayerNorm_row(x_local @ w.T) * gamma + beta on this rank's rows.  The statistics are per row, so
    the row-sharded form needs no exchange either (BASELINE config 4 shards exactly like config 5)."""
    if x_local.shape[0] == 0:
        return
    from . import _C
    _C.cutlass_parallel_gemmrc_lnr(x_local, w, out_local, gamma, beta, eps)


def all_gather_rows(c_local: torch.Tensor, m: int, group=None) -> torch.Tensor:
    """Assembles the full C [m, N] on every rank from the ranks' row blocks (row_block order).
    Equal blocks use one all_gather_into_tensor (a single NCCL all-gather over NVLink on GPUs);
    ragged blocks fall back to per-rank broadcasts."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    n = c_local.shape[1]
    full = torch.empty((m, n), dtype=c_local.dtype, device=c_local.device)
    if m % world == 0:
        dist.all_gather_into_tensor(full, c_local.contiguous(), group=group)
        return full
    for r in range(world):
        s, e = row_block(m, world, r)
        if e > s:
            if r == rank:
                full[s:e].copy_(c_local)
            dist.broadcast(full[s:e], src=dist.get_global_rank(group, r) if group is not None else r, group=group)
    return full


class GatheredC:
    """The gathered C[world * m_local, n] of a row-sharded GEMM, allocated as torch symmetric memory so that every
    rank holds device pointers to every other rank's copy.  `tensor` is this rank's copy; `ptrs[d]` is rank d's."""

    def __init__(self, m_local: int, n: int, group=None, device=None):
        import torch.distributed._symmetric_memory as symm_mem
        group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.m_local, self.n = int(m_local), int(n)
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.tensor = symm_mem.empty((self.world * self.m_local, self.n), dtype=torch.float16, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]

    def barrier(self):
        """Stream-ordered barrier across the ranks: after it, every rank's stores issued before it have landed."""
        self.handle.barrier()


def gemmrc_allgather(a_local: torch.Tensor, b: torch.Tensor, gathered: "GatheredC", **knobs) -> torch.Tensor:
    """gathered.tensor (on every rank) = concat over ranks of a_local_r @ b.T, computed and gathered by ONE kernel per
    rank: each finished tile is TMA-stored into all ranks' buffers over NVLink while the main loop continues.
    Returns gathered.tensor; it is complete after gathered.barrier() (called here)."""
    from . import _C
    if a_local.shape[0] != gathered.m_local or b.shape[0] != gathered.n:
        raise ValueError("a_local must have %d rows and b %d rows" % (gathered.m_local, gathered.n))
    gathered.barrier()  # nobody may still be reading the previous contents
    _C.gemmrc_allgather(a_local, b, gathered.ptrs, gathered.rank, gathered.n, **knobs)
    gathered.barrier()
    return gathered.tensor


def bind_to_gpu_numa_node(device_index: Optional[int] = None) -> bool:
    """Pins the calling process to the CPUs that NVML names as closest to the GPU (its NUMA node), so that host
    buffers allocated and first touched afterwards (pinned staging memory in particular) are local to the GPU's PCIe
    root.  On a two-socket host an unbound rank otherwise allocates wherever it happens to run, and every copy then
    crosses the socket interconnect.  Reads NVML and changes this process's own CPU affinity, nothing on the GPU.
    Returns False (and changes nothing) when NVML or the affinity call is unavailable."""
    import os
    try:
        import pynvml
        pynvml.nvmlInit()
        if device_index is None:
            device_index = torch.cuda.current_device()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        if visible:
            try:
                device_index = int(visible.split(",")[device_index])
            except (ValueError, IndexError):
                pass
        handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = {64 * w + b for w, bits in enumerate(mask) for b in range(64) if (int(bits) >> b) & 1}
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return False
        os.sched_setaffinity(0, allowed)
        return True
    except Exception:
        return False


def b_shard_rows(n: int, world: int, rank: int) -> Tuple[int, int]:
    """[start, stop) of the rows of B that rank `rank` uploads in ShardedHostGemm (equal shards)."""
    if world <= 0 or not (0 <= rank < world) or n % world != 0:
        raise ValueError("N=%d does not divide over world=%d (rank %d)" % (n, world, rank))
    per = n // world
    return rank * per, (rank + 1) * per


class ShardedHostGemm:
    """Row-sharded rc GEMM for operands that live in HOST memory on every rank: C_local = A_local @ B.T.

    Sending B over PCIe once per rank would move world x |B| bytes through the host for nothing.  Here rank r
    uploads only rows [r*N/world, (r+1)*N/world) of B, the ranks all-gather the shards over NVLink (one NCCL
    all-gather, no host traffic), and the rank's rows of A and C then flow through beam_gemmrc_fp16_host_rows
    (A up, C back, pipelined).  Per step and rank PCIe carries |A_local| + |B| / world up and |C_local| down.
    """

    def __init__(self, n: int, k: int, group=None, device=None):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.n, self.k = int(n), int(k)
        if self.n % self.world != 0:
            raise ValueError("N=%d must divide evenly over %d ranks" % (self.n, self.world))
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.b_dev = torch.empty((self.n, self.k), dtype=torch.float16, device=self.device)
        self.shard = torch.empty((self.n // self.world, self.k), dtype=torch.float16, device=self.device)

    def shard_rows(self) -> Tuple[int, int]:
        """[start, stop) of the rows of B this rank uploads."""
        return b_shard_rows(self.n, self.world, self.rank)

    def __call__(self, a_local_host: torch.Tensor, b_host: torch.Tensor, c_local_host: torch.Tensor) -> None:
        """b_host is the whole B on the host (every rank has it); only this rank's shard of it is read."""
        from . import _C
        s, e = self.shard_rows()
        self.shard.copy_(b_host[s:e], non_blocking=True)
        dist.all_gather_into_tensor(self.b_dev, self.shard, group=self.group)
        _C.gemmrc_host_rows(a_local_host, self.b_dev, c_local_host)
