"""Process mesh ``(dp, tp)`` and rank arithmetic.

Global rank layout follows the reference's descriptor
``rank = (pp * DP + dp) * TP + tp`` (reference: ``src/tensor/sharding.zig:357-412``), i.e. tensor
parallel ranks are contiguous GPUs. Pipeline parallelism is accepted only with size 1.
One process per GPU; groups are ``torch.distributed`` groups (NCCL on GPUs, gloo in CPU tests).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.distributed as dist


@dataclass
class ParallelContext:
    world_size: int = 1
    rank: int = 0
    tp_size: int = 1
    dp_size: int = 1
    tp_rank: int = 0
    dp_rank: int = 0
    tp_group: Optional[object] = None
    dp_group: Optional[object] = None
    sequence_parallel: bool = False
    comm_backend: str = "nccl"          # "fused" (peer-memory kernels) or "nccl"
    tp_ranks: List[int] = field(default_factory=lambda: [0])
    dp_ranks: List[int] = field(default_factory=lambda: [0])
    symm: Optional[object] = None       # runtime.symm.SymmetricArena of the TP group (fused backend)
    # context parallelism: ``cp_size`` consecutive members of the data-parallel group share one batch and
    # split its sequence dimension (ring attention); for gradients they are ordinary data-parallel ranks
    cp_size: int = 1
    cp_rank: int = 0
    cp_group: Optional[object] = None
    cp_ranks: List[int] = field(default_factory=lambda: [0])
    cp_mode: str = "ring"               # "ring" or "ulysses" (all-to-all head scatter)

    @property
    def is_distributed(self) -> bool:
        return self.world_size > 1


def global_rank(dp_rank: int, tp_rank: int, tp_size: int, pp_rank: int = 0, dp_size: int = 1) -> int:
    return (pp_rank * dp_size + dp_rank) * tp_size + tp_rank


def mesh_coords(rank: int, tp_size: int, dp_size: int):
    """-> (dp_rank, tp_rank)"""
    return (rank // tp_size) % dp_size, rank % tp_size


def init_distributed(backend: Optional[str] = None, timeout_s: float = 600.0) -> int:
    """Initialises ``torch.distributed`` from the launcher's environment (RANK, WORLD_SIZE,
    MASTER_ADDR, MASTER_PORT, LOCAL_RANK). Returns the world size (1 when not launched distributed)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return 1
    if dist.is_initialized():
        return dist.get_world_size()
    import datetime
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    kw = {}
    if backend == "nccl":
        local = int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0")))
        torch.cuda.set_device(local)
        kw["device_id"] = torch.device("cuda", local)
    dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return dist.get_world_size()


def build_context(tp_size: int = 1, sequence_parallel: bool = True, comm_backend: str = "nccl", cp_size: int = 1,
                  cp_mode: str = "ring") -> ParallelContext:
    """Creates the (dp, tp) groups, and with ``cp_size > 1`` the context-parallel groups inside every
    data-parallel group (``dp_rank = replica * cp_size + cp_rank``). Every rank must call this with the
    same arguments."""
    if not dist.is_initialized():
        return ParallelContext(sequence_parallel=False, comm_backend=comm_backend)
    world, rank = dist.get_world_size(), dist.get_rank()
    if world % tp_size != 0:
        raise ValueError(f"world size {world} is not a multiple of tensor_parallel_size {tp_size}")
    dp_size = world // tp_size
    dp_rank, tp_rank = mesh_coords(rank, tp_size, dp_size)
    ctx = ParallelContext(world_size=world, rank=rank, tp_size=tp_size, dp_size=dp_size, tp_rank=tp_rank, dp_rank=dp_rank,
                          sequence_parallel=sequence_parallel and tp_size > 1, comm_backend=comm_backend)
    for d in range(dp_size):
        ranks = [global_rank(d, t, tp_size) for t in range(tp_size)]
        g = dist.new_group(ranks) if tp_size > 1 else None
        if d == dp_rank:
            ctx.tp_group, ctx.tp_ranks = g, ranks
    for t in range(tp_size):
        ranks = [global_rank(d, t, tp_size) for d in range(dp_size)]
        g = dist.new_group(ranks) if dp_size > 1 else None
        if t == tp_rank:
            ctx.dp_group, ctx.dp_ranks = g, ranks
    if cp_size > 1:
        if dp_size % cp_size != 0:
            raise ValueError(f"data-parallel size {dp_size} is not a multiple of context_parallel_size {cp_size}")
        ctx.cp_size, ctx.cp_rank, ctx.cp_mode = cp_size, dp_rank % cp_size, cp_mode
        for t in range(tp_size):
            for rep in range(dp_size // cp_size):
                ranks = [global_rank(rep * cp_size + c, t, tp_size) for c in range(cp_size)]
                g = dist.new_group(ranks)
                if t == tp_rank and rep == dp_rank // cp_size:
                    ctx.cp_group, ctx.cp_ranks = g, ranks
    return ctx
