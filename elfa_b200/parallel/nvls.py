"""Collectives through the NVSwitch multicast mapping of a symmetric arena (``csrc/multimem.cu``).

``multimem.ld_reduce`` sums one address over all GPUs inside the switch and ``multimem.st`` writes one value to all of them,
so an all-reduce is one pass over this rank's ``1 / world`` slice. Opt-in (``ELFA_NVLS=1``): the arena is then bound to a
multicast object, which must not outlive any rank of the group - jobs in which ranks may leave (fault plans, heartbeats,
the restart loop) keep to the peer-pointer kernels.

reference: the collective set of ``src/runtime/nccl.zig:222-333`` (all-reduce, reduce-scatter, all-gather) and the barrier of
``src/runtime/main.zig:170-176``; the switch reduction itself has no counterpart there.
"""
from __future__ import annotations

import ctypes

import torch

from ..native import lib, stream_ptr
from ..runtime.symm import Region, SymmetricArena

_DT = {torch.float32: 0, torch.bfloat16: 1}


class MultimemGroup:
    def __init__(self, arena: SymmetricArena):
        if not arena.multicast_ptr:
            raise RuntimeError("the arena has no multicast mapping: NVLS is unavailable or ELFA_NVLS=1 was not set before it was created")
        self.arena = arena
        self.flags = arena.alloc(1024, "nvls.barrier")
        self.peers = (ctypes.c_uint64 * arena.world)(*[arena.peer_address(r, self.flags) for r in range(arena.world)])
        self.epoch = 0
        arena.barrier()

    def _barrier(self, stream: int) -> None:
        self.epoch += 1
        lib.call("elfa_symm_barrier", ctypes.addressof(self.peers), self.flags.tensor, self.arena.rank, self.arena.world, self.epoch, 0,
                 stream)

    def _run(self, region: Region, n: int, dtype: torch.dtype, out, scale: float, mode: int, offset_elems: int = 0) -> None:
        a = self.arena
        st = stream_ptr(region.tensor)
        esz = 2 if dtype == torch.bfloat16 else 4
        self._barrier(st)                       # every rank's operand is complete and visible
        lib.call("elfa_multimem_collective", a.multicast_ptr, a.buf, out, region.offset + offset_elems * esz, n, _DT[dtype], a.rank,
                 a.world, float(scale), mode, st)
        self._barrier(st)                       # every rank's stores have landed / every read is done

    def all_reduce_(self, region: Region, n: int, dtype: torch.dtype = torch.float32, scale: float = 1.0, offset_elems: int = 0) -> None:
        """In place: the first ``n`` elements of ``region`` become ``scale *`` their sum over the group, on every rank."""
        self._run(region, n, dtype, None, scale, 0, offset_elems)

    def reduce_scatter(self, region: Region, n: int, out: torch.Tensor, dtype: torch.dtype = torch.float32, scale: float = 1.0) -> torch.Tensor:
        """``out [n / world]`` = ``scale *`` the group sum of this rank's slice of ``region``."""
        assert out.numel() * self.arena.world == n and out.dtype == dtype and out.is_contiguous()
        self._run(region, n, dtype, out, scale, 1)
        return out

    def all_gather_(self, region: Region, n: int, dtype: torch.dtype = torch.float32) -> None:
        """This rank's slice of the first ``n`` elements of ``region`` is written to every rank's copy of the region."""
        self._run(region, n, dtype, None, 1.0, 2)
