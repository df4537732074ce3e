"""Symmetric memory arena for the peer-memory communication kernels.

Every rank of a group allocates one arena of identical size; after the rendezvous each rank holds
the device addresses of all peers' arenas (mapped over NVLink), so a kernel can load from / store
to a peer with plain pointers. Regions are carved out with a bump allocator whose call sequence is
identical on all ranks, which makes region offsets symmetric. A region of 32-bit signal words
lives in the same arena.

Native counterpart of the reference's peer-access plumbing and its host "device arenas"
(reference: ``src/runtime/main.zig:382-388`` all-pairs ``enablePeerAccess``, ``src/runtime/cuda.zig:481-491``,
``src/memory.zig:4-70`` per-device bump arenas with peer copies), which the reference never used for
communication. Allocation and address exchange use ``torch.distributed._symmetric_memory``
(CUDA VMM handles exchanged over the process group); every data-path kernel is this library's own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

ALIGN = 1024     # bytes
CANARY = 0xE1FAB200E1FAB200 - (1 << 64)     # guard word (as int64) written behind every region
GUARD = 1024     # bytes of guard words behind every region (the arena's allocation quantum)


@dataclass
class Region:
    offset: int                  # bytes from the arena base (same on every rank)
    nbytes: int
    tensor: torch.Tensor         # this rank's view (uint8)

    def view(self, dtype: torch.dtype, shape) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        esz = torch.empty(0, dtype=dtype).element_size()
        assert n * esz <= self.nbytes, "region too small for the requested view"
        return self.tensor[: n * esz].view(dtype).view(shape)


class SymmetricArena:
    """One arena per (group, device)."""

    _instances: Dict[Tuple[int, int], "SymmetricArena"] = {}

    def __init__(self, group, device: torch.device, nbytes: int):
        import os
        # Only plain peer pointers are used unless ELFA_NVLS=1 asks for the multimem kernels: without it the arena is not bound
        # to an NVLink multicast object, so a rank that leaves (fault plan, heartbeat failure, restart loop) cannot raise
        # NVLink faults on its peers' GPUs.
        if os.environ.get("ELFA_NVLS", "0") != "1":
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.device = device
        self.nbytes = nbytes
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.peer_ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        # multicast address of the arena (0 when the fabric has no NVLS or ELFA_NVLS is not 1): the multimem kernels' operand
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0) if os.environ.get("ELFA_NVLS", "0") == "1" else 0
        assert self.peer_ptrs[self.rank] == self.buf.data_ptr()
        self.buf.zero_()
        self._cursor = 0
        self._guards: List[Tuple[int, str]] = []
        self._named: Dict[str, Region] = {}
        self.epochs: Dict[str, int] = {}
        # device copy of the peer base addresses (kernels index it by rank)
        self.peer_table = torch.tensor(self.peer_ptrs, dtype=torch.int64, device=device)
        dist.barrier(self.group)
        torch.cuda.synchronize(device)

    @classmethod
    def for_group(cls, group, device: torch.device, nbytes: Optional[int] = None) -> "SymmetricArena":
        key = (id(group), device.index or 0)
        inst = cls._instances.get(key)
        if inst is None:
            if nbytes is None:
                import os
                nbytes = int(os.environ.get("ELFA_SYMM_BYTES", str(6 << 30)))
            inst = cls(group, device, nbytes)
            cls._instances[key] = inst
        return inst

    # ------------------------------------------------------------------ allocation
    def alloc(self, nbytes: int, name: Optional[str] = None) -> Region:
        """Bump allocation; with ``name`` the region is created once and reused afterwards.
        Must be called in the same order with the same sizes on every rank."""
        if name is not None and name in self._named:
            r = self._named[name]
            if r.nbytes < nbytes:
                raise RuntimeError(f"symmetric region '{name}' was created with {r.nbytes} bytes, {nbytes} requested")
            return r
        size = (nbytes + ALIGN - 1) // ALIGN * ALIGN
        if self._cursor + size + GUARD > self.nbytes:
            raise MemoryError(f"symmetric arena exhausted ({self._cursor} + {size} > {self.nbytes}); set ELFA_SYMM_BYTES")
        r = Region(self._cursor, size, self.buf[self._cursor:self._cursor + size])
        self._cursor += size
        # guard words behind the region: a kernel (this rank's or a peer's) that writes past a region's end lands here first
        g = self.buf[self._cursor:self._cursor + GUARD].view(torch.int64)
        g.fill_(CANARY)
        self._guards.append((self._cursor, name or f"region@{r.offset}"))
        self._cursor += GUARD
        if name is not None:
            self._named[name] = r
        return r

    def check_canaries(self) -> List[str]:
        """Names of the regions whose guard words were overwritten (synchronises the device). The stand-in for a memory
        checker on the peer-addressable memory, where an out-of-range store from another GPU would otherwise go unnoticed
        (reference: ``scripts/profile.sh:43-57`` runs compute-sanitizer memcheck / racecheck instead)."""
        torch.cuda.synchronize(self.device)
        bad = []
        for off, name in self._guards:
            if not bool((self.buf[off:off + GUARD].view(torch.int64) == CANARY).all()):
                bad.append(name)
        return bad

    def peer_address(self, rank: int, region: Region) -> int:
        return self.peer_ptrs[rank] + region.offset

    def next_epoch(self, name: str) -> int:
        """Monotonic per-region call counter (identical on all ranks because the call sequence is);
        signal words are compared against ``epoch * contributions`` and never reset."""
        e = self.epochs.get(name, 0) + 1
        self.epochs[name] = e
        return e

    def barrier(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
