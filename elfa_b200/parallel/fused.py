"""Fused compute + collective primitives over NVLink peer memory (the ``fused`` comm backend).

* ``ag_gemm``  - all-gather → GEMM in one kernel (reference call sites:
  ``src/distributed/tensor_parallel.zig:77-129``, ``src/distributed/sequence_parallel.zig:79-128``);
* ``gemm_rs``  - GEMM → reduce-scatter in one kernel (``tensor_parallel.zig:154-170``,
  ``sequence_parallel.zig:184-200``).

Buffers live in the group's :class:`~elfa_b200.runtime.symm.SymmetricArena`. Each primitive owns a
ring of two slots (gathered-A buffers / receive buffers) with one set of arrival counters per
slot. Counters only ever grow; the host tracks how many arrivals each slot has been promised so
far and passes that number as the wait target. Two slots are enough because every fused op needs
data from every peer: a rank can be at most one op ahead of the slowest rank, so the slot it
writes into is never the one a peer is still reading.

Shapes the kernels do not cover (rows per rank not a multiple of 128) take the library path.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Tuple

import torch

from ..native import EPI_GELU, EPI_STORE_PREACT, lib, stream_ptr
from .mesh import ParallelContext

RING = 2
_WAIT_MS = int(os.environ.get("ELFA_FLAG_TIMEOUT_MS", "10000"))


class _Slot:
    def __init__(self, arena, name: str, nbytes: int):
        self.data = arena.alloc(nbytes, name + ".data")
        self.flags = arena.alloc(1024, name + ".flags")
        w = arena.world
        self.peer_data = (ctypes.c_uint64 * w)(*[arena.peer_address(r, self.data) for r in range(w)])
        self.peer_flags = (ctypes.c_uint64 * w)(*[arena.peer_address(r, self.flags) for r in range(w)])
        self.arrivals = ctypes.c_uint(0)


class _State:
    def __init__(self, arena):
        self.arena = arena
        self.slots: Dict[Tuple[str, int, int], _Slot] = {}
        self.counter = {"ag": 0, "rs": 0}
        self.side: Optional[torch.cuda.Stream] = None      # copies of gathered inputs out of the ring
        self.pending: Optional[torch.cuda.Event] = None

    def next_slot(self, kind: str, nbytes: int) -> _Slot:
        i = self.counter[kind] % RING
        self.counter[kind] += 1
        key = (kind, i, nbytes)
        s = self.slots.get(key)
        if s is None:
            # sizes are rounded up to 1 MiB classes so that a few shapes share a slot
            s = _Slot(self.arena, f"{kind}{i}_{nbytes}", nbytes)
            self.slots[key] = s
            # a new slot changes which buffers exist on every rank: make sure all ranks created it
            # (and zeroed counters are visible) before any peer writes into it
            self.arena.barrier()
        return s


_states: Dict[int, _State] = {}


def _state(pc: ParallelContext) -> _State:
    st = _states.get(id(pc.symm))
    if st is None:
        st = _State(pc.symm)
        _states[id(pc.symm)] = st
    return st


def wait_pending_copies(pc: ParallelContext) -> None:
    """Makes the current stream wait for the side-stream copy of the last gathered input. Called
    before the next all-gather kernel (whose peers may overwrite the ring slot two calls later) and
    before a backward pass reads such a copy."""
    st = _states.get(id(pc.symm)) if pc.symm is not None else None
    if st is not None and st.pending is not None:
        torch.cuda.current_stream().wait_event(st.pending)
        st.pending = None


def _round_class(nbytes: int) -> int:
    q = 1 << 20
    return (nbytes + q - 1) // q * q


def supported(rows_local: int, K: int, N: int) -> bool:
    return rows_local % 128 == 0 and K % 8 == 0 and N % 8 == 0


def ag_gemm(x_local: torch.Tensor, w: torch.Tensor, pc: ParallelContext, *, b_mn: bool, act: Optional[str] = None,
            preact: bool = False, keep: bool = True, defer_copy: bool = False):
    """``y = act(all_gather_rows(x_local) @ op(w))`` → ``(y, x_full, pre)``. With ``keep`` the gathered
    input is copied out of the ring (on a side stream; it outlives the slot). Without it ``x_full`` is
    the ring slot itself, valid until the second all-gather after this one. ``defer_copy``: the caller
    promises to call :func:`wait_pending_copies` before it reads ``x_full`` (the next fused all-gather
    does so by itself); otherwise the current stream waits for the copy right away."""
    world, rank = pc.tp_size, pc.tp_rank
    Ml, K = x_local.shape
    N = w.shape[1] if b_mn else w.shape[0]
    if not supported(Ml, K, N) or x_local.dtype != torch.bfloat16:
        from . import tp
        saved, pc.comm_backend = pc.comm_backend, "nccl"
        try:
            return tp.ag_gemm(x_local, w, pc, b_mn=b_mn, act=act, preact=preact, keep=keep, defer_copy=defer_copy)
        finally:
            pc.comm_backend = saved
    M = Ml * world
    st = _state(pc)
    wait_pending_copies(pc)
    slot = st.next_slot("ag", _round_class(M * K * 2))
    xl = x_local if x_local.is_contiguous() else x_local.contiguous()
    y = torch.empty((M, N), dtype=torch.bfloat16, device=x_local.device)
    pre = torch.empty((M, N), dtype=torch.bfloat16, device=x_local.device) if (act == "gelu" and preact) else None
    flags = 0
    if act == "gelu":
        flags |= EPI_GELU
        if pre is not None:
            flags |= EPI_STORE_PREACT
    lib.call("elfa_gemm_ag", xl, xl.stride(0), ctypes.addressof(slot.peer_data), ctypes.addressof(slot.peer_flags),
             slot.flags.tensor, ctypes.addressof(slot.arrivals), w, y, M, N, K, w.stride(0), y.stride(0), int(b_mn), pre,
             pre.stride(0) if pre is not None else 0, flags, rank, world, _WAIT_MS, stream_ptr(xl))
    view = slot.data.view(torch.bfloat16, (M, K))
    if not keep:
        return y, view, pre
    # kept for the weight gradient: copied while the following kernels run
    if st.side is None:
        st.side = torch.cuda.Stream(x_local.device)
    x_full = torch.empty((M, K), dtype=torch.bfloat16, device=x_local.device)
    cur = torch.cuda.current_stream()
    st.side.wait_stream(cur)
    with torch.cuda.stream(st.side):
        x_full.copy_(view)
        ev = torch.cuda.Event()
        ev.record(st.side)
    x_full.record_stream(st.side)
    st.pending = ev
    if not defer_copy:
        wait_pending_copies(pc)
    return y, x_full, pre


def gemm_rs(a: torch.Tensor, w: torch.Tensor, pc: ParallelContext, *, b_mn: bool, max_ctas: int = 0) -> torch.Tensor:
    """``reduce_scatter_rows(a @ op(w))`` → ``[M / world, N]``. ``max_ctas`` caps the grid so that a GEMM
    on another stream can run next to this (communication-bound) kernel."""
    world, rank = pc.tp_size, pc.tp_rank
    M, K = a.shape
    N = w.shape[1] if b_mn else w.shape[0]
    if M % world or not supported(M // world, K, N) or N % 64 or a.dtype != torch.bfloat16:
        from . import tp
        saved, pc.comm_backend = pc.comm_backend, "nccl"
        try:
            return tp.gemm_rs(a, w, pc, b_mn=b_mn)
        finally:
            pc.comm_backend = saved
    st = _state(pc)
    slot = st.next_slot("rs", _round_class(M * N * 2))
    ac = a if a.is_contiguous() else a.contiguous()
    out = torch.empty((M // world, N), dtype=torch.bfloat16, device=a.device)
    lib.call("elfa_gemm_rs", ac, ac.stride(0), w, w.stride(0), int(b_mn), M, N, K, ctypes.addressof(slot.peer_data),
             ctypes.addressof(slot.peer_flags), slot.flags.tensor, ctypes.addressof(slot.arrivals), out, out.stride(0), rank, world,
             _WAIT_MS, max_ctas, stream_ptr(ac))
    return out
