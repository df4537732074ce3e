"""Fused compute + collective primitives over NVLink peer memory (the ``fused`` comm backend).

* ``ag_gemm``  - all-gather → GEMM in one kernel (reference call sites:
  ``src/distributed/tensor_parallel.zig:77-129``, ``src/distributed/sequence_parallel.zig:79-128``);
* ``gemm_rs``  - GEMM → reduce-scatter in one kernel (``tensor_parallel.zig:154-170``,
  ``sequence_parallel.zig:184-200``);
* ``ag_gemm_mxfp8`` - the all-gather → GEMM of MXFP8 layers: every rank quantises its rows into its
  ring slot (e4m3 payload + scale atoms, 1.03 bytes per element instead of 2); one kernel then pushes
  that slice into every peer's slot while its tensor cores multiply block-scaled tiles, own rows
  first, a peer's rows as soon as that peer's arrival counter says they are there.

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
# MXFP8 all-gather -> GEMM as one kernel (in-kernel push of payload rows and scale atoms); "0" selects the
# quantise / barrier / peer-load gather / GEMM sequence of separate launches
_ONE_KERNEL = os.environ.get("ELFA_AG_MXFP8_ONE_KERNEL", "1") not in ("0", "")


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
        self.counter = {"ag": 0, "rs": 0, "agq": 0, "xent": 0}
        self.bar = None                                     # signal words of the stream-ordered barrier
        self.bar_peers = None
        self.bar_epoch = 0
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


    def stream_barrier(self, stream: int) -> None:
        """Barrier over the group's ranks as a kernel on ``stream`` (bounded wait on peer signal words)."""
        a = self.arena
        if self.bar is None:
            self.bar = a.alloc(1024, "fused.barrier")
            self.bar_peers = (ctypes.c_uint64 * a.world)(*[a.peer_address(r, self.bar) for r in range(a.world)])
            a.barrier()                                     # zeroed words visible everywhere before the first signal
        self.bar_epoch += 1
        lib.call("elfa_symm_barrier", ctypes.addressof(self.bar_peers), self.bar.tensor, a.rank, a.world, self.bar_epoch,
                 _WAIT_MS, stream)


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


def supported_mxfp8(rows_local: int, K: int, N: int) -> bool:
    return rows_local % 128 == 0 and K % 128 == 0 and N % 8 == 0


def ag_gemm_mxfp8(x_local: torch.Tensor, w_op, pc: ParallelContext, *, act: Optional[str] = None, preact: bool = False):
    """``y = act(all_gather_rows(q(x_local)) @ w_op^T)`` with MXFP8 operands → ``(y, x_full, pre)``.
    ``x_local [M / world, K]`` bf16 is quantised here; ``w_op`` is the cached right-hand operand
    (``[N, K]`` payload). ``x_full`` is the bf16 tensor of the gathered quantised rows (what backward
    multiplies for the weight gradient), produced on a side stream: call :func:`wait_pending_copies`
    before reading it. Only the payload and the scales cross NVLink."""
    from ..ops.gemm_mxfp8 import Mxfp8Operand, gemm_mxfp8
    world, rank = pc.tp_size, pc.tp_rank
    Ml, K = x_local.shape
    M, N = Ml * world, w_op.rows
    kt = K // 128
    pay_l, sf_l = Ml * K, (Ml // 128) * kt * 512            # this rank's share of payload / scale atoms
    st = _state(pc)
    wait_pending_copies(pc)
    slot = st.next_slot("agq", _round_class(world * (pay_l + sf_l)))
    xl = x_local if x_local.is_contiguous() else x_local.contiguous()
    stream = stream_ptr(xl)
    buf = slot.data.tensor
    payload = buf[: world * pay_l].view(M, K)
    scales = buf[world * pay_l: world * (pay_l + sf_l)]
    # 1. quantise the local rows into this rank's own slot, at the place they have in the gathered operand
    lib.call("elfa_mxfp8_quantize_gemm", xl, xl.stride(0), payload[rank * Ml:], scales[rank * sf_l:], None, Ml, K, 0, stream)
    pre = torch.empty((M, N), dtype=torch.bfloat16, device=x_local.device) if (act == "gelu" and preact) else None
    if _ONE_KERNEL:
        # 2. one kernel: push warps send this rank's payload rows and scale atoms to every peer's slot while the tensor
        #    cores start on the own rows; tiles of a peer's rows wait for that peer's arrival counter
        y = torch.empty((M, N), dtype=torch.bfloat16, device=x_local.device)
        flags = 0
        if act == "gelu":
            flags |= EPI_GELU | (EPI_STORE_PREACT if pre is not None else 0)
        lib.call("elfa_gemm_ag_mxfp8", ctypes.addressof(slot.peer_data), ctypes.addressof(slot.peer_flags), slot.flags.tensor,
                 ctypes.addressof(slot.arrivals), w_op.payload, w_op.scales, y, M, N, K, y.stride(0), pre,
                 pre.stride(0) if pre is not None else 0, flags, rank, world, _WAIT_MS, stream)
    else:
        # 2. every rank's rows are in its slot
        st.stream_barrier(stream)
        # 3. pull the other ranks' payloads and scale atoms (peer loads)
        base = [int(slot.peer_data[r]) for r in range(world)]
        src_pay = (ctypes.c_uint64 * world)(*[base[r] + r * pay_l for r in range(world)])
        src_sf = (ctypes.c_uint64 * world)(*[base[r] + world * pay_l + r * sf_l for r in range(world)])
        lib.call("elfa_zero3_gather", ctypes.addressof(src_pay), world, 0, pay_l, payload, stream)
        lib.call("elfa_zero3_gather", ctypes.addressof(src_sf), world, 0, sf_l, scales, stream)
        # 4. block-scaled GEMM on the gathered operand
        a_op = Mxfp8Operand(payload, scales, M, K, False)
        y = gemm_mxfp8(a_op, w_op, gelu=act == "gelu", preact=pre)
    # 5. bf16 copy of the gathered rows for the weight gradient, out of the ring on the side stream
    if st.side is None:
        st.side = torch.cuda.Stream(x_local.device)
    x_full = torch.empty((M, K), dtype=torch.bfloat16, device=x_local.device)
    cur = torch.cuda.current_stream()
    st.side.wait_stream(cur)
    with torch.cuda.stream(st.side):
        lib.call("elfa_mxfp8_dequantize", payload, scales, x_full, M, K, 0, st.side.cuda_stream)
        ev = torch.cuda.Event()
        ev.record(st.side)
    x_full.record_stream(st.side)
    st.pending = ev
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


def supported_rs_mxfp8(M: int, K: int, N: int, world: int) -> bool:
    return M % world == 0 and (M // world) % 128 == 0 and K % 32 == 0 and N % 64 == 0


def gemm_rs_mxfp8(a_op, w_op, pc: ParallelContext, max_ctas: int = 0) -> torch.Tensor:
    """``reduce_scatter_rows(a @ w^T)`` with MXFP8 operands (``a_op`` left operand ``[M, K]``, ``w_op`` right operand ``[N, K]``):
    the block-scaled product inside the fused GEMM → reduce-scatter kernel. Returns ``[M / world, N]`` bf16."""
    world, rank = pc.tp_size, pc.tp_rank
    M, K, N = a_op.rows, a_op.cols, w_op.rows
    st = _state(pc)
    cols = int(lib.raw("elfa_gemm_rs_slot_cols")(N))
    slot = st.next_slot("rs", _round_class(M * cols * 2))
    out = torch.empty((M // world, N), dtype=torch.bfloat16, device=a_op.payload.device)
    lib.call("elfa_gemm_rs_mxfp8", a_op.payload, a_op.scales, w_op.payload, w_op.scales, M, N, K, ctypes.addressof(slot.peer_data),
             ctypes.addressof(slot.peer_flags), slot.flags.tensor, ctypes.addressof(slot.arrivals), out, out.stride(0), rank, world,
             _WAIT_MS, max_ctas, stream_ptr(a_op.payload))
    return out


def xent_stats_exchange(logits2: torch.Tensor, targets1: torch.Tensor, pc: ParallelContext, rows: int, v_local: int, vocab_lo: int,
                        vocab_total: int) -> torch.Tensor:
    """Pass 1 of the vocabulary-parallel cross-entropy with the exchange inside the kernel: every rank's per-token statistics
    (max, sum-exp, target logit, sum of logits) are stored into its slot of every rank's ``[world, rows, 4]`` table with peer
    stores, then a signal barrier. Two tables alternate: a rank that is one loss ahead writes into the other one.
    Returns this rank's table (valid until the second call after this one)."""
    st = _state(pc)
    world, rank = pc.tp_size, pc.tp_rank
    slot = st.next_slot("xent", _round_class(world * rows * 16))
    stream = stream_ptr(logits2)
    lib.call("elfa_xent_stats_push", logits2, logits2.stride(0), targets1, ctypes.addressof(slot.peer_data), rank, world, rows, v_local,
             vocab_lo, vocab_total, stream)
    st.stream_barrier(stream)          # all ranks' stores have landed (the barrier's signal is a release after a system fence)
    return slot.data.view(torch.float32, (world, rows, 4))
