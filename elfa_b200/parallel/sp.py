"""Sequence / context parallel primitives: split, gather, ring exchange, halo exchange and the exact
cross-rank composition of the EFLA state.

reference: ``src/distributed/sequence_parallel.zig:54-77`` (``splitSequence`` contiguous token blocks),
``:79-128`` (``gatherSequence``), ``:130-159`` (``ringExchange(step)``: send to ``(r + step) % N``, receive
from ``(r - step) % N``), ``:184-200`` (``reduceScatterGradients``), ``:202-240`` (``syncCrossBoundary``: a
halo of ``boundary x hidden`` values for the neighbour). The reference has no consumer for the ring
and combines chunk states by addition; here the halo feeds ShortConv and the EFLA state crosses ranks
as an affine map ``S_out = A S_in + B`` (see ``ops/efla.py``), which is exact for the delta rule.

All functions work on any ``torch.distributed`` backend (NCCL on GPUs, gloo on CPU).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .descriptors import ShardSpec


def split_sequence(x: torch.Tensor, rank: int, world: int, dim: int = 1) -> torch.Tensor:
    """This rank's contiguous block of the sequence dimension (remainder-aware)."""
    s = ShardSpec(dim, world, rank)
    n = x.shape[dim]
    return x.narrow(dim, s.offset(n), s.local_size(n)).contiguous()


def gather_sequence(x_local: torch.Tensor, group=None, dim: int = 1) -> torch.Tensor:
    """Concatenation of every rank's block along ``dim`` (blocks may differ in length by one)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    n_local = torch.tensor([x_local.shape[dim]], dtype=torch.int64, device=x_local.device)
    sizes = [torch.zeros_like(n_local) for _ in range(world)]
    dist.all_gather(sizes, n_local, group=group)
    parts = []
    for s in sizes:
        shp = list(x_local.shape)
        shp[dim] = int(s)
        parts.append(torch.empty(shp, dtype=x_local.dtype, device=x_local.device))
    if len({p.shape for p in parts}) == 1:
        dist.all_gather(parts, x_local.contiguous(), group=group)
    else:
        # uneven blocks: one broadcast per rank
        ranks = dist.get_process_group_ranks(group) if group is not None else list(range(world))
        for r in range(world):
            if r == rank:
                parts[r].copy_(x_local)
            dist.broadcast(parts[r], src=ranks[r], group=group)
    return torch.cat(parts, dim=dim)


_MAILBOXES = {}      # (id(group), step) -> PeerMailbox: neighbour hand-offs that go over NVLink peer memory


def register_mailboxes(group, arena, nbytes: int) -> None:
    """Routes the neighbour exchanges of ``group`` (``ring_exchange`` with step +1 / -1 on CUDA tensors of at most ``nbytes``)
    through peer-memory mailboxes in ``arena`` (write-then-flag over NVLink) instead of library send / receive. Collective."""
    _MAILBOXES[(id(group), 1)] = PeerMailbox(arena, nbytes, "sp.mailbox.right", direction=1)
    _MAILBOXES[(id(group), -1)] = PeerMailbox(arena, nbytes, "sp.mailbox.left", direction=-1)


def ring_exchange(x: torch.Tensor, step: int = 1, group=None) -> torch.Tensor:
    """Sends ``x`` to rank ``(r + step) % N`` and returns the tensor received from ``(r - step) % N``."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    if world == 1:
        return x.clone()
    box = _MAILBOXES.get((id(group), step)) if x.is_cuda else None
    if box is not None and x.numel() * x.element_size() <= box.nbytes and (x.numel() * x.element_size()) % 16 == 0:
        return ring_exchange_peer(x, box)
    ranks = dist.get_process_group_ranks(group) if group is not None else list(range(world))
    dst, src = ranks[(rank + step) % world], ranks[(rank - step) % world]
    out = torch.empty_like(x)
    ops = [dist.P2POp(dist.isend, x.contiguous(), dst, group), dist.P2POp(dist.irecv, out, src, group)]
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    return out


class _HaloFromLeft(torch.autograd.Function):
    """Forward: every rank sends the tail of its block to the right neighbour. Backward: the gradient of what a rank
    received travels back to the left neighbour and is added to the gradient of that neighbour's tail."""

    @staticmethod
    def forward(ctx, x_local, width, group, dim):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        ctx.cfg = (width, group, dim, rank, world, x_local.shape[dim])
        tail = x_local.narrow(dim, x_local.shape[dim] - width, width).contiguous()
        if world == 1:
            return torch.zeros_like(tail)
        recv = ring_exchange(tail, 1, group)
        if rank == 0:
            recv.zero_()
        return recv

    @staticmethod
    def backward(ctx, g):
        width, group, dim, rank, world, n = ctx.cfg
        g = g.contiguous()
        dx_tail = torch.zeros_like(g)
        if world > 1:
            if rank == 0:
                g = torch.zeros_like(g)           # rank 0 received nothing it used
            dx_tail = ring_exchange(g, -1, group)  # what the right neighbour's halo contributed, sent back
            if rank == world - 1:
                dx_tail.zero_()                    # nobody read the last rank's tail
        shape = list(g.shape)
        shape[dim] = n
        dx = torch.zeros(shape, dtype=g.dtype, device=g.device)
        dx.narrow(dim, n - width, width).copy_(dx_tail)
        return dx, None, None, None


def halo_from_left(x_local: torch.Tensor, width: int, group=None, dim: int = 1) -> torch.Tensor:
    """The last ``width`` positions of the left neighbour's block (zeros on rank 0): what a causal
    convolution of window ``width + 1`` needs in front of the local block. Differentiable: in backward the halo's
    gradient returns to the neighbour it came from (reference: ``src/distributed/sequence_parallel.zig:202-240``
    ``syncCrossBoundary``, forward only there)."""
    return _HaloFromLeft.apply(x_local, width, group, dim)


class _GatherStack(torch.autograd.Function):
    """``x`` (same shape on every rank) → ``[world, *x.shape]``; backward sums the ranks' gradients of slice r on rank r."""

    @staticmethod
    def forward(ctx, x, group):
        world = dist.get_world_size(group)
        ctx.group = group
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.stack(parts, 0)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        return g[dist.get_rank(ctx.group)], None


def efla_cross_rank_state(k_local: torch.Tensor, v_local: torch.Tensor, beta: torch.Tensor, group=None) -> torch.Tensor:
    """The true EFLA state at the start of this rank's token block when the sequence is split over
    the group: every rank reduces its block to the affine map ``(A_r, B_r)``, the maps are gathered
    (``2 * H * d * d`` numbers per rank) and composed in rank order. Returns ``S_in [B, H, d, d]``.
    Differentiable end to end (the maps come out of the scan, whose backward accepts a final-state gradient; the gather's
    backward returns every map's gradient to the rank that owns it), so a sequence-parallel run trains exactly like a
    single rank on the whole sequence (reference: ``src/distributed/sequence_parallel.zig:130-159`` ring exchange of
    activations; the reference has no state hand-off and no backward through it)."""
    from ..ops.efla import chunk_affine_map
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    A, Bm = chunk_affine_map(k_local, v_local, beta)
    if world == 1:
        return torch.zeros_like(Bm)
    allA = _GatherStack.apply(A, group)
    allB = _GatherStack.apply(Bm, group)
    # every rank's result depends (with weight zero where nothing else does) on the gathered maps, so that every rank runs
    # the gather's backward collective: rank 0 composes nothing and would otherwise skip it
    S = torch.zeros_like(Bm) + 0.0 * (allA.sum() + allB.sum())
    for r in range(rank):
        S = allA[r] @ S + allB[r]
    return S


def reduce_scatter_gradients(g: torch.Tensor, group=None) -> torch.Tensor:
    """Sum over the group, each rank keeps its contiguous 1/N of dim 0."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    n = g.shape[0] // world
    if g.is_cuda:
        out = torch.empty((n, *g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(out, g.contiguous(), group=group)
        return out
    g = g.contiguous().clone()
    dist.all_reduce(g, group=group)
    return g[rank * n:(rank + 1) * n].clone()


class PeerMailbox:
    """Write-then-flag hand-off to the right neighbour of a ring over NVLink peer memory (GPU only).

    Every rank owns a two-slot mailbox and two counters in the group's symmetric arena: ``arrivals``
    (raised by the left neighbour after its stores) and ``acks`` (raised by the right neighbour after it
    has copied a message out). ``send`` waits (bounded) until the slot it is about to overwrite was
    acknowledged, stores into the neighbour's slot and raises the neighbour's arrival counter;
    ``recv`` waits (bounded) for the arrival, copies the slot out and acknowledges to the left.
    All waits are kernels on the current stream: nothing blocks the host.

    reference: ``src/distributed/sequence_parallel.zig:130-159`` (``ringExchange``), ``:202-240``
    (``syncCrossBoundary``) - grouped NCCL send / receive there.
    """

    def __init__(self, arena, nbytes: int, name: str = "sp.mailbox", direction: int = 1):
        """``direction`` +1: messages travel to the right neighbour (rank + 1); -1: to the left one."""
        import ctypes
        self.arena = arena
        self.nbytes = (nbytes + 15) // 16 * 16
        self.rank, self.world = arena.rank, arena.world
        self.data = arena.alloc(2 * self.nbytes, name + ".data")
        self.flags = arena.alloc(1024, name + ".flags")          # u32[0] arrivals, u32[64] acks (separate cache lines)
        self.right, self.left = (self.rank + direction) % self.world, (self.rank - direction) % self.world
        self._scratch = torch.zeros(4, dtype=torch.int32, device=arena.device)   # 16-byte payload of an acknowledgement
        self._ack_sink = arena.alloc(1024, name + ".acksink")
        self._blocks = ctypes.c_int(0)
        self.sent = 0                     # messages sent to the right
        self.received = 0                 # messages received from the left
        self.arrivals_expected = 0        # running total of arrival-counter increments expected on this rank
        self.acks_expected_blocks = 0
        arena.barrier()

    def _blocks_for(self, nbytes: int) -> int:
        return min(64, (nbytes // 16 + 255) // 256)

    def send(self, t: torch.Tensor) -> None:
        from ..native import lib, stream_ptr
        import ctypes
        src = t.contiguous().view(torch.uint8).reshape(-1)
        n = src.numel()
        assert n <= self.nbytes and n % 16 == 0, "message does not fit the mailbox (sizes are multiples of 16 bytes)"
        st = stream_ptr(src)
        slot = self.sent % 2
        if self.sent >= 2:
            # the message two sends ago used this slot: one acknowledgement per consumed message
            lib.call("elfa_p2p_wait", self.flags.tensor[256:], self.sent - 1, 0, st)
        dst = self.arena.peer_address(self.right, self.data) + slot * self.nbytes
        cnt = self.arena.peer_address(self.right, self.flags)
        lib.call("elfa_p2p_send", src, dst, n, cnt, ctypes.addressof(self._blocks), st)
        self.sent += 1
        self._last_blocks = self._blocks.value

    def recv(self, out: torch.Tensor) -> torch.Tensor:
        from ..native import lib, stream_ptr
        import ctypes
        n = out.numel() * out.element_size()
        st = stream_ptr(out)
        self.arrivals_expected += self._blocks_for(n)
        lib.call("elfa_p2p_wait", self.flags.tensor, self.arrivals_expected, 0, st)
        slot = self.received % 2
        out.view(torch.uint8).reshape(-1).copy_(self.data.tensor[slot * self.nbytes: slot * self.nbytes + n])
        self.received += 1
        # acknowledge: a 16-byte store into the left neighbour's sink raises its ack counter by one block
        sink = self.arena.peer_address(self.left, self._ack_sink)
        ack = self.arena.peer_address(self.left, self.flags) + 256
        lib.call("elfa_p2p_send", self._scratch, sink, 16, ack, ctypes.addressof(self._blocks), st)
        return out


def ring_exchange_peer(x: torch.Tensor, box: "PeerMailbox") -> torch.Tensor:
    """``ring_exchange(x, 1)`` through a :class:`PeerMailbox` (every rank sends right and receives from the left)."""
    box.send(x)
    return box.recv(torch.empty_like(x))
