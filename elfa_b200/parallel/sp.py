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

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .descriptors import ShardSpec


def split_sequence(x: torch.Tensor, rank: int, world: int, dim: int = 1) -> torch.Tensor:
    """This rank's contiguous block of the sequence dimension (remainder-aware)."""
    s = ShardSpec(dim, world, rank)
    n = x.shape[dim]
    return x.narrow(dim, s.offset(n), s.local_size(n)).contiguous()


def gather_sequence(x_local: torch.Tensor, group=None, dim: int = 1) -> torch.Tensor:
    world = dist.get_world_size(group)
    sizes = [torch.zeros(1, dtype=torch.int64, device=x_local.device) for _ in range(world)]
    dist.all_gather(sizes, torch.tensor([x_local.shape[dim]], dtype=torch.int64, device=x_local.device), group=group)
    parts = []
    for s in sizes:
        shp = list(x_local.shape)
        shp[dim] = int(s)
        parts.append(torch.empty(shp, dtype=x_local.dtype, device=x_local.device))
    dist.all_gather(parts, x_local.contiguous(), group=group) if len({p.shape for p in parts}) == 1 else _uneven_all_gather(parts, x_local, group)
    return torch.cat(parts, dim=dim)


def _uneven_all_gather(parts, x_local, group):
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    ranks = dist.get_process_group_ranks(group) if group is not None else list(range(world))
    for r in range(world):
        if r == rank:
            parts[r].copy_(x_local)
        dist.broadcast(parts[r], src=ranks[r], group=group)


def ring_exchange(x: torch.Tensor, step: int = 1, group=None) -> torch.Tensor:
    """Sends ``x`` to rank ``(r + step) % N`` and returns the tensor received from ``(r - step) % N``."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    if world == 1:
        return x.clone()
    ranks = dist.get_process_group_ranks(group) if group is not None else list(range(world))
    dst, src = ranks[(rank + step) % world], ranks[(rank - step) % world]
    out = torch.empty_like(x)
    ops = [dist.P2POp(dist.isend, x.contiguous(), dst, group), dist.P2POp(dist.irecv, out, src, group)]
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    return out


def halo_from_left(x_local: torch.Tensor, width: int, group=None, dim: int = 1) -> torch.Tensor:
    """The last ``width`` positions of the left neighbour's block (zeros on rank 0): what a causal
    convolution of window ``width + 1`` needs in front of the local block."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    tail = x_local.narrow(dim, x_local.shape[dim] - width, width).contiguous()
    if world == 1:
        return torch.zeros_like(tail)
    recv = ring_exchange(tail, 1, group)
    if rank == 0:
        recv.zero_()
    return recv


def efla_cross_rank_state(k_local: torch.Tensor, v_local: torch.Tensor, beta: torch.Tensor, group=None) -> torch.Tensor:
    """The true EFLA state at the start of this rank's token block when the sequence is split over
    the group: every rank reduces its block to the affine map ``(A_r, B_r)``, the maps are gathered
    (``2 * H * d * d`` numbers per rank) and composed in rank order. Returns ``S_in [B, H, d, d]``."""
    from ..ops.efla import chunk_affine_map
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    A, Bm = chunk_affine_map(k_local, v_local, beta)
    if world == 1:
        return torch.zeros_like(Bm)
    allA = [torch.empty_like(A) for _ in range(world)]
    allB = [torch.empty_like(Bm) for _ in range(world)]
    dist.all_gather(allA, A.contiguous(), group=group)
    dist.all_gather(allB, Bm.contiguous(), group=group)
    S = torch.zeros_like(Bm)
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
