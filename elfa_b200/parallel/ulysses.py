"""All-to-all (head-scatter) context parallelism: the alternative to the ring for softmax attention.

Between attention layers every rank holds a contiguous block of the sequence with all heads; for the
attention itself one all-to-all turns that into the whole sequence with ``H / N`` heads, the ordinary
causal attention kernel runs unchanged, and a second all-to-all restores the sequence split. Two
all-to-alls of the activation size per layer instead of ``N - 1`` key / value hops, no load imbalance
under the causal mask, but the head count must be a multiple of the group size.

reference: ``src/runtime/nccl.zig:83,322-332`` (``ncclAlltoAll`` / ``NcclCollectives.alltoAll``: bound,
never called), ``src/futhark/efla_kernels.fut`` (sequence-parallel scatter / gather).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def _all_to_all(x: torch.Tensor, group) -> torch.Tensor:
    """``x [N, ...]``: slice ``i`` goes to rank ``i``; returns ``[N, ...]`` with slice ``i`` received from rank ``i``."""
    out = torch.empty_like(x)
    if x.is_cuda:
        dist.all_to_all_single(out, x.contiguous(), group=group)
    else:   # gloo has no all_to_all_single for every dtype: one scatter per source rank is equivalent
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        ranks = dist.get_process_group_ranks(group) if group is not None else list(range(world))
        xs = [t.contiguous() for t in x.unbind(0)]
        for src in range(world):
            dist.scatter(out[src], xs if src == rank else None, src=ranks[src], group=group)
    return out


class _SeqToHeads(torch.autograd.Function):
    """``[S_l, B, C, H, hd]`` (sequence split) -> ``[N * S_l, B, C, H / N, hd]`` (heads split); backward is the inverse."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return seq_to_heads(x, group)

    @staticmethod
    def backward(ctx, g):
        return heads_to_seq(g.contiguous(), ctx.group), None


class _HeadsToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return heads_to_seq(x, group)

    @staticmethod
    def backward(ctx, g):
        return seq_to_heads(g.contiguous(), ctx.group), None


def seq_to_heads(x: torch.Tensor, group=None) -> torch.Tensor:
    n = dist.get_world_size(group)
    sl, B, C, H, hd = x.shape
    assert H % n == 0, "all-to-all context parallelism: the head count must be a multiple of the group size"
    send = x.reshape(sl, B, C, n, H // n, hd).permute(3, 0, 1, 2, 4, 5).contiguous()     # [N(dest), S_l, B, C, H/N, hd]
    recv = _all_to_all(send, group)                                                    # [N(src = sequence block), ...]
    return recv.reshape(n * sl, B, C, H // n, hd)


def heads_to_seq(x: torch.Tensor, group=None) -> torch.Tensor:
    n = dist.get_world_size(group)
    S, B, C, hl, hd = x.shape
    sl = S // n
    send = x.reshape(n, sl, B, C, hl, hd).contiguous()                                    # slice i = sequence block of rank i
    recv = _all_to_all(send, group)                                                    # [N(src = head group), S_l, B, C, H/N, hd]
    return recv.permute(1, 2, 3, 0, 4, 5).reshape(sl, B, C, n * hl, hd)


def ulysses_attention(qkv_local: torch.Tensor, group=None, causal: bool = True, scale: Optional[float] = None) -> torch.Tensor:
    """``qkv_local [S_l, B, 3, H, hd]`` (this rank's sequence block, equal blocks in rank order) ->
    ``[S_l, B, H * hd]``, differentiable; equals attention over the whole sequence."""
    from ..ops.attention import attention
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    if world == 1:
        return attention(qkv_local, causal=causal, seq_first=True, scale=scale)
    sl, B, _, H, hd = qkv_local.shape
    full = _SeqToHeads.apply(qkv_local, group)                                         # [S, B, 3, H/N, hd]
    o = attention(full, causal=causal, seq_first=True, scale=scale)                    # [S, B, (H/N) * hd]
    o = o.reshape(world * sl, B, 1, H // world, hd)
    return _HeadsToSeq.apply(o, group).reshape(sl, B, H * hd)
