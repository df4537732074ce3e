"""Ring (context-parallel) causal attention: the sequence is split into contiguous blocks over a
process group, every rank keeps its query block and the key / value blocks travel round the ring.

Rank ``r`` holds tokens ``[r * S_l, (r + 1) * S_l)``. At step ``t`` it owns the key / value block of rank
``j = (r - t) mod N``; blocks with ``j > r`` lie entirely in the future of its queries and are skipped,
``j == r`` is the causal diagonal block and ``j < r`` is a full (unmasked) block (the zig-zag split of
:func:`block_schedule` gives every rank the same number of block products instead). Every block product
runs on the tcgen05 attention kernel (CUDA) and returns the block output with its row log-sum-exp; the
partial results are merged with the usual log-sum-exp rescaling, so the result equals attention over
the whole sequence. The exchange of step ``t + 1`` is started before the block of step ``t`` is
computed, so the transfer (NCCL send / receive on its own stream) overlaps the math.

Backward keeps the global output and log-sum-exp: with them the probabilities of any block are
``exp(s * scale - lse)`` without renormalisation, so the block backward kernel is the ordinary one. The
key / value block travels round the ring a second time together with its fp32 gradient accumulator
and is home after ``N`` exchanges.

reference: ``src/tensor/sharding.zig:224-287`` (``SequenceParallelConfig.use_ring_attention``: a flag
without a consumer), ``src/distributed/sequence_parallel.zig:130-159`` (``ringExchange``),
``src/futhark/attention.fut:94-165`` (blocked attention with running maximum / log-sum-exp).
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


# --------------------------------------------------------------------------- one block
def _lse_rows(lse: torch.Tensor) -> torch.Tensor:
    """``[B, H, S]`` -> ``[S, B, H, 1]`` (broadcasts over the head dimension of a ``[S, B, H, hd]`` tensor)."""
    return lse.permute(2, 0, 1).unsqueeze(-1)


def block_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Attention of one query block against one key / value block of the same length.
    ``q, k, v``: ``[S, B, H, hd]``. Returns ``(o [S, B, H, hd], lse [B, H, S] fp32, natural log)``."""
    S, B, H, hd = q.shape
    if q.is_cuda:
        from ..native import lib, stream_ptr
        assert q.dtype == torch.bfloat16, "ring attention: bf16 required on CUDA"
        qkv = torch.stack((q, k, v), dim=2)                                  # [S, B, 3, H, hd], packed
        out = torch.empty((S, B, H * hd), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
        lib.call("elfa_attention_fwd", qkv, qkv.stride(0), qkv.stride(1), out, out.stride(0), out.stride(1), lse,
                 S, B, H, hd, float(scale), int(causal), stream_ptr(qkv))
        return out.view(S, B, H, hd), lse
    s = torch.einsum("sbhd,tbhd->bhst", q.float(), k.float()) * scale
    if causal:
        s = s.masked_fill(torch.ones(S, S, dtype=torch.bool, device=s.device).triu(1), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)                                         # [B, H, S]
    o = torch.einsum("bhst,tbhd->sbhd", torch.exp(s - lse.unsqueeze(-1)), v.float())
    return o.to(q.dtype), lse


def block_backward(q, k, v, out, dout, lse, causal: bool, scale: float):
    """Gradients of one block given the GLOBAL output ``out`` and log-sum-exp ``lse`` of the query rows.
    Returns ``(dq, dk, dv)`` in fp32, each ``[S, B, H, hd]``."""
    S, B, H, hd = q.shape
    if q.is_cuda:
        from ..native import lib, stream_ptr
        qkv = torch.stack((q, k, v), dim=2)
        o2 = out.reshape(S, B, H * hd)
        do2 = dout.reshape(S, B, H * hd).contiguous()
        dqkv = torch.empty_like(qkv)
        delta = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
        lib.call("elfa_attention_bwd", qkv, qkv.stride(0), qkv.stride(1), o2, do2, o2.stride(0), o2.stride(1), lse, delta,
                 dqkv, dqkv.stride(0), dqkv.stride(1), S, B, H, hd, float(scale), int(causal), stream_ptr(qkv))
        return dqkv[:, :, 0].float(), dqkv[:, :, 1].float(), dqkv[:, :, 2].float()
    qf, kf, vf, of, dof = (t.float() for t in (q, k, v, out, dout))
    s = torch.einsum("sbhd,tbhd->bhst", qf, kf) * scale
    p = torch.exp(s - lse.unsqueeze(-1))
    if causal:
        p = p.masked_fill(torch.ones(S, S, dtype=torch.bool, device=s.device).triu(1), 0.0)
    dv = torch.einsum("bhst,sbhd->tbhd", p, dof)
    dp = torch.einsum("sbhd,tbhd->bhst", dof, vf)
    delta = (dof * of).sum(-1).permute(1, 2, 0)                              # [B, H, S]
    ds = p * (dp - delta.unsqueeze(-1)) * scale
    dq = torch.einsum("bhst,tbhd->sbhd", ds, kf)
    dk = torch.einsum("bhst,sbhd->tbhd", ds, qf)
    return dq, dk, dv


def merge_partial(o_acc: Optional[torch.Tensor], lse_acc: Optional[torch.Tensor], o_blk: torch.Tensor, lse_blk: torch.Tensor):
    """Combines two normalised partial attention results over disjoint key sets (fp32 accumulators)."""
    if o_acc is None:
        return o_blk.float(), lse_blk.clone()
    lse_new = torch.logaddexp(lse_acc, lse_blk)
    o = o_acc * torch.exp(_lse_rows(lse_acc - lse_new)) + o_blk.float() * torch.exp(_lse_rows(lse_blk - lse_new))
    return o, lse_new


# --------------------------------------------------------------------------- the ring
class _Exchange:
    """One hop of the ring in flight: the constructor posts the sends to the right neighbour and the receives
    from the left one, ``wait`` returns the received tensors. The sent tensors must stay untouched until then."""

    def __init__(self, tensors: List[torch.Tensor], group):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        ranks = dist.get_process_group_ranks(group) if group is not None else list(range(world))
        dst, src = ranks[(rank + 1) % world], ranks[(rank - 1) % world]
        self.out = [torch.empty_like(t) for t in tensors]
        ops = []
        for t, o in zip(tensors, self.out):
            ops.append(dist.P2POp(dist.isend, t, dst, group))
            ops.append(dist.P2POp(dist.irecv, o, src, group))
        self.work = dist.batch_isend_irecv(ops)

    def wait(self) -> List[torch.Tensor]:
        for w in self.work:
            w.wait()
        return self.out


def block_schedule(rank: int, j: int, causal: bool, zigzag: bool):
    """Block products rank ``rank`` owes to the key / value block of rank ``j``: ``(query part, key part, masked)``.

    Contiguous split: one part per rank; ``j > rank`` is all future (nothing), ``j == rank`` the masked diagonal.
    Zig-zag split (causal only): a rank holds two half blocks, chunk ``rank`` and chunk ``2N - 1 - rank`` of ``2N``
    chunks (parts 0 and 1). Part 0 of any rank lies before part 1 of every rank, so every step has two half-size
    products whatever ``j`` is (three on the diagonal, two of them masked): the work is the same on all ranks."""
    if not zigzag:
        if not causal:
            return [(0, 0, False)]
        return [(0, 0, j == rank)] if j <= rank else []
    if j == rank:
        return [(0, 0, True), (1, 0, False), (1, 1, True)]
    if j < rank:
        return [(0, 0, False), (1, 0, False)]
    return [(1, 0, False), (1, 1, False)]


class _RingAttention(torch.autograd.Function):
    """``q, k, v [S_l, B, H, hd]``; with ``zigzag`` the local sequence is two half blocks (see :func:`block_schedule`)."""

    @staticmethod
    def forward(ctx, q, k, v, group, scale, causal, zigzag):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        parts = 2 if zigzag else 1
        hl = q.shape[0] // parts
        kv = torch.stack((k, v), dim=0).contiguous()                       # travels as one message
        qs = [q[i * hl:(i + 1) * hl] for i in range(parts)]
        acc = [[None, None] for _ in range(parts)]                        # (o, lse) per query part
        for t in range(world):
            j = (rank - t) % world
            nxt = _Exchange([kv], group) if t + 1 < world else None          # overlaps the blocks below
            for qi, ki, masked in block_schedule(rank, j, causal, zigzag):
                o_blk, lse_blk = block_forward(qs[qi], kv[0, ki * hl:(ki + 1) * hl], kv[1, ki * hl:(ki + 1) * hl], masked, scale)
                acc[qi] = list(merge_partial(acc[qi][0], acc[qi][1], o_blk, lse_blk))
            if nxt is not None:
                kv = nxt.wait()[0]
        out = torch.cat([a[0] for a in acc], 0).to(q.dtype).contiguous()
        lse = torch.stack([a[1] for a in acc], 0)                          # [parts, B, H, hl]
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (group, scale, causal, zigzag)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        group, scale, causal, zigzag = ctx.cfg
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        parts = 2 if zigzag else 1
        hl = q.shape[0] // parts
        dout = dout.contiguous()
        kv = torch.stack((k, v), dim=0).contiguous()
        dkv = torch.zeros(kv.shape, dtype=torch.float32, device=kv.device)   # gradient of the block in hand
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        sl = [slice(i * hl, (i + 1) * hl) for i in range(parts)]
        for t in range(world):
            j = (rank - t) % world
            nxt = _Exchange([kv], group) if t + 1 < world else None          # the block itself can leave at once
            for qi, ki, masked in block_schedule(rank, j, causal, zigzag):
                dq_b, dk_b, dv_b = block_backward(q[sl[qi]], kv[0, sl[ki]], kv[1, sl[ki]], out[sl[qi]], dout[sl[qi]], lse[qi], masked, scale)
                dq[sl[qi]] += dq_b
                dkv[0, sl[ki]] += dk_b
                dkv[1, sl[ki]] += dv_b
            dkv = _Exchange([dkv], group).wait()[0]                           # after N hops the block is home
            if nxt is not None:
                kv = nxt.wait()[0]
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None, None, None


def zigzag_slices(seq_len: int, rank: int, world: int):
    """The two ``(start, stop)`` ranges of the sequence that rank ``rank`` holds under the zig-zag split."""
    hl = seq_len // (2 * world)
    return (rank * hl, (rank + 1) * hl), ((2 * world - 1 - rank) * hl, (2 * world - rank) * hl)


def ring_attention(qkv_local: torch.Tensor, group=None, causal: bool = True, seq_first: bool = True,
                   scale: Optional[float] = None, zigzag: bool = False) -> torch.Tensor:
    """Attention over a sequence split in equal contiguous blocks over ``group`` (rank order = token order), or with
    ``zigzag`` split in ``2N`` chunks of which this rank holds chunk ``rank`` followed by chunk ``2N - 1 - rank``
    (:func:`zigzag_slices`; causal only - it evens out the work that the causal mask leaves to each rank).
    ``qkv_local``: this rank's ``[S_l, B, 3, H, hd]`` (or ``[B, S_l, 3, H, hd]``); returns ``[S_l, B, H*hd]``
    (``[B, S_l, H*hd]``), differentiable. With a group of one it is :func:`elfa_b200.ops.attention`."""
    from ..ops.attention import attention
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    if world == 1:
        return attention(qkv_local, causal=causal, seq_first=seq_first, scale=scale)
    x = qkv_local if seq_first else qkv_local.transpose(0, 1)               # [S_l, B, 3, H, hd]
    S, B, _, H, hd = x.shape
    sc = scale if scale is not None else 1.0 / math.sqrt(hd)
    q, k, v = (x[:, :, i].contiguous() for i in range(3))
    assert not zigzag or (causal and S % 2 == 0), "the zig-zag split is for causal attention over two equal half blocks"
    o = _RingAttention.apply(q, k, v, group, sc, causal, zigzag).reshape(S, B, H * hd)
    return o if seq_first else o.transpose(0, 1).contiguous()


def ring_attention_emulated(qkv: torch.Tensor, world: int, causal: bool = True, scale: Optional[float] = None,
                            dout: Optional[torch.Tensor] = None):
    """The computation of :func:`ring_attention` for every rank of a ``world``-rank ring, run one rank after
    the other in this process (no communication): the same block kernels, the same merge and the same
    gradient accumulation. ``qkv``: the whole sequence ``[S, B, 3, H, hd]`` with ``S`` a multiple of
    ``world``. Returns ``out [S, B, H*hd]`` and, when ``dout`` is given, also ``dqkv``. It is how a single
    GPU checks the block kernels (non-causal blocks, external log-sum-exp in backward) against attention
    over the whole sequence."""
    S, B, _, H, hd = qkv.shape
    assert S % world == 0
    sl = S // world
    sc = scale if scale is not None else 1.0 / math.sqrt(hd)
    blk = [[qkv[r * sl:(r + 1) * sl, :, i].contiguous() for i in range(3)] for r in range(world)]
    outs, lses = [], []
    for r in range(world):
        o_acc = lse_acc = None
        for j in range(world):
            if causal and j > r:
                continue
            o_b, l_b = block_forward(blk[r][0], blk[j][1], blk[j][2], causal and j == r, sc)
            o_acc, lse_acc = merge_partial(o_acc, lse_acc, o_b, l_b)
        outs.append(o_acc.to(qkv.dtype).contiguous())
        lses.append(lse_acc)
    out = torch.cat(outs, 0).reshape(S, B, H * hd)
    if dout is None:
        return out
    dqkv = torch.zeros(qkv.shape, dtype=torch.float32, device=qkv.device)
    do = dout.reshape(S, B, H, hd)
    for r in range(world):
        for j in range(world):
            if causal and j > r:
                continue
            dq, dk, dv = block_backward(blk[r][0], blk[j][1], blk[j][2], outs[r], do[r * sl:(r + 1) * sl].contiguous(), lses[r],
                                        causal and j == r, sc)
            dqkv[r * sl:(r + 1) * sl, :, 0] += dq
            dqkv[j * sl:(j + 1) * sl, :, 1] += dk
            dqkv[j * sl:(j + 1) * sl, :, 2] += dv
    return out, dqkv.to(qkv.dtype)
