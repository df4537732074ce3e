"""Causal softmax attention over a fused qkv tensor.

``qkv`` is ``[S, B, 3, H, hd]`` (``seq_first=True``, the layout of the model's sequence-first
activations) or ``[B, S, 3, H, hd]``; the result is ``[S, B, H*hd]`` / ``[B, S, H*hd]``. Grouped-query
attention (``model.num_kv_heads < num_heads``; reference: ``src/util/config.zig:74,109,200``, sketch
``src/futhark/efla_kernels.fut:222-260``) takes ``[S, B, H + 2 * Hkv, hd]``; packed sequences
(``data.pack_sequences``; reference: ``src/data/dataset.zig:421``) pass the start of each token's document.
CUDA tensors run the tcgen05 kernels (forward keeps only O and the row log-sum-exp; backward
recomputes the probabilities); CPU tensors run the fp32 PyTorch formula.

reference: ``src/futhark/attention.fut:28-51`` (causal scaled-dot-product attention),
``:94-165`` (blocked attention with running max / log-sum-exp).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..native import lib, stream_ptr


def _split_heads(x: torch.Tensor, num_heads: Optional[int]):
    """``x [B, S, 3, H, hd]`` or ``[B, S, H + 2 * Hkv, hd]`` (``num_heads`` = H) → q ``[B, H, S, hd]``, k, v ``[B, Hkv, S, hd]``."""
    if x.dim() == 5:
        return tuple(x[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    H = num_heads
    Hkv = (x.shape[2] - H) // 2
    q, k, v = x[:, :, :H], x[:, :, H:H + Hkv], x[:, :, H + Hkv:]
    return q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3)


def attention_ref(qkv: torch.Tensor, causal: bool = True, seq_first: bool = True, scale: Optional[float] = None,
                  num_heads: Optional[int] = None, doc_start: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 reference. Returns the same layout/dtype as :func:`attention`. ``doc_start [B, S]``: first position of each
    token's document (packed sequences): a query sees the keys of its own document only."""
    x = qkv if not seq_first else qkv.transpose(0, 1)            # [B, S, ...]
    q, k, v = (t.float() for t in _split_heads(x, num_heads))
    B, H, S, hd = q.shape
    if k.shape[1] != H:                                            # grouped-query attention: repeat each key / value head
        k = k.repeat_interleave(H // k.shape[1], dim=1)
        v = v.repeat_interleave(H // v.shape[1], dim=1)
    sc = scale if scale is not None else 1.0 / math.sqrt(hd)
    s = (q @ k.transpose(-1, -2)) * sc
    if causal:
        mask = torch.ones(S, S, dtype=torch.bool, device=s.device).triu(1)
        s = s.masked_fill(mask, float("-inf"))
    if doc_start is not None:
        keys = torch.arange(S, device=s.device)
        before = keys[None, None, :] < doc_start.to(s.device)[:, :, None]       # [B, S(query), S(key)]
        s = s.masked_fill(before[:, None], float("-inf"))
    o = torch.softmax(s, -1) @ v                                   # [B, H, S, hd]
    o = o.permute(0, 2, 1, 3).reshape(B, S, H * hd)
    if seq_first:
        o = o.transpose(0, 1)
    return o.contiguous().to(qkv.dtype)


def _strides(qkv: torch.Tensor, seq_first: bool, num_heads: Optional[int] = None):
    """→ (S, B, H, Hkv, hd, stride_s, stride_b) of a fused tensor ``[.., .., 3, H, hd]`` or ``[.., .., H + 2 * Hkv, hd]``."""
    if qkv.dim() == 5:
        assert qkv.shape[2] == 3
        H, hd = qkv.shape[3], qkv.shape[4]
        Hkv = H
        assert qkv.stride(4) == 1 and qkv.stride(3) == hd and qkv.stride(2) == H * hd, "qkv: the last three dims must be packed"
    else:
        assert qkv.dim() == 4 and num_heads, "a 4-D fused tensor [.., .., H + 2 * Hkv, hd] needs num_heads"
        H, hd = num_heads, qkv.shape[3]
        Hkv = (qkv.shape[2] - H) // 2
        assert Hkv > 0 and H + 2 * Hkv == qkv.shape[2] and H % Hkv == 0, "heads must be [H query | Hkv key | Hkv value], H a multiple of Hkv"
        assert qkv.stride(3) == 1 and qkv.stride(2) == hd, "qkv: the last two dims must be packed"
    if seq_first:
        S, B = qkv.shape[0], qkv.shape[1]
        return S, B, H, Hkv, hd, qkv.stride(0), qkv.stride(1)
    B, S = qkv.shape[0], qkv.shape[1]
    return S, B, H, Hkv, hd, qkv.stride(1), qkv.stride(0)


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, causal, seq_first, scale, num_heads, doc_start):
        S, B, H, Hkv, hd, ss, sb = _strides(qkv, seq_first, num_heads)
        out = torch.empty((S, B, H * hd) if seq_first else (B, S, H * hd), dtype=qkv.dtype, device=qkv.device)
        oss, osb = (out.stride(0), out.stride(1)) if seq_first else (out.stride(1), out.stride(0))
        lse = torch.empty((B, H, S), dtype=torch.float32, device=qkv.device)
        lib.call("elfa_attention_fwd_ex", qkv, ss, sb, out, oss, osb, lse, S, B, H, Hkv, hd, float(scale), int(causal), doc_start,
                 stream_ptr(qkv))
        ctx.save_for_backward(qkv, out, lse)
        ctx.cfg = (causal, seq_first, scale, num_heads)
        ctx.doc_start = doc_start
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        causal, seq_first, scale, num_heads = ctx.cfg
        S, B, H, Hkv, hd, ss, sb = _strides(qkv, seq_first, num_heads)
        dout = dout.contiguous()
        dqkv = torch.empty_like(qkv)
        oss, osb = (out.stride(0), out.stride(1)) if seq_first else (out.stride(1), out.stride(0))
        dss, dsb = (dqkv.stride(0), dqkv.stride(1)) if seq_first else (dqkv.stride(1), dqkv.stride(0))
        delta = torch.empty((B, H, S), dtype=torch.float32, device=qkv.device)
        lib.call("elfa_attention_bwd_ex", qkv, ss, sb, out, dout, oss, osb, lse, delta, dqkv, dss, dsb, S, B, H, Hkv, hd, float(scale),
                 int(causal), ctx.doc_start, stream_ptr(qkv))
        return dqkv, None, None, None, None, None


def attention(qkv: torch.Tensor, causal: bool = True, seq_first: bool = True, scale: Optional[float] = None,
              num_heads: Optional[int] = None, doc_start: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``qkv``: ``[S, B, 3, H, hd]`` or, for grouped-query attention, ``[S, B, H + 2 * Hkv, hd]`` with ``num_heads = H``
    (``[B, S, ...]`` when not ``seq_first``). ``doc_start [B, S]`` int32: packed sequences (causal only)."""
    hd = qkv.shape[-1]
    sc = scale if scale is not None else 1.0 / math.sqrt(hd)
    if not qkv.is_cuda:
        return attention_ref(qkv, causal, seq_first, sc, num_heads, doc_start)
    assert qkv.dtype == torch.bfloat16, "attention: bf16 required on CUDA"
    if doc_start is not None:
        assert causal and doc_start.dtype == torch.int32 and doc_start.is_contiguous() and doc_start.is_cuda
    return _Attention.apply(qkv, causal, seq_first, sc, num_heads, doc_start)
