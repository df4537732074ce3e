"""Causal softmax attention over a fused qkv tensor.

``qkv`` is ``[S, B, 3, H, hd]`` (``seq_first=True``, the layout of the model's sequence-first
activations) or ``[B, S, 3, H, hd]``; the result is ``[S, B, H*hd]`` / ``[B, S, H*hd]``.
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


def attention_ref(qkv: torch.Tensor, causal: bool = True, seq_first: bool = True, scale: Optional[float] = None) -> torch.Tensor:
    """fp32 reference. Returns the same layout/dtype as :func:`attention`."""
    x = qkv if not seq_first else qkv.transpose(0, 1)            # [B, S, 3, H, hd]
    B, S, _, H, hd = x.shape
    q, k, v = (x[:, :, i].permute(0, 2, 1, 3).float() for i in range(3))   # [B, H, S, hd]
    sc = scale if scale is not None else 1.0 / math.sqrt(hd)
    s = (q @ k.transpose(-1, -2)) * sc
    if causal:
        mask = torch.ones(S, S, dtype=torch.bool, device=s.device).triu(1)
        s = s.masked_fill(mask, float("-inf"))
    o = torch.softmax(s, -1) @ v                                   # [B, H, S, hd]
    o = o.permute(0, 2, 1, 3).reshape(B, S, H * hd)
    if seq_first:
        o = o.transpose(0, 1)
    return o.contiguous().to(qkv.dtype)


def _strides(qkv: torch.Tensor, seq_first: bool):
    assert qkv.dim() == 5 and qkv.shape[2] == 3
    H, hd = qkv.shape[3], qkv.shape[4]
    assert qkv.stride(4) == 1 and qkv.stride(3) == hd and qkv.stride(2) == H * hd, "qkv: the last three dims must be packed"
    if seq_first:
        S, B = qkv.shape[0], qkv.shape[1]
        return S, B, H, hd, qkv.stride(0), qkv.stride(1)
    B, S = qkv.shape[0], qkv.shape[1]
    return S, B, H, hd, qkv.stride(1), qkv.stride(0)


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, causal, seq_first, scale):
        S, B, H, hd, ss, sb = _strides(qkv, seq_first)
        out = torch.empty((S, B, H * hd) if seq_first else (B, S, H * hd), dtype=qkv.dtype, device=qkv.device)
        oss, osb = (out.stride(0), out.stride(1)) if seq_first else (out.stride(1), out.stride(0))
        lse = torch.empty((B, H, S), dtype=torch.float32, device=qkv.device)
        lib.call("elfa_attention_fwd", qkv, ss, sb, out, oss, osb, lse, S, B, H, hd, float(scale), int(causal), stream_ptr(qkv))
        ctx.save_for_backward(qkv, out, lse)
        ctx.cfg = (causal, seq_first, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        causal, seq_first, scale = ctx.cfg
        S, B, H, hd, ss, sb = _strides(qkv, seq_first)
        dout = dout.contiguous()
        dqkv = torch.empty_like(qkv)
        oss, osb = (out.stride(0), out.stride(1)) if seq_first else (out.stride(1), out.stride(0))
        dss, dsb = (dqkv.stride(0), dqkv.stride(1)) if seq_first else (dqkv.stride(1), dqkv.stride(0))
        delta = torch.empty((B, H, S), dtype=torch.float32, device=qkv.device)
        lib.call("elfa_attention_bwd", qkv, ss, sb, out, dout, oss, osb, lse, delta, dqkv, dss, dsb, S, B, H, hd, float(scale),
                 int(causal), stream_ptr(qkv))
        return dqkv, None, None, None


def attention(qkv: torch.Tensor, causal: bool = True, seq_first: bool = True, scale: Optional[float] = None) -> torch.Tensor:
    hd = qkv.shape[-1]
    sc = scale if scale is not None else 1.0 / math.sqrt(hd)
    if not qkv.is_cuda:
        return attention_ref(qkv, causal, seq_first, sc)
    assert qkv.dtype == torch.bfloat16, "attention: bf16 required on CUDA"
    return _Attention.apply(qkv, causal, seq_first, sc)
