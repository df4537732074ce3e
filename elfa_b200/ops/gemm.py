"""GEMM and Linear.

``gemm`` is the raw call into the tcgen05 kernel; ``linear`` is the autograd function used by
every projection. Weights are stored ``[in, out]`` like the reference's ``Linear``
(reference: ``src/nn/layers.zig:322-431``; cuBLAS path ``kernels/cuda/gemm.cu:315-327,412-423,564``).

Operand conventions of the kernel: an operand is *K-major* when the contraction index is
contiguous (A ``[M,K]``, B ``[N,K]``) and *MN-major* when the output index is contiguous
(A ``[K,M]``, B ``[K,N]``). With ``W [in,out]``:

* forward   ``y[T,out] = x[T,in] @ W``      : A = x (K-major), B = W (MN-major)
* dgrad     ``dx[T,in] = dy[T,out] @ W^T``  : A = dy (K-major), B = W read as ``[N=in, K=out]`` (K-major)
* wgrad     ``dW[in,out] = x^T @ dy``       : A = x read as ``[K=T, M=in]`` (MN-major), B = dy (MN-major)

CPU tensors take the plain PyTorch path (the oracle of the tests).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import native
from ..native import (EPI_ACCUM, EPI_ADD_AUX, EPI_BIAS, EPI_DGELU_AUX, EPI_GELU, EPI_OUT_F32, EPI_STORE_PREACT, lib,
                      stream_ptr)

_GELU_K = 0.7978845608028654


def gelu_tanh_ref(x: torch.Tensor) -> torch.Tensor:
    return 0.5 * x * (1.0 + torch.tanh(_GELU_K * (x + 0.044715 * x * x * x)))


def dgelu_tanh_ref(x: torch.Tensor) -> torch.Tensor:
    u = _GELU_K * (x + 0.044715 * x * x * x)
    t = torch.tanh(u)
    return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * _GELU_K * (1 + 3 * 0.044715 * x * x)


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, out: Optional[torch.Tensor] = None,
         bias: Optional[torch.Tensor] = None, aux: Optional[torch.Tensor] = None, preact: Optional[torch.Tensor] = None,
         gelu: bool = False, dgelu_aux: bool = False, add_aux: bool = False, accumulate: bool = False,
         out_dtype: torch.dtype = torch.bfloat16, alpha: float = 1.0, force_bn: int = 0, max_ctas: int = 0, staged: bool = False) -> torch.Tensor:
    """``out[M,N] = epilogue(alpha * op(a) @ op(b))`` on the tcgen05 kernel (bf16 operands).

    ``a`` is ``[M,K]`` (or ``[K,M]`` when ``a_mn``), ``b`` is ``[N,K]`` (or ``[K,N]`` when ``b_mn``);
    both must be 2-D with a contiguous last dimension. Epilogue order: ``+bias`` → store ``preact`` →
    GELU → ``*gelu'(aux)`` or ``+aux`` → ``+out`` (accumulate) → store.
    """
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    assert K == Kb, f"gemm: contraction mismatch {K} vs {Kb}"
    if not a.is_cuda:
        af = (a.t() if a_mn else a).float()
        bf = (b if b_mn else b.t()).float()
        r = alpha * (af @ bf)
        if bias is not None:
            r = r + bias.float()
        if preact is not None:
            preact.copy_(r.to(preact.dtype))
        if gelu:
            r = gelu_tanh_ref(r)
        if dgelu_aux:
            r = r * dgelu_tanh_ref(aux.float())
        elif add_aux:
            r = r + aux.float()
        if out is None:
            return r.to(out_dtype if a.dtype == torch.bfloat16 else a.dtype)
        if accumulate:
            r = r + out.float()
        out.copy_(r.to(out.dtype))
        return out
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "gemm: bf16 operands required on CUDA"
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        assert not accumulate
    assert out.dim() == 2 and out.shape == (M, N) and out.stride(1) == 1
    flags = 0
    if bias is not None:
        flags |= EPI_BIAS
    if gelu:
        flags |= EPI_GELU
    if dgelu_aux:
        flags |= EPI_DGELU_AUX
    if add_aux:
        flags |= EPI_ADD_AUX
    if accumulate:
        flags |= EPI_ACCUM
    if out.dtype == torch.float32:
        flags |= EPI_OUT_F32
    else:
        assert out.dtype == torch.bfloat16
    if preact is not None:
        flags |= EPI_STORE_PREACT
    if staged:
        flags |= 128            # ELFA_EPI_STAGED: shared-memory + TMA-store epilogue (what the fused reduce-scatter kernel uses)
    if aux is not None:
        assert aux.dtype == torch.bfloat16 and aux.shape == (M, N) and aux.stride(1) == 1
    lib.call("elfa_gemm_bf16", a, b, out, M, N, K, a.stride(0), b.stride(0), out.stride(0), int(a_mn), int(b_mn), bias, aux,
             aux.stride(0) if aux is not None else 0, preact, preact.stride(0) if preact is not None else 0, float(alpha),
             flags, force_bn, max_ctas, stream_ptr(a))
    return out


def _accumulate_main_grad(w: torch.Tensor, x2: torch.Tensor, dy2: torch.Tensor) -> bool:
    """Writes ``x2^T @ dy2`` straight into ``w.main_grad`` (fp32, owned by the optimizer's flat
    gradient buffer) and returns True; returns False when the parameter has no such buffer."""
    mg = getattr(w, "main_grad", None)
    if mg is None:
        return False
    fresh = getattr(w, "_grad_fresh", False)
    gemm(x2, dy2, a_mn=True, b_mn=True, out=mg, accumulate=not fresh)
    w._grad_fresh = False
    return True


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, act):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        pre = None
        fetch = getattr(w, "_gemm_gather", None)     # ZeRO stage 3: this product fetches the parameter itself (parallel/zero3.py)
        if fetch is not None and bias is None and act in (None, "gelu") and fetch.pending(w):
            if act == "gelu":
                pre = torch.empty((x2.shape[0], w.shape[1]), dtype=x2.dtype, device=x2.device)
            y = fetch.gemm(x2, w, act == "gelu", pre)
        elif act == "gelu":
            pre = torch.empty((x2.shape[0], w.shape[1]), dtype=x2.dtype, device=x2.device)
            y = gemm(x2, w, b_mn=True, bias=bias, gelu=True, preact=pre, out_dtype=x2.dtype)
        else:
            y = gemm(x2, w, b_mn=True, bias=bias, out_dtype=x2.dtype)
        ctx.save_for_backward(x2, w, pre)
        ctx.has_bias = bias is not None
        ctx.w_ref = w
        ctx.in_shape = x.shape
        return y.reshape(*x.shape[:-1], w.shape[1])

    @staticmethod
    def backward(ctx, dy):
        x2, w, pre = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if pre is not None:
            if dy2.is_cuda:
                dpre = torch.empty_like(dy2)
                lib.call("elfa_elementwise", 1, pre, dy2, dpre, dy2.numel(), 1.0, stream_ptr(dy2))
                dy2 = dpre
            else:
                dy2 = (dy2.float() * dgelu_tanh_ref(pre.float())).to(dy2.dtype)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, out_dtype=dy2.dtype).reshape(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            if not (dy2.is_cuda and _accumulate_main_grad(ctx.w_ref, x2, dy2)):
                dw = gemm(x2, dy2, a_mn=True, b_mn=True, out_dtype=w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy2.dtype)
        return dx, dw, db, None


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: Optional[str] = None) -> torch.Tensor:
    """``act(x @ w + bias)`` with ``w [in, out]``; ``act`` is ``None`` or ``"gelu"`` (tanh form,
    fused into the GEMM epilogue; the pre-activation is kept for backward)."""
    return _Linear.apply(x, w, bias, act)


class _LinearNT(torch.autograd.Function):
    """``x @ w^T`` with ``w [out, in]`` - the tied-embedding vocabulary projection
    (reference: ``src/model/model.zig:587-631`` forward, ``:678-760`` backward, both host loops)."""

    @staticmethod
    def forward(ctx, x, w):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        ctx.save_for_backward(x2, w)
        ctx.w_ref = w
        ctx.in_shape = x.shape
        return gemm(x2, w, out_dtype=x2.dtype).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True, out_dtype=dy2.dtype).reshape(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.w_ref, "main_grad", None)
            if dy2.is_cuda and mg is not None:
                fresh = getattr(ctx.w_ref, "_grad_fresh", False)
                gemm(dy2, x2, a_mn=True, b_mn=True, out=mg, accumulate=not fresh)
                ctx.w_ref._grad_fresh = False
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=w.dtype)
        return dx, dw


def linear_nt(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return _LinearNT.apply(x, w)
