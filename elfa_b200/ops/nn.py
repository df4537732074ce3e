"""Normalisation, activation, embedding and cross-entropy ops.

Each op is a ``torch.autograd.Function`` whose CUDA branch calls the native kernels and whose CPU
branch is the plain PyTorch formula (the oracle the GPU tests compare against).

reference math: ``src/nn/layers.zig:60-135`` (RMSNorm, eps 1e-6), ``:180-271`` (LayerNorm, eps 1e-5),
``:316-319`` (GELU), ``:459-501`` (embedding), ``src/kernels/nn_kernels.zig:269-318`` (cross-entropy
with label smoothing).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..native import lib, stream_ptr
from .gemm import gelu_tanh_ref

LAYERNORM, RMSNORM = 0, 1


def _grad_target(p: torch.Tensor):
    """(buffer, is_fp32, accumulate) for a parameter that owns a ``main_grad`` view, else None."""
    mg = getattr(p, "main_grad", None)
    if mg is None:
        return None
    fresh = getattr(p, "_grad_fresh", False)
    p._grad_fresh = False
    return mg, not fresh


# ------------------------------------------------------------------------------------------ norms
def norm_ref(x, w, b, eps, kind, residual=None):
    xf = x.float()
    if residual is not None:
        xf = (xf + residual.float()).to(x.dtype).float()
    if kind == RMSNORM:
        r = torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps)
        y = xf * r * w.float()
    else:
        mu = xf.mean(-1, keepdim=True)
        var = ((xf * xf).mean(-1, keepdim=True) - mu * mu).clamp_min(0)
        y = (xf - mu) * torch.rsqrt(var + eps) * w.float()
        if b is not None:
            y = y + b.float()
    return y.to(x.dtype), (xf.to(x.dtype) if residual is not None else None)


_scratch = {}


def _norm_scratch(device, n_floats: int) -> torch.Tensor:
    buf = _scratch.get(device)
    if buf is None or buf.numel() < n_floats:
        buf = torch.empty(max(n_floats, 1 << 20), dtype=torch.float32, device=device)
        _scratch[device] = buf
    return buf


class _Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, residual, eps, kind):
        D = x.shape[-1]
        x2 = x.reshape(-1, D)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        ctx.kind, ctx.shape, ctx.has_res, ctx.has_b = kind, x.shape, residual is not None, b is not None
        ctx.w_ref, ctx.b_ref = w, b
        if not x2.is_cuda:
            with torch.enable_grad():
                xin = x2.detach().requires_grad_(True)
                rin = residual.reshape(-1, D).detach().requires_grad_(True) if residual is not None else None
                win = w.detach().requires_grad_(True)
                bin_ = b.detach().requires_grad_(True) if b is not None else None
                y, s = norm_ref(xin, win, bin_, eps, kind, rin)
            ctx.cpu_graph = (xin, rin, win, bin_, y, s)
            ctx.save_for_backward()
            ys = y.detach().reshape(x.shape)
            if residual is not None:
                return ys, s.detach().reshape(x.shape)
            return ys
        y = torch.empty_like(x2)
        s = torch.empty_like(x2) if residual is not None else None
        mean = torch.empty(rows, dtype=torch.float32, device=x.device) if kind == LAYERNORM else None
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        r2 = residual.reshape(-1, D).contiguous() if residual is not None else None
        lib.call("elfa_norm_fwd", x2, r2, w, b, y, s, mean, rstd, rows, D, float(eps), kind, stream_ptr(x2))
        xin = s if s is not None else x2
        ctx.save_for_backward(xin, w, mean, rstd)
        if s is not None:
            return y.reshape(x.shape), s.reshape(x.shape)
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy, dsum=None):
        D = ctx.shape[-1]
        if not dy.is_cuda:
            xin, rin, win, bin_, y, s = ctx.cpu_graph
            outs, gouts = [y], [dy.reshape(y.shape)]
            if s is not None and dsum is not None:
                outs.append(s)
                gouts.append(dsum.reshape(s.shape))
            ins = [t for t in (xin, rin, win, bin_) if t is not None]
            gs = list(torch.autograd.grad(outs, ins, gouts, allow_unused=True))
            gx = gs.pop(0)
            gr = gs.pop(0) if rin is not None else None
            gw = gs.pop(0)
            gb = gs.pop(0) if bin_ is not None else None
            gx = gx.reshape(ctx.shape)
            if rin is None and dsum is not None:
                gx = gx + dsum
            return gx, gw, gb, (gr.reshape(ctx.shape) if gr is not None else None), None, None
        xin, w, mean, rstd = ctx.saved_tensors
        rows = xin.shape[0]
        dy2 = dy.reshape(-1, D)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres = None
        if dsum is not None:
            dres = dsum.reshape(-1, D)
            if not dres.is_contiguous():
                dres = dres.contiguous()
        dx = torch.empty_like(xin)
        P = lib.raw("elfa_norm_bwd_partials")(rows, D)
        scratch = _norm_scratch(xin.device, 2 * P * D)
        tw = _grad_target(ctx.w_ref)
        tb = _grad_target(ctx.b_ref) if ctx.has_b else None
        dw_ret = db_ret = None
        if tw is not None and (tb is not None or not ctx.has_b) and (tb is None or tb[1] == tw[1]):
            dwb, acc = tw
            dbb = tb[0] if tb is not None else None
            lib.call("elfa_norm_bwd", dy2, xin, w, mean, rstd, dres, dx, dwb, dbb, scratch, rows, D, ctx.kind, 1, int(acc),
                     stream_ptr(xin))
        else:
            dw_ret = torch.empty(D, dtype=torch.float32, device=xin.device)
            db_ret = torch.empty(D, dtype=torch.float32, device=xin.device) if ctx.has_b else None
            lib.call("elfa_norm_bwd", dy2, xin, w, mean, rstd, dres, dx, dw_ret, db_ret, scratch, rows, D, ctx.kind, 1, 0,
                     stream_ptr(xin))
            dw_ret = dw_ret.to(w.dtype)
            db_ret = db_ret.to(w.dtype) if db_ret is not None else None
        dx = dx.reshape(ctx.shape)
        # dx already contains dsum (added in the kernel); with a fused residual both inputs get it
        return dx, dw_ret, db_ret, (dx if ctx.has_res else None), None, None


def norm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None, *, eps: float, kind: int,
         residual: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(norm(x + residual) * w + b, x + residual)``; the second value is the updated
    residual stream (``x`` itself when ``residual`` is None)."""
    if residual is None:
        return _Norm.apply(x, w, b, None, eps, kind), x
    return _Norm.apply(x, w, b, residual, eps, kind)


def layer_norm(x, w, b=None, eps: float = 1e-5, residual=None):
    return norm(x, w, b, eps=eps, kind=LAYERNORM, residual=residual)


def rms_norm(x, w, eps: float = 1e-6, residual=None):
    return norm(x, w, None, eps=eps, kind=RMSNORM, residual=residual)


# -------------------------------------------------------------------------------------- activations
_EW = {"gelu": (0, 1), "silu": (4, 5), "relu": (6, 7), "gelu_erf": (8, 9)}


def _act_ref(name, x):
    if name == "gelu":
        return gelu_tanh_ref(x)
    if name == "silu":
        return x * torch.sigmoid(x)
    if name == "relu":
        return torch.relu(x)
    if name == "gelu_erf":
        return 0.5 * x * (1 + torch.erf(x * 0.7071067811865476))
    raise ValueError(name)


class _Act(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, name):
        ctx.name = name
        ctx.save_for_backward(x)
        if not x.is_cuda:
            return _act_ref(name, x.float()).to(x.dtype)
        xc = x.contiguous()
        y = torch.empty_like(xc)
        lib.call("elfa_elementwise", _EW[name][0], xc, None, y, xc.numel(), 1.0, stream_ptr(xc))
        return y

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        if not x.is_cuda:
            with torch.enable_grad():
                xi = x.detach().float().requires_grad_(True)
                y = _act_ref(ctx.name, xi)
            (g,) = torch.autograd.grad(y, xi, dy.float())
            return g.to(x.dtype), None
        xc, dyc = x.contiguous(), dy.contiguous()
        dx = torch.empty_like(xc)
        lib.call("elfa_elementwise", _EW[ctx.name][1], xc, dyc, dx, xc.numel(), 1.0, stream_ptr(xc))
        return dx, None


def activation(x: torch.Tensor, name: str = "gelu") -> torch.Tensor:
    return _Act.apply(x, name)


def gelu(x):
    return _Act.apply(x, "gelu")


# ---------------------------------------------------------------------------------------- embedding
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, tok, pos, pos0, vocab_lo, seq_first, vocab_total):
        if seq_first:
            T, B = ids.shape
        else:
            B, T = ids.shape
        D = tok.shape[1]
        ctx.args = (B, T, D, pos0, vocab_lo, tok.shape[0], pos is not None, seq_first)
        ctx.tok_ref, ctx.pos_ref = tok, pos
        ctx.save_for_backward(ids)
        if not tok.is_cuda:
            local = ids - vocab_lo
            mask = (local >= 0) & (local < tok.shape[0])
            out = tok[local.clamp(0, tok.shape[0] - 1)] * mask.unsqueeze(-1).to(tok.dtype)
            if pos is not None and vocab_lo == 0:
                out = out + pos[pos0:pos0 + T].unsqueeze(1 if seq_first else 0)
            return out
        idc = ids.contiguous().view(-1)
        out = torch.empty((*ids.shape, D), dtype=tok.dtype, device=tok.device)
        lib.call("elfa_embedding_fwd", idc, tok, pos, out, B * T, D, T, B if seq_first else 1, pos0, vocab_lo,
                 vocab_lo + tok.shape[0], vocab_total if vocab_total else vocab_lo + tok.shape[0], stream_ptr(out))
        return out

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        B, T, D, pos0, vocab_lo, vloc, has_pos, seq_first = ctx.args
        tok, pos = ctx.tok_ref, ctx.pos_ref
        if not dy.is_cuda:
            local = (ids - vocab_lo).view(-1)
            mask = (local >= 0) & (local < vloc)
            dtok = torch.zeros((vloc, D), dtype=torch.float32)
            dtok.index_add_(0, local[mask], dy.reshape(-1, D).float()[mask])
            dpos = None
            if has_pos:
                dpos = torch.zeros_like(pos, dtype=torch.float32)
                if vocab_lo == 0:
                    dpos[pos0:pos0 + T] = dy.float().sum(1 if seq_first else 0)
                dpos = dpos.to(pos.dtype)
            return None, dtok.to(tok.dtype), dpos, None, None, None, None
        dyc = dy.contiguous()
        idc = ids.contiguous().view(-1)
        tt = _grad_target(tok)
        tp = _grad_target(pos) if has_pos else None
        dtok_ret = dpos_ret = None
        if tt is not None:
            dtok_buf, acc = tt
            if not acc:
                dtok_buf.zero_()
        else:
            dtok_buf = dtok_ret = torch.zeros((vloc, D), dtype=torch.float32, device=dy.device)
        dpos_buf = None
        if has_pos:
            if tp is not None:
                dpos_buf, accp = tp
                if not accp:
                    dpos_buf.zero_()
            else:
                dpos_buf = dpos_ret = torch.zeros(pos.shape, dtype=torch.float32, device=dy.device)
        from .. import native
        if native.deterministic():
            # runtime.deterministic: no atomics. Rows of dy are grouped by token id (stable sort) and summed per group in a
            # fixed order; positions likewise (every position gets one row per batch entry).
            local = idc - vocab_lo
            keep = (local >= 0) & (local < vloc)
            dy2 = dyc.view(B * T, D)
            order = torch.argsort(torch.where(keep, local, torch.full_like(local, vloc)), stable=True)
            srt = local[order]
            nkeep = int(keep.sum())
            if nkeep:
                uniq, counts = torch.unique_consecutive(srt[:nkeep], return_counts=True)
                sums = torch.segment_reduce(dy2[order[:nkeep]].float(), "sum", lengths=counts)
                dtok_buf.index_put_((uniq,), dtok_buf[uniq] + sums)
            if dpos_buf is not None and vocab_lo == 0:
                per_pos = dy2.view(T, B, D).float().sum(1) if seq_first else dy2.view(B, T, D).float().sum(0)
                dpos_buf[pos0:pos0 + T] += per_pos
        else:
            lib.call("elfa_embedding_bwd", idc, dyc, dtok_buf, dpos_buf, B * T, D, T, B if seq_first else 1, pos0, vocab_lo,
                     vocab_lo + vloc, 1, stream_ptr(dyc))
        if dtok_ret is not None:
            dtok_ret = dtok_ret.to(tok.dtype)
        if dpos_ret is not None:
            dpos_ret = dpos_ret.to(pos.dtype)
        return None, dtok_ret, dpos_ret, None, None, None, None


def embedding(ids: torch.Tensor, tok: torch.Tensor, pos: Optional[torch.Tensor] = None, pos0: int = 0,
              vocab_lo: int = 0, seq_first: bool = False, vocab_total: int = 0) -> torch.Tensor:
    """``tok[ids - vocab_lo] (+ pos[pos0 + t])`` for ids inside this rank's vocabulary slice, zeros
    for the others (summing over vocabulary-parallel ranks gives the full embedding)."""
    return _Embedding.apply(ids, tok, pos, pos0, vocab_lo, seq_first, vocab_total)


# ------------------------------------------------------------------------------------ cross-entropy
def cross_entropy_ref(logits: torch.Tensor, targets: torch.Tensor, smoothing: float = 0.0) -> torch.Tensor:
    """Per-token loss, fp32: ``-((1-eps) * logp[target] + eps/V * sum_j logp[j])``; 0 where target == -100."""
    lf = logits.float()
    logp = lf - torch.logsumexp(lf, -1, keepdim=True)
    V = lf.shape[-1]
    valid = targets >= 0
    t = targets.clamp_min(0)
    nll = -logp.gather(-1, t.unsqueeze(-1)).squeeze(-1)
    loss = (1 - smoothing) * nll - (smoothing / V) * logp.sum(-1)
    return loss * valid


class _CrossEntropy(torch.autograd.Function):
    """Mean loss over valid tokens. The CUDA path computes the gradient in the same two passes that
    compute the loss and stores it *in place of the logits*; backward only rescales it."""

    @staticmethod
    def forward(ctx, logits, targets, smoothing, denom, grad_scale):
        V = logits.shape[-1]
        l2 = logits.reshape(-1, V)
        t1 = targets.reshape(-1)
        if not l2.is_cuda:
            per = cross_entropy_ref(l2, t1, smoothing)
            ctx.cpu = True
            ctx.save_for_backward(l2, t1)
            ctx.smoothing, ctx.denom, ctx.shape, ctx.grad_scale = smoothing, denom, logits.shape, grad_scale
            return per.sum() / denom
        assert l2.is_contiguous() and l2.dtype == torch.bfloat16
        rows = l2.shape[0]
        stats = torch.empty((rows, 4), dtype=torch.float32, device=l2.device)
        per = torch.empty(rows, dtype=torch.float32, device=l2.device)
        st = stream_ptr(l2)
        lib.call("elfa_xent_stats", l2, l2.stride(0), t1, stats, rows, V, 0, V, st)
        lib.call("elfa_xent_grad", l2, l2.stride(0), l2, l2.stride(0), t1, stats, 1, per, rows, V, 0, V, float(smoothing), None,
                 grad_scale / denom, st)
        ctx.cpu = False
        ctx.save_for_backward(l2)
        ctx.shape = logits.shape
        return per.sum() / denom

    @staticmethod
    def backward(ctx, dloss):
        if ctx.cpu:
            l2, t1 = ctx.saved_tensors
            with torch.enable_grad():
                li = l2.detach().requires_grad_(True)
                loss = cross_entropy_ref(li, t1, ctx.smoothing).sum() / ctx.denom
            (g,) = torch.autograd.grad(loss, li, dloss * ctx.grad_scale)
            return g.reshape(ctx.shape), None, None, None, None
        (g,) = ctx.saved_tensors
        # g already holds grad_scale * d(mean loss)/d(logits). The upstream gradient is taken to be 1
        # (call loss.backward() directly; a loss scale goes through `grad_scale`): checking it would
        # cost a host synchronisation, applying it a full pass over the logits.
        return g.reshape(ctx.shape), None, None, None, None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, smoothing: float = 0.0, denom: Optional[float] = None,
                  grad_scale: float = 1.0) -> torch.Tensor:
    """Mean token cross-entropy (fp32 scalar). On CUDA the logits tensor is overwritten with its
    gradient times ``grad_scale`` (do not reuse it) and backward expects a unit upstream gradient.
    ``denom`` defaults to the number of target tokens."""
    if denom is None:
        denom = float(targets.numel())
    return _CrossEntropy.apply(logits, targets, smoothing, denom, float(grad_scale))


def softmax(x: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """Row softmax of ``x * scale`` over the last dimension (reference: ``src/nn/nn_kernels.zig:226-267``).
    CUDA bf16 tensors use the warp-per-row kernel; everything else plain PyTorch."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.stride(-1) == 1 and scale > 0:
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        out = torch.empty_like(x2)
        lib.call("elfa_softmax_rows", x2, out, x2.shape[0], x2.shape[1], x2.stride(0), out.stride(0), float(scale), stream_ptr(x2))
        return out.view(x.shape)
    return torch.softmax(x.float() * scale, dim=-1).to(x.dtype)
