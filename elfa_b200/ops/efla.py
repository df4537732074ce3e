"""EFLA (error-free linear attention), PRISM refinement and ShortConv ops.

Math restated from the reference (all three are host loops there):

* EFLA recurrence per (batch, head) with state ``S [d, d]`` (row = key index, column = value index):
  ``lam = |k_t|^2``, ``c = (1 - exp(-beta*lam)) / lam`` (series ``beta - beta^2 lam/2 + beta^3 lam^2/6``
  for ``lam < 1e-6``), ``p = S^T k_t``, ``S += c * k_t (v_t - p)^T``, ``o_t = S^T k_t`` with the updated
  state (reference: ``src/model/efla.zig:27-49,275-329``; CUDA ``kernels/cuda/efla.cu:93-197``,
  ``kernels/cuda/efla_scan.cu:99-152``). Note ``o_t = p + c*lam*(v_t - p)``, which the kernels use.
* chunk / cross-device composition: the update is affine in ``S`` (``S' = (I - c k k^T) S + c k v^T``), so
  chunks compose as affine maps ``(A, B)``; the reference adds chunk states, which is only right for
  additive linear attention (``efla.zig:702-732``, ``efla.cu:534-552``).
* PRISM (``src/model/prism.zig:318-421``): ``u = ShortConv(x)``; residual ``r = v - u`` per group of ``d``
  channels; per iteration ``l``: ``p = sigmoid(u W_p^l)``, ``delta = gelu(p * r)``, ``r -= delta``,
  ``refined += delta``; output ``u + refined``. The fast-weight state it also maintains never feeds
  back into the output within a step; :func:`prism_state_update` computes it for state carry.
* ShortConv (``prism.zig:948-973``, ``kernels/cuda/convolution.cu:4-57``):
  ``y[b,t,c] = bias[c] + sum_w x[b,t-w,c] * weight[c,w]`` (zero for ``t-w < 0``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..native import lib, stream_ptr
from .gemm import gelu_tanh_ref


def stable_coefficient(beta: torch.Tensor, lam: torch.Tensor) -> torch.Tensor:
    small = lam < 1e-6
    safe = torch.where(small, torch.ones_like(lam), lam)
    big = (1.0 - torch.exp(-beta * safe)) / safe
    ser = beta - 0.5 * beta * beta * lam + beta ** 3 * lam * lam / 6.0
    return torch.where(small, ser, big)


def efla_scan_ref(k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, state: Optional[torch.Tensor] = None
                  ) -> Tuple[torch.Tensor, torch.Tensor]:
    """k, v ``[B, T, H, d]`` → (o ``[B, T, H, d]``, final state ``[B, H, d, d]``), fp32, differentiable."""
    B, T, H, d = k.shape
    kf, vf = k.float(), v.float()
    S = torch.zeros(B, H, d, d, dtype=torch.float32, device=k.device) if state is None else state.float()
    outs = []
    b = beta.float().reshape(())
    for t in range(T):
        kt, vt = kf[:, t], vf[:, t]                       # [B, H, d]
        lam = (kt * kt).sum(-1)                           # [B, H]
        c = stable_coefficient(b, lam)
        p = torch.einsum("bhi,bhij->bhj", kt, S)
        S = S + c[..., None, None] * kt[..., :, None] * (vt - p)[..., None, :]
        outs.append(torch.einsum("bhij,bhi->bhj", S, kt))
    return torch.stack(outs, 1), S


def efla_scan_chunked_ref(k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, state: Optional[torch.Tensor] = None, chunk: int = 64
                          ) -> Tuple[torch.Tensor, torch.Tensor]:
    """The same recurrence in chunk-parallel (WY) form: everything inside a chunk of ``C`` tokens is matrix products,
    only ``T / C`` steps remain sequential. With ``K, V [C, d]`` the chunk's keys / values, ``c`` its coefficients and
    ``S0`` the state at its start, the pseudo-values ``u_t = c_t (v_t - S_{t-1}^T k_t)`` satisfy
    ``(I + diag(c) tril(K K^T, -1)) U = diag(c) (V - K S0)``, so with ``Tm = (I + diag(c) tril(K K^T, -1))^{-1} diag(c)``
    (a unit-lower-triangular solve, independent of the state and hence parallel over all chunks):
    ``U = Tm V - (Tm K) S0``, ``O = K S0 + tril(K K^T) U``, ``S_end = S0 + K^T U``.
    fp32, differentiable; equal to :func:`efla_scan_ref` up to rounding. It is the oracle for a tensor-core kernel of this
    form (the CUDA kernels here are sequential in time) and a faster CPU path for long sequences."""
    B, T, H, d = k.shape
    C = min(chunk, T)
    pad = (-T) % C
    kf, vf = k.float(), v.float()
    if pad:        # zero keys change nothing: their update and their output are zero
        kf = torch.nn.functional.pad(kf, (0, 0, 0, 0, 0, pad))
        vf = torch.nn.functional.pad(vf, (0, 0, 0, 0, 0, pad))
    nc = (T + pad) // C
    K = kf.view(B, nc, C, H, d).permute(0, 3, 1, 2, 4)                     # [B, H, nc, C, d]
    V = vf.view(B, nc, C, H, d).permute(0, 3, 1, 2, 4)
    c = stable_coefficient(beta.float().reshape(()), (K * K).sum(-1))      # [B, H, nc, C]
    G = K @ K.transpose(-1, -2)                                            # [B, H, nc, C, C]
    A = torch.eye(C, dtype=torch.float32, device=k.device) + c.unsqueeze(-1) * torch.tril(G, -1)
    W = torch.linalg.solve_triangular(A, c.unsqueeze(-1) * torch.cat((V, K), -1), upper=False, unitriangular=True)
    Wv, Wk = W[..., :d], W[..., d:]                                        # Tm V, Tm K
    Gi = torch.tril(G)
    S = torch.zeros(B, H, d, d, dtype=torch.float32, device=k.device) if state is None else state.float()
    outs = []
    for n in range(nc):                                                     # the only sequential part
        Kn = K[:, :, n]
        U = Wv[:, :, n] - Wk[:, :, n] @ S
        outs.append(Kn @ S + Gi[:, :, n] @ U)
        S = S + Kn.transpose(-1, -2) @ U
    o = torch.stack(outs, 2).permute(0, 2, 3, 1, 4).reshape(B, nc * C, H, d)
    return o[:, :T], S


class _EflaScan(torch.autograd.Function):
    """CUDA path: sequential-in-time kernels, one warp per (batch, head, 32 value columns) with its columns
    of the fp32 state in registers; backward recomputes the states inside each chunk from the
    chunk-boundary states saved by forward."""

    @staticmethod
    def forward(ctx, k, v, beta, state, chunk):
        B, T, H, d = k.shape
        kc, vc = k.contiguous(), v.contiguous()
        o = torch.empty_like(kc)
        nchunks = (T + chunk - 1) // chunk
        ckpt = torch.empty((B, H, nchunks, d, d), dtype=torch.float32, device=k.device)
        s_out = torch.empty((B, H, d, d), dtype=torch.float32, device=k.device)
        bt = beta.detach().float().reshape(1).contiguous()
        st0 = state.float().contiguous() if state is not None else None
        lib.call("elfa_efla_scan_fwd", kc, vc, bt, st0, o, s_out, ckpt, B, T, H, d, chunk, stream_ptr(kc))
        ctx.save_for_backward(kc, vc, bt, ckpt)
        ctx.cfg = (B, T, H, d, chunk, state is not None)
        return o, s_out

    @staticmethod
    def backward(ctx, do, ds_out):
        kc, vc, bt, ckpt = ctx.saved_tensors
        B, T, H, d, chunk, has_state = ctx.cfg
        dk = torch.empty_like(kc)
        dv = torch.empty_like(vc)
        rows = B * T * H
        dbeta = torch.empty(rows, dtype=torch.float32, device=kc.device)                 # per-token terms, summed below
        ds0 = torch.empty((B, H, d, d), dtype=torch.float32, device=kc.device)
        work = torch.empty((B * H, chunk, d, d), dtype=torch.float32, device=kc.device)
        dk_part = torch.empty((d // 32, rows, d), dtype=torch.float32, device=kc.device)  # one slice per block of 32 value columns
        dc_part = torch.empty((d // 32, rows), dtype=torch.float32, device=kc.device)
        dso = ds_out.float().contiguous() if ds_out is not None else None
        lib.call("elfa_efla_scan_bwd", kc, vc, bt, ckpt, do.contiguous(), dso, dk, dv, dbeta, ds0, work, dk_part, dc_part,
                 B, T, H, d, chunk, stream_ptr(kc))
        return dk, dv, dbeta.sum().reshape(1), (ds0 if has_state else None), None


def efla_scan(k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, state: Optional[torch.Tensor] = None, chunk: int = 16
              ) -> Tuple[torch.Tensor, torch.Tensor]:
    """EFLA recurrence. CPU tensors use the differentiable reference loop; CUDA bf16 tensors use the
    native kernels when the head dimension is supported (multiple of 32, at most 128)."""
    d = k.shape[-1]
    if k.is_cuda and k.dtype == torch.bfloat16 and d % 32 == 0 and d <= 128:
        o, s = _EflaScan.apply(k, v, beta.reshape(1), state, chunk)
        return o, s
    # CPU / unsupported shapes: the chunk-parallel form for long sequences (same values up to fp32 rounding, a fraction of
    # the Python-loop time), the token-by-token oracle otherwise
    o, s = efla_scan_chunked_ref(k, v, beta, state, 64) if k.shape[1] > 64 else efla_scan_ref(k, v, beta, state)
    return o.to(k.dtype), s


def compose_affine(a1: torch.Tensor, b1: torch.Tensor, a2: torch.Tensor, b2: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Composition of two state maps ``S -> A S + B`` (1 applied first, then 2)."""
    return a2 @ a1, a2 @ b1 + b2


def chunk_affine_map(k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """The affine map ``(A, B)`` of a block of tokens: ``S_end = A S_start + B`` with
    ``A = prod_t (I - c_t k_t k_t^T)`` and ``B`` the final state from a zero start. k, v ``[B, T, H, d]``.
    Used to stitch chunks or sequence-parallel ranks together exactly. Both come out of the scan itself:
    ``B`` is its final state from a zero start, ``A`` its final state for zero values started from the identity
    (then ``S_end = A I + 0``), so a block of any length costs two scans instead of a Python loop over its tokens."""
    B_, T, H, d = k.shape
    eye = torch.eye(d, dtype=torch.float32, device=k.device).expand(B_, H, d, d).contiguous()
    _, Bm = efla_scan(k, v, beta)
    _, A = efla_scan(k, torch.zeros_like(v), beta, eye)
    return A, Bm


# --------------------------------------------------------------------------------------- ShortConv
def shortconv_ref(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x ``[B, T, C]``, weight ``[C, W]`` → causal depthwise convolution, fp32 math."""
    B, T, C = x.shape
    W = weight.shape[1]
    xf = torch.nn.functional.pad(x.float(), (0, 0, W - 1, 0))          # left pad time
    y = torch.zeros(B, T, C, dtype=torch.float32, device=x.device)
    for w in range(W):
        y = y + xf[:, W - 1 - w:W - 1 - w + T] * weight.float()[:, w]
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


class _ShortConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        B, T, C = x.shape
        xc = x.contiguous()
        y = torch.empty_like(xc)
        lib.call("elfa_shortconv_fwd", xc, weight, bias, y, B, T, C, weight.shape[1], stream_ptr(xc))
        ctx.save_for_backward(xc, weight)
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, weight = ctx.saved_tensors
        B, T, C = xc.shape
        W = weight.shape[1]
        dyc = dy.contiguous()
        dx = torch.empty_like(xc)
        dw = torch.empty((C, W), dtype=torch.float32, device=xc.device)
        db = torch.empty(C, dtype=torch.float32, device=xc.device) if ctx.has_bias else None
        lib.call("elfa_shortconv_bwd", xc, weight, dyc, dx, dw, db, B, T, C, W, stream_ptr(xc))
        return dx, dw.to(weight.dtype), (db.to(weight.dtype) if db is not None else None)


def shortconv(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    if x.is_cuda and x.dtype == torch.bfloat16:
        return _ShortConv.apply(x, weight, bias)
    return shortconv_ref(x, weight, bias)


# ------------------------------------------------------------------------------------------- PRISM
class _PrismRefine(torch.autograd.Function):
    """CUDA path: one kernel forward, one backward (recomputes the residuals; the gradient of the
    gates is summed over the groups inside the thread that owns the channel: no atomics)."""

    @staticmethod
    def forward(ctx, u, v, group_dim, *ps):
        import ctypes
        B, T, D = u.shape
        uc, vc = u.contiguous(), v.contiguous()
        pcs = [p.contiguous() for p in ps]
        y = torch.empty_like(uc)
        arr = (ctypes.c_uint64 * len(pcs))(*[p.data_ptr() for p in pcs])
        lib.call("elfa_prism_fwd", uc, vc, ctypes.addressof(arr), y, B * T, D // group_dim, group_dim, len(pcs), stream_ptr(uc))
        ctx.save_for_backward(uc, vc, *pcs)
        ctx.group_dim = group_dim
        return y

    @staticmethod
    def backward(ctx, dy):
        import ctypes
        uc, vc, *pcs = ctx.saved_tensors
        B, T, D = uc.shape
        d = ctx.group_dim
        dyc = dy.contiguous()
        du, dv = torch.empty_like(uc), torch.empty_like(vc)
        dps = [torch.empty((B, T, d), dtype=torch.float32, device=uc.device) for _ in pcs]
        parr = (ctypes.c_uint64 * len(pcs))(*[p.data_ptr() for p in pcs])
        darr = (ctypes.c_uint64 * len(pcs))(*[p.data_ptr() for p in dps])
        lib.call("elfa_prism_bwd", uc, vc, ctypes.addressof(parr), dyc, du, dv, ctypes.addressof(darr), B * T, D // d, d, len(pcs),
                 stream_ptr(uc))
        return (du, dv, None) + tuple(g.to(p.dtype) for g, p in zip(dps, pcs))


def prism_refine(u: torch.Tensor, v: torch.Tensor, p_list, group_dim: int) -> torch.Tensor:
    """``u``, ``v`` ``[B, T, D]``; ``p_list[l]`` ``[B, T, d]`` (already sigmoid-ed). Returns ``u + refined``."""
    if u.is_cuda and u.dtype == torch.bfloat16 and 1 <= len(p_list) <= 8 and all(p.dtype == torch.bfloat16 for p in p_list):
        return _PrismRefine.apply(u, v, group_dim, *p_list)
    return prism_refine_ref(u, v, p_list, group_dim)


def prism_refine_ref(u: torch.Tensor, v: torch.Tensor, p_list, group_dim: int) -> torch.Tensor:
    """Plain PyTorch form (CPU path and test oracle)."""
    B, T, D = u.shape
    G = D // group_dim
    r = (v.float() - u.float()).view(B, T, G, group_dim)
    refined = torch.zeros_like(r)
    for p in p_list:
        delta = gelu_tanh_ref(p.float().unsqueeze(2) * r)
        r = r - delta
        refined = refined + delta
    return (u.float() + refined.view(B, T, D)).to(u.dtype)


@torch.no_grad()
def prism_state_update(state: torch.Tensor, deltas, betas, ks, forget: float) -> torch.Tensor:
    """Carries the PRISM fast-weight state ``[B, G, d, d]`` over a block of tokens.
    ``deltas[l]`` ``[B, T, G, d]``, ``betas[l]`` ``[B, T]``, ``ks[l]`` ``[B, T, d]`` (unit norm).
    Iteration 0: ``S <- a S - a b (S k) k^T + b delta k^T``; later iterations: ``S <- S + b delta k^T``."""
    S = state.float().clone()
    T = deltas[0].shape[1]
    for t in range(T):
        for l, (dl, bl, kl) in enumerate(zip(deltas, betas, ks)):
            k = kl[:, t].float()                              # [B, d]
            b = bl[:, t].float()[:, None, None, None]
            d_t = dl[:, t].float()                            # [B, G, d]
            outer = d_t[..., :, None] * k[:, None, None, :]   # [B, G, d, d]
            if l == 0:
                Sk = torch.einsum("bgij,bj->bgi", S, k)
                S = forget * S - forget * b * Sk[..., :, None] * k[:, None, None, :] + b * outer
            else:
                S = S + b * outer
    return S
