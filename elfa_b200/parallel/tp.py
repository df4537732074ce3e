"""Tensor parallelism with sequence parallelism (Megatron style) and parameter sharding helpers.

Capabilities of the reference's gen-1 tensor/sequence-parallel code
(reference: ``src/distributed/tensor_parallel.zig:51-201`` shard / gather / all-reduce / broadcast,
``src/distributed/sequence_parallel.zig:54-200`` split / gather / reduce-scatter,
descriptors ``src/tensor/sharding.zig:183-287``), restated per rank:

* column-parallel linear (QKV, MLP-up): input is the sequence shard ``[S/tp, B, D]``; the
  all-gather along the sequence feeds the GEMM (**all-gather → GEMM**);
* row-parallel linear (attention-out, MLP-down): the GEMM output is a partial sum that is
  reduce-scattered along the sequence (**GEMM → reduce-scatter**). Partial sums are *summed*
  (the reference's ``allReduceTensor`` divides by the world size, which is wrong for a
  row-parallel product);
* vocabulary-parallel embedding, logits and cross-entropy.

Two backends implement the two fused primitives ``ag_gemm`` and ``gemm_rs``:
``nccl`` (library all-gather / reduce-scatter around the GEMM - the baseline) and ``fused``
(one kernel that moves the tiles over NVLink peer memory while the tensor cores run; see
``elfa_b200/parallel/fused.py``).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..ops.gemm import gemm
from ..quant.qat import (QuantSpec, cached_weight_operand, cached_weight_operand_bwd, cached_weight_quant, cached_weight_quant_bwd, fake_quant,
                         quantize_grad, use_block_scaled_bwd, use_block_scaled_gemm)
from .mesh import ParallelContext


# ------------------------------------------------------------------------------- parameter shards
def shard_param(full: torch.Tensor, kind: str, tp: int, rank: int) -> torch.Tensor:
    """Slice of a full parameter owned by ``rank``. Kinds: ``col`` (split dim 1), ``row`` and ``vocab``
    (split dim 0), ``col_qkv`` (``[D, 3D]`` laid out ``[Q|K|V]`` → this rank's heads of each),
    ``col_gated`` (``[D, 2F]`` laid out ``[gate|up]``), ``replicated``."""
    if tp == 1 or kind == "replicated":
        return full
    if kind == "col":
        n = full.shape[1] // tp
        return full[:, rank * n:(rank + 1) * n]
    if kind in ("row", "vocab"):
        n = full.shape[0] // tp
        return full[rank * n:(rank + 1) * n]
    if kind in ("col_qkv", "col_gated"):
        parts = 3 if kind == "col_qkv" else 2
        w = full.shape[1] // parts
        n = w // tp
        return torch.cat([full[:, i * w + rank * n:i * w + (rank + 1) * n] for i in range(parts)], dim=1)
    if kind.startswith("col_gqa:"):
        # grouped-query projection [D, (H + 2 Hkv) hd] laid out [Q | K | V]: this rank's query heads and its key / value heads
        H, Hkv, hd = (int(v) for v in kind.split(":")[1:])
        bounds = [(0, H * hd), (H * hd, (H + Hkv) * hd), ((H + Hkv) * hd, (H + 2 * Hkv) * hd)]
        out = []
        for a, b in bounds:
            n = (b - a) // tp
            out.append(full[:, a + rank * n:a + (rank + 1) * n])
        return torch.cat(out, dim=1)
    raise ValueError(kind)


def unshard_param(shards: List[torch.Tensor], kind: str) -> torch.Tensor:
    """Inverse of :func:`shard_param` (``shards[r]`` belongs to rank r)."""
    tp = len(shards)
    if tp == 1 or kind == "replicated":
        return shards[0]
    if kind == "col":
        return torch.cat(shards, dim=1)
    if kind in ("row", "vocab"):
        return torch.cat(shards, dim=0)
    if kind in ("col_qkv", "col_gated"):
        parts = 3 if kind == "col_qkv" else 2
        n = shards[0].shape[1] // parts
        return torch.cat([torch.cat([s[:, i * n:(i + 1) * n] for s in shards], dim=1) for i in range(parts)], dim=1)
    if kind.startswith("col_gqa:"):
        H, Hkv, hd = (int(v) for v in kind.split(":")[1:])
        nq, nk = H * hd // tp, Hkv * hd // tp
        cuts = [(0, nq), (nq, nq + nk), (nq + nk, nq + 2 * nk)]
        return torch.cat([torch.cat([s[:, a:b] for s in shards], dim=1) for a, b in cuts], dim=1)
    raise ValueError(kind)


# ------------------------------------------------------------------------------------ collectives
def _all_gather_dim0(x: torch.Tensor, pc: ParallelContext) -> torch.Tensor:
    out = torch.empty((x.shape[0] * pc.tp_size, *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=pc.tp_group)
    return out


def _reduce_scatter_dim0(x: torch.Tensor, pc: ParallelContext) -> torch.Tensor:
    n = x.shape[0] // pc.tp_size
    x = x.contiguous()
    if x.is_cuda:
        out = torch.empty((n, *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x, group=pc.tp_group)
        return out
    dist.all_reduce(x, group=pc.tp_group)           # gloo has no reduce-scatter
    return x[pc.tp_rank * n:(pc.tp_rank + 1) * n].clone()


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pc):
        ctx.pc = pc
        return _all_gather_dim0(x, pc)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_dim0(g, ctx.pc), None


class _ReduceScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pc):
        ctx.pc = pc
        return _reduce_scatter_dim0(x, pc)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_dim0(g, ctx.pc), None


class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pc):
        ctx.pc = pc
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.pc.tp_group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pc):
        x = x.contiguous()
        dist.all_reduce(x, group=pc.tp_group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


# ------------------------------------------------------------------- the two fused primitives
def ag_gemm(x_local: torch.Tensor, w: torch.Tensor, pc: ParallelContext, *, b_mn: bool, act: Optional[str] = None,
            preact: bool = False, keep: bool = True, defer_copy: bool = False) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """``y = act(all_gather_rows(x_local) @ op(w))``. Returns ``(y, x_full, pre)`` - the gathered
    input is a by-product that backward needs for the weight gradient. ``w`` is ``[K, N]`` when
    ``b_mn`` else ``[N, K]``."""
    if pc.comm_backend == "fused" and x_local.is_cuda:
        from . import fused
        return fused.ag_gemm(x_local, w, pc, b_mn=b_mn, act=act, preact=preact, keep=keep, defer_copy=defer_copy)
    x_full = _all_gather_dim0(x_local, pc)
    pre = None
    if act == "gelu":
        pre = torch.empty((x_full.shape[0], w.shape[1] if b_mn else w.shape[0]), dtype=x_full.dtype, device=x_full.device) if preact else None
        y = gemm(x_full, w, b_mn=b_mn, gelu=True, preact=pre, out_dtype=x_full.dtype)
    else:
        y = gemm(x_full, w, b_mn=b_mn, out_dtype=x_full.dtype)
    return y, x_full, pre


def gemm_rs(a: torch.Tensor, w: torch.Tensor, pc: ParallelContext, *, b_mn: bool, max_ctas: int = 0) -> torch.Tensor:
    """``reduce_scatter_rows(a @ op(w))``: every rank contributes a partial product over its slice of
    the contraction dimension and receives the summed rows ``[M/tp, N]`` it owns."""
    if pc.comm_backend == "fused" and a.is_cuda:
        from . import fused
        return fused.gemm_rs(a, w, pc, b_mn=b_mn, max_ctas=max_ctas)
    return _reduce_scatter_dim0(gemm(a, w, b_mn=b_mn, out_dtype=a.dtype), pc)


def _wgrad(w_ref: torch.Tensor, x2: torch.Tensor, dy2: torch.Tensor, w_dtype, max_ctas: int = 0) -> Optional[torch.Tensor]:
    """x2^T @ dy2 into ``w_ref.main_grad`` (returns None) or as a new tensor."""
    mg = getattr(w_ref, "main_grad", None)
    if mg is not None and dy2.is_cuda:
        fresh = getattr(w_ref, "_grad_fresh", False)
        gemm(x2, dy2, a_mn=True, b_mn=True, out=mg, accumulate=not fresh, max_ctas=max_ctas)
        w_ref._grad_fresh = False
        return None
    return gemm(x2, dy2, a_mn=True, b_mn=True, out_dtype=w_dtype, max_ctas=max_ctas)


_side_streams = {}


def _overlap_wgrad(pc: ParallelContext, t: torch.Tensor) -> bool:
    """Whether the weight-gradient GEMM runs on a second stream next to the fused GEMM→reduce-scatter kernel
    (which then gets 7/16 of the SMs). Off unless ``ELFA_OVERLAP_WGRAD=1``: on the 7B configuration at 2 ranks, where the
    products dominate, it costs 5 % (60.0 against 62.9 K tokens/s), and at 8 ranks 4.5 % (139.6 against 146.2 K): the
    reduce-scatter kernel's own GEMM and store pipeline slow down more than the overlap saves."""
    import os
    if not (t.is_cuda and pc.comm_backend == "fused" and pc.tp_size > 1):
        return False
    return os.environ.get("ELFA_OVERLAP_WGRAD", "0") not in ("0", "")


def _block_scaled_rs(pc: ParallelContext, M: int, K: int, N: int) -> bool:
    """Whether a GEMM → reduce-scatter of MXFP8 operands runs block-scaled inside the fused kernel (``ELFA_RS_MXFP8=0``: the
    same kernel on the dequantised bf16 values)."""
    import os
    if pc.comm_backend != "fused" or pc.tp_size == 1 or os.environ.get("ELFA_RS_MXFP8", "1") in ("0", ""):
        return False
    from . import fused
    return fused.supported_rs_mxfp8(M, K, N, pc.tp_size)


def _quantised_gather_enabled() -> bool:
    import os
    return os.environ.get("ELFA_AG_MXFP8", "1") not in ("0", "")


def _quantised_gather(x2: torch.Tensor, w: torch.Tensor, pc: ParallelContext, quant) -> bool:
    """Whether a column-parallel MXFP8 layer all-gathers quantised payloads (``fused.ag_gemm_mxfp8``) instead of
    fake-quantised bf16 rows. ``ELFA_AG_MXFP8=0`` switches it off."""
    import os
    if quant is None or quant.fmt != "mxfp8" or pc.comm_backend != "fused" or pc.tp_size == 1:
        return False
    if os.environ.get("ELFA_AG_MXFP8", "1") in ("0", ""):
        return False
    from . import fused
    return use_block_scaled_gemm(x2, w, quant) and fused.supported_mxfp8(x2.shape[0], x2.shape[1], w.shape[1])


class _ColumnParallelSP(torch.autograd.Function):
    """x_local ``[S/tp, B, D]`` → ``act(all_gather(x) @ w_local)`` ``[S, B, N/tp]``."""

    @staticmethod
    def forward(ctx, x, w, pc, act, quant):
        Sl, B, D = x.shape
        x2 = x.reshape(Sl * B, D)
        if _quantised_gather(x2, w, pc, quant):
            # quantise before sending: e4m3 payloads and scales cross NVLink (half the bytes), the product runs on
            # the block-scaled tensor-core path; x_full is the bf16 form of the gathered quantised rows
            from . import fused
            y, x_full, pre = fused.ag_gemm_mxfp8(x2, cached_weight_operand(w, quant), pc, act=act, preact=True)
        else:
            xq = fake_quant(x2, quant) if quant is not None else x2
            wq = cached_weight_quant(w, quant) if quant is not None else w
            y, x_full, pre = ag_gemm(xq, wq, pc, b_mn=True, act=act, preact=True, defer_copy=True)   # backward waits for the copy
        # the bf16 fake-quantised copy of the weight is not kept: paths that need it ask the per-step cache again
        ctx.save_for_backward(x_full, pre)
        ctx.pc, ctx.w_ref, ctx.shape, ctx.quant = pc, w, (Sl, B, D), quant
        return y.view(Sl * pc.tp_size, B, -1)

    @staticmethod
    def backward(ctx, dy):
        x_full, pre = ctx.saved_tensors
        pc = ctx.pc
        wdt = ctx.w_ref.dtype
        wq = None
        if pc.comm_backend == "fused" and x_full.is_cuda:
            from . import fused
            fused.wait_pending_copies(pc)        # x_full may have been copied on a side stream
        Sl, B, D = ctx.shape
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if pre is not None:
            if dy2.is_cuda:
                from ..native import lib, stream_ptr
                dpre = torch.empty_like(dy2)
                lib.call("elfa_elementwise", 1, pre, dy2, dpre, dy2.numel(), 1.0, stream_ptr(dy2))
                dy2 = dpre
            else:
                dy2 = (dy2.float() * ops.dgelu_tanh_ref(pre.float())).to(dy2.dtype)
        if ctx.quant is not None and ctx.quant.quant_backward:
            # quantised backward: dy in MXFP8 blocks along its last dimension, the weight along the same (contraction)
            # dimension; the reduce-scatter kernel multiplies the dequantised values (the same product)
            dy_op, dy2 = quantize_grad(dy2)
            if dy_op is not None and use_block_scaled_bwd(dy2, ctx.w_ref, ctx.quant) and _block_scaled_rs(pc, dy2.shape[0], dy2.shape[1], ctx.w_ref.shape[0]):
                from . import fused
                w_op = cached_weight_operand_bwd(ctx.w_ref, ctx.quant)
                if _overlap_wgrad(pc, dy2) and getattr(ctx.w_ref, "main_grad", None) is not None:
                    # the NVLink-bound reduce-scatter kernel on part of the SMs, the weight gradient on the rest (second stream)
                    dev = dy2.device
                    side = _side_streams.get(dev)
                    if side is None:
                        side = _side_streams[dev] = torch.cuda.Stream(dev)
                    cur = torch.cuda.current_stream(dev)
                    sms = torch.cuda.get_device_properties(dev).multi_processor_count
                    rs_ctas = max(16, (sms * 7 // 16) // 2 * 2)
                    side.wait_stream(cur)
                    with torch.cuda.stream(side):
                        dw = _wgrad(ctx.w_ref, x_full, dy2, wdt, max_ctas=sms - rs_ctas)
                    dx = fused.gemm_rs_mxfp8(dy_op, w_op, pc, max_ctas=rs_ctas)
                    cur.wait_stream(side)
                    return dx.view(Sl, B, D), dw, None, None, None
                dx = fused.gemm_rs_mxfp8(dy_op, w_op, pc)     # block-scaled dy @ w^T
                dw = _wgrad(ctx.w_ref, x_full, dy2, wdt)
                return dx.view(Sl, B, D), dw, None, None, None
            wq = cached_weight_quant_bwd(ctx.w_ref, ctx.quant)
        if wq is None:
            wq = cached_weight_quant(ctx.w_ref, ctx.quant) if ctx.quant is not None else ctx.w_ref
        if _overlap_wgrad(pc, dy2) and getattr(ctx.w_ref, "main_grad", None) is not None:
            # the two products are independent: the weight gradient runs on a second stream on the SMs that the
            # (NVLink-bound) reduce-scatter kernel leaves free
            dev = dy2.device
            side = _side_streams.get(dev)
            if side is None:
                side = _side_streams[dev] = torch.cuda.Stream(dev)
            cur = torch.cuda.current_stream(dev)
            sms = torch.cuda.get_device_properties(dev).multi_processor_count
            rs_ctas = max(16, (sms * 7 // 16) // 2 * 2)
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                dw = _wgrad(ctx.w_ref, x_full, dy2, wdt, max_ctas=sms - rs_ctas)
            dx = gemm_rs(dy2, wq, pc, b_mn=False, max_ctas=rs_ctas)
            cur.wait_stream(side)
        else:
            dx = gemm_rs(dy2, wq, pc, b_mn=False)              # dy @ w^T, summed over ranks, rows scattered
            dw = _wgrad(ctx.w_ref, x_full, dy2, wdt)
        return dx.view(Sl, B, D), dw, None, None, None


class _RowParallelSP(torch.autograd.Function):
    """x ``[S, B, K/tp]`` → ``reduce_scatter(x @ w_local)`` ``[S/tp, B, D]``."""

    @staticmethod
    def forward(ctx, x, w, pc, quant):
        S, B, K = x.shape
        x2 = x.reshape(S * B, K)
        if (quant is not None and quant.fmt == "mxfp8" and use_block_scaled_gemm(x2, w, quant)
                and _block_scaled_rs(pc, x2.shape[0], x2.shape[1], w.shape[1])):
            # e4m3 payloads and scales straight into the block-scaled MMAs of the fused kernel; the bf16 copy of the quantised
            # activations (same values) is kept for the weight gradient
            from ..ops.gemm_mxfp8 import quantize_mxfp8
            from . import fused
            x_op, xq = quantize_mxfp8(x2 if x2.is_contiguous() else x2.contiguous(), dequantized=True)
            y = fused.gemm_rs_mxfp8(x_op, cached_weight_operand(w, quant), pc)
        else:
            xq = fake_quant(x2, quant) if quant is not None else x2
            wq = cached_weight_quant(w, quant) if quant is not None else w
            y = gemm_rs(xq, wq, pc, b_mn=True)
        ctx.save_for_backward(xq)
        ctx.pc, ctx.w_ref, ctx.shape, ctx.quant = pc, w, (S, B, K), quant
        return y.view(S // pc.tp_size, B, -1)

    @staticmethod
    def backward(ctx, dy):
        (xq,) = ctx.saved_tensors
        pc = ctx.pc
        S, B, K = ctx.shape
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        q = ctx.quant
        if q is not None and q.quant_backward:
            from . import fused
            if (pc.comm_backend == "fused" and use_block_scaled_bwd(dy2, ctx.w_ref, q)
                    and fused.supported_mxfp8(dy2.shape[0], dy2.shape[1], ctx.w_ref.shape[0]) and _quantised_gather_enabled()):
                # e4m3 payloads and scales of dy cross NVLink, the input gradient is a block-scaled product; dy_full is the
                # bf16 form of the gathered quantised rows
                dx, dy_full, _ = fused.ag_gemm_mxfp8(dy2, cached_weight_operand_bwd(ctx.w_ref, q), pc)
                fused.wait_pending_copies(pc)
            else:
                _, dyq = quantize_grad(dy2)
                dx, dy_full, _ = ag_gemm(dyq, cached_weight_quant_bwd(ctx.w_ref, q), pc, b_mn=False, keep=False)
        else:
            wq = cached_weight_quant(ctx.w_ref, q) if q is not None else ctx.w_ref
            dx, dy_full, _ = ag_gemm(dy2, wq, pc, b_mn=False, keep=False)   # all_gather(dy) @ w^T; dy_full is consumed right below
        dw = _wgrad(ctx.w_ref, xq, dy_full, ctx.w_ref.dtype)
        return dx.view(S, B, K), dw, None, None


class _QuantLinear(torch.autograd.Function):
    """Single-rank linear with fake-quantised operands (straight-through backward)."""

    @staticmethod
    def forward(ctx, x, w, act, quant):
        x2 = x.reshape(-1, x.shape[-1])
        pre = torch.empty((x2.shape[0], w.shape[1]), dtype=x2.dtype, device=x2.device) if act == "gelu" else None
        if use_block_scaled_gemm(x2, w, quant):
            # e4m3 payloads + ue8m0 scales straight into the block-scaled MMA; the bf16 copy of the
            # quantised activations (same values) is kept for the weight gradient
            xc = x2 if x2.is_contiguous() else x2.contiguous()
            if quant.fmt == "nvfp4":
                from ..ops.gemm_nvfp4 import gemm_nvfp4, quantize_nvfp4
                x_op, xq = quantize_nvfp4(xc, dequantized=True)
                y = gemm_nvfp4(x_op, cached_weight_operand(w, quant), gelu=act == "gelu", preact=pre)
            else:
                from ..ops.gemm_mxfp8 import gemm_mxfp8, quantize_mxfp8
                x_op, xq = quantize_mxfp8(xc, dequantized=True)
                y = gemm_mxfp8(x_op, cached_weight_operand(w, quant), gelu=act == "gelu", preact=pre)
        else:
            xq = fake_quant(x2, quant)
            wq = cached_weight_quant(w, quant)
            if act == "gelu":
                y = gemm(xq, wq, b_mn=True, gelu=True, preact=pre, out_dtype=x2.dtype)
            else:
                y = gemm(xq, wq, b_mn=True, out_dtype=x2.dtype)
        # the bf16 fake-quantised weight is not kept (2 bytes per parameter on the block-scaled paths for nothing): backward
        # asks the per-step cache again where it multiplies bf16 operands
        ctx.save_for_backward(xq, pre)
        ctx.w_ref, ctx.shape, ctx.quant = w, x.shape, quant
        return y.view(*x.shape[:-1], w.shape[1])

    @staticmethod
    def backward(ctx, dy):
        xq, pre = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if pre is not None:
            if dy2.is_cuda:
                from ..native import lib, stream_ptr
                dpre = torch.empty_like(dy2)
                lib.call("elfa_elementwise", 1, pre, dy2, dpre, dy2.numel(), 1.0, stream_ptr(dy2))
                dy2 = dpre
            else:
                dy2 = (dy2.float() * ops.dgelu_tanh_ref(pre.float())).to(dy2.dtype)
        q = ctx.quant
        if q is not None and q.quant_backward:
            dy_op, dy2 = quantize_grad(dy2)           # from here on dy2 holds the dequantised values
            if dy_op is not None and use_block_scaled_bwd(dy2, ctx.w_ref, q):
                from ..ops.gemm_mxfp8 import gemm_mxfp8
                dx = gemm_mxfp8(dy_op, cached_weight_operand_bwd(ctx.w_ref, q)).view(ctx.shape)
            else:
                dx = gemm(dy2, cached_weight_quant_bwd(ctx.w_ref, q), out_dtype=dy2.dtype).view(ctx.shape)
        else:
            dx = gemm(dy2, cached_weight_quant(ctx.w_ref, q), out_dtype=dy2.dtype).view(ctx.shape)
        dw = _wgrad(ctx.w_ref, xq, dy2, ctx.w_ref.dtype)
        return dx, dw, None, None


def column_parallel_linear(x: torch.Tensor, w: torch.Tensor, pc: ParallelContext, act: Optional[str] = None,
                           quant: Optional[QuantSpec] = None) -> torch.Tensor:
    if quant is not None and not quant.enabled:
        quant = None
    if pc.tp_size == 1:
        return _QuantLinear.apply(x, w, act, quant) if quant is not None else ops.linear(x, w, None, act)
    if pc.sequence_parallel:
        return _ColumnParallelSP.apply(x, w, pc, act, quant)
    x = _CopyToTP.apply(x, pc)
    return _QuantLinear.apply(x, w, act, quant) if quant is not None else ops.linear(x, w, None, act)


def row_parallel_linear(x: torch.Tensor, w: torch.Tensor, pc: ParallelContext, quant: Optional[QuantSpec] = None) -> torch.Tensor:
    if quant is not None and not quant.enabled:
        quant = None
    if pc.tp_size == 1:
        return _QuantLinear.apply(x, w, None, quant) if quant is not None else ops.linear(x, w)
    if pc.sequence_parallel:
        return _RowParallelSP.apply(x, w, pc, quant)
    y = _QuantLinear.apply(x, w, None, quant) if quant is not None else ops.linear(x, w)
    return _ReduceFromTP.apply(y, pc)


# ------------------------------------------------------------------ vocabulary-parallel pieces
def embedding_reduce(x: torch.Tensor, pc: ParallelContext) -> torch.Tensor:
    """Sum of the per-rank partial embeddings; with sequence parallelism the sum is scattered
    along the sequence so that each rank keeps ``S/tp`` tokens."""
    if pc.tp_size == 1:
        return x
    if pc.sequence_parallel:
        return _ReduceScatterSeq.apply(x, pc)
    return _ReduceFromTP.apply(x, pc)


def vocab_parallel_logits(n: torch.Tensor, head: torch.Tensor, pc: ParallelContext, gather: bool) -> torch.Tensor:
    """``n [S(/tp), B, D] @ head_local^T`` → ``[S, B, V/tp]`` (``[S, B, V]`` when ``gather``)."""
    if pc.tp_size == 1:
        return ops.linear_nt(n, head)
    n_full = _GatherSeq.apply(n, pc) if pc.sequence_parallel else _CopyToTP.apply(n, pc)
    logits = ops.linear_nt(n_full, head)
    if gather:
        parts = [torch.empty_like(logits) for _ in range(pc.tp_size)]
        dist.all_gather(parts, logits.contiguous(), group=pc.tp_group)
        logits = torch.cat(parts, dim=-1)
    return logits


class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, pc, vocab_lo, vocab_total, smoothing, denom, grad_scale):
        Vl = logits.shape[-1]
        l2 = logits.reshape(-1, Vl)
        t1 = targets.reshape(-1)
        rows = l2.shape[0]
        ctx.shape = logits.shape
        if l2.is_cuda:
            from ..native import lib, stream_ptr
            st = stream_ptr(l2)
            if pc.comm_backend == "fused" and pc.symm is not None:
                # the statistics kernel stores its four numbers per token straight into every rank's table (peer stores)
                from . import fused
                allst = fused.xent_stats_exchange(l2, t1, pc, rows, Vl, vocab_lo, vocab_total)
            else:
                mine = torch.empty((rows, 4), dtype=torch.float32, device=l2.device)
                lib.call("elfa_xent_stats", l2, l2.stride(0), t1, mine, rows, Vl, vocab_lo, vocab_total, st)
                allst = torch.empty((pc.tp_size, rows, 4), dtype=torch.float32, device=l2.device)
                dist.all_gather_into_tensor(allst, mine, group=pc.tp_group)
            per = torch.empty(rows, dtype=torch.float32, device=l2.device)
            lib.call("elfa_xent_grad", l2, l2.stride(0), l2, l2.stride(0), t1, allst, pc.tp_size, per, rows, Vl, vocab_lo,
                     vocab_total, float(smoothing), None, grad_scale / denom, st)
            ctx.save_for_backward(l2)
            ctx.cuda = True
            return per.sum() / denom
        # CPU (gloo) path: same algebra in fp32
        lf = l2.float()
        m_loc = lf.max(-1).values
        m = m_loc.clone()
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=pc.tp_group)
        e = torch.exp(lf - m.unsqueeze(-1))
        s = e.sum(-1)
        sx = lf.sum(-1)
        local_t = t1 - vocab_lo
        mine = (local_t >= 0) & (local_t < Vl)
        tl = torch.where(mine, lf.gather(-1, local_t.clamp(0, Vl - 1).unsqueeze(-1)).squeeze(-1), torch.zeros_like(m))
        pack = torch.stack([s, sx, tl], 0)
        dist.all_reduce(pack, group=pc.tp_group)
        s, sx, tl = pack[0], pack[1], pack[2]
        lse = m + torch.log(s)
        valid = (t1 >= 0) & (t1 < vocab_total)
        per = -((1 - smoothing) * (tl - lse) + (smoothing / vocab_total) * (sx - vocab_total * lse)) * valid
        grad = torch.exp(lf - lse.unsqueeze(-1)) - smoothing / vocab_total
        onehot = torch.zeros_like(grad)
        onehot[mine, local_t[mine]] = 1 - smoothing
        grad = (grad - onehot) * valid.unsqueeze(-1) * (grad_scale / denom)
        ctx.save_for_backward(grad.to(logits.dtype))
        ctx.cuda = False
        return per.sum() / denom

    @staticmethod
    def backward(ctx, dloss):
        (g,) = ctx.saved_tensors
        if not ctx.cuda:
            g = g * dloss
        return g.view(ctx.shape), None, None, None, None, None, None, None


def vocab_parallel_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, pc: ParallelContext, vocab_lo: int, vocab_total: int,
                                 smoothing: float = 0.0, denom: Optional[float] = None, grad_scale: float = 1.0) -> torch.Tensor:
    """Mean cross-entropy over ``targets`` with the vocabulary split across the TP group. Each
    rank reduces its slice to four numbers per token (max, sum-exp, target logit, sum of logits);
    those are exchanged, and the loss and the in-place gradient follow from them."""
    if denom is None:
        denom = float(targets.numel())
    if pc.tp_size == 1:
        return ops.cross_entropy(logits, targets, smoothing, denom, grad_scale)
    return _VocabParallelCE.apply(logits, targets, pc, vocab_lo, vocab_total, smoothing, denom, float(grad_scale))
