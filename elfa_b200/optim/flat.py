"""Flat parameter / gradient buffers.

All parameters of a rank live in one contiguous buffer (model dtype) and all gradients in one fp32
buffer of the same layout; ``param.main_grad`` is the parameter's view into the gradient buffer and
the backward kernels accumulate into it directly (weight-gradient GEMM epilogue, norm backward,
embedding scatter-add). One contiguous layout is what lets the optimizer be a handful of kernel
launches and lets ZeRO shard optimizer state by plain index ranges:

    [ TP-replicated, partial grads | TP-replicated, identical grads | TP-sharded ]  each part ordered (decay, no-decay)

* the first part (``[0, reduce_end)``) is the only region whose gradients need an all-reduce over the tensor
  parallel group (norm weights and position embeddings under sequence parallelism); the second part holds
  replicated parameters that every rank differentiates on the same full activations (no reduction); both count
  once in the gradient norm (``[0, replicated_end)``);
* ZeRO-1/2 give data-parallel rank ``r`` the slice ``[r * shard, (r+1) * shard)`` of the whole
  buffer (the buffer is padded to a multiple of ``dp * 1024`` elements).

reference: per-tensor ``len / num_gpus`` shards (``src/distributed/zero_sharding.zig:73-113``) and
the 1 MiB round-robin ownership rule (``src/tensor/sharding.zig:331-342``); a flat range per rank
replaces both because one kernel can then reduce, update and re-broadcast a whole bucket.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch

ALIGN = 64          # elements; keeps every parameter 128-byte aligned in bf16 (TMA needs 16 bytes)


@dataclass
class Segment:
    start: int
    end: int
    weight_decay: bool
    replicated: bool          # every tensor-parallel rank holds these parameters: their gradient counts once in the norm
    reduce: bool = False      # ... and each rank holds only a partial gradient: summed over the tensor-parallel group


class FlatParams:
    def __init__(self, named_params: Iterable[Tuple[str, torch.nn.Parameter]], dp_size: int = 1, dp_rank: int = 0,
                 grad_dtype: torch.dtype = torch.float32, allocator=None):
        items = []
        seen = set()
        for name, p in named_params:
            if id(p) in seen or not p.requires_grad:
                continue
            seen.add(id(p))
            items.append((name, p))
        if not items:
            raise ValueError("no trainable parameters")
        # stable sort: replicated first, then decay before no-decay
        # tensor-parallel classes: 0 = replicated with partial gradients (`tp_replicated`: summed over the group),
        # 1 = replicated with identical gradients on every rank (`tp_identical`: no reduction), 2 = sharded
        def key(it):
            p = it[1]
            cls = 0 if getattr(p, "tp_replicated", False) else (1 if getattr(p, "tp_identical", False) else 2)
            return (cls, 1 if getattr(p, "no_decay", False) or p.dim() < 2 else 0)
        items.sort(key=key)
        self.names = [n for n, _ in items]
        self.params = [p for _, p in items]
        # the buffer has the dtype of the model's weights (the largest parameter's), not of whichever parameter sorts first: a small
        # fp32 parameter (a learned scalar) may lead the order and is then stored in the model dtype like everything else
        self.dtype = max(self.params, key=lambda p: p.numel()).dtype
        self.device = self.params[0].device
        self.dp_size, self.dp_rank = dp_size, dp_rank
        offsets, off = [], 0
        for p in self.params:
            offsets.append(off)
            off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        quantum = dp_size * 1024
        self.numel = (off + quantum - 1) // quantum * quantum
        self.offsets = offsets
        self.symm = None
        if allocator is not None:
            # `allocator` is a symmetric arena: both buffers become regions that peers can address
            esz = torch.empty(0, dtype=self.dtype).element_size()
            gsz = torch.empty(0, dtype=grad_dtype).element_size()
            r_flat = allocator.alloc(self.numel * esz, "flat.params")
            r_grads = allocator.alloc(self.numel * gsz, "flat.grads")
            self.flat = r_flat.view(self.dtype, (self.numel,))
            self.grads = r_grads.view(grad_dtype, (self.numel,))
            self.symm = (allocator, r_flat, r_grads)
        else:
            self.flat = torch.zeros(self.numel, dtype=self.dtype, device=self.device)
            self.grads = torch.zeros(self.numel, dtype=grad_dtype, device=self.device)
        self.flat.zero_()
        self.grads.zero_()
        self.segments: List[Segment] = []
        for p, o in zip(self.params, offsets):
            n = p.numel()
            view = self.flat[o:o + n].view(p.shape)
            with torch.no_grad():
                view.copy_(p.data)
            p.data = view
            p.main_grad = self.grads[o:o + n].view(p.shape)
            p._grad_fresh = False
            k = key(("", p))
            seg_end = o + (n + ALIGN - 1) // ALIGN * ALIGN
            last = self.segments[-1] if self.segments else None
            if last is not None and last.replicated == (k[0] < 2) and last.reduce == (k[0] == 0) and last.weight_decay == (k[1] == 0):
                last.end = seg_end
            else:
                self.segments.append(Segment(o, seg_end, k[1] == 0, k[0] < 2, k[0] == 0))
        self.segments[-1].end = self.numel
        self.replicated_end = max((s.end for s in self.segments if s.replicated), default=0)
        self.reduce_end = max((s.end for s in self.segments if s.reduce), default=0)
        self.shard_size = self.numel // dp_size
        self.shard_lo = dp_rank * self.shard_size
        self.shard_hi = self.shard_lo + self.shard_size

    # ------------------------------------------------------------------
    def zero_grad(self) -> None:
        self.grads.zero_()
        for p in self.params:
            p.grad = None

    def fold_autograd_grads(self) -> None:
        """Adds gradients that autograd left in ``p.grad`` (ops without a fused accumulate, CPU
        runs) into the flat buffer."""
        for p in self.params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                p.grad = None

    def param_view(self, i: int) -> torch.Tensor:
        return self.params[i].data

    def grad_view(self, i: int) -> torch.Tensor:
        return self.params[i].main_grad

    def wd_ranges(self, lo: Optional[int] = None, hi: Optional[int] = None) -> List[Tuple[int, int, bool]]:
        """Maximal ``(start, end, weight_decay)`` runs clipped to ``[lo, hi)``."""
        lo = 0 if lo is None else lo
        hi = self.numel if hi is None else hi
        out: List[Tuple[int, int, bool]] = []
        for s in self.segments:
            a, b = max(s.start, lo), min(s.end, hi)
            if a >= b:
                continue
            if out and out[-1][2] == s.weight_decay and out[-1][1] == a:
                out[-1] = (out[-1][0], b, s.weight_decay)
            else:
                out.append((a, b, s.weight_decay))
        return out

    def param_slices(self) -> Dict[str, Tuple[int, int]]:
        return {n: (o, o + p.numel()) for n, p, o in zip(self.names, self.params, self.offsets)}

    # ------------------------------------------------------------------ optimizer state as logical tensors (checkpoints)
    def logical_state(self, v: torch.Tensor, lo: int, hi: int, pc) -> Dict[str, torch.Tensor]:
        """One optimizer-state buffer (``v`` covers the flat range ``[lo, hi)`` of this rank) as full per-parameter host
        tensors, independent of the data- and tensor-parallel sizes. Collective over both groups: every rank must call."""
        import torch.distributed as dist
        from ..parallel import tp as tpl
        v = v.detach()
        if hi - lo != self.numel:
            if v.is_cuda:
                full = torch.empty(self.numel, dtype=v.dtype, device=v.device)
                dist.all_gather_into_tensor(full, v.contiguous(), group=pc.dp_group)
            else:
                parts = [torch.empty_like(v) for _ in range(pc.dp_size)]
                dist.all_gather(parts, v.contiguous(), group=pc.dp_group)
                full = torch.cat(parts)
        else:
            full = v
        out: Dict[str, torch.Tensor] = {}
        for name, p, o in zip(self.names, self.params, self.offsets):
            t = full[o:o + p.numel()].view(p.shape)
            shard = getattr(p, "tp_shard", None)
            if pc.tp_size > 1 and shard is not None:
                parts = [torch.empty_like(t) for _ in range(pc.tp_size)]
                dist.all_gather(parts, t.contiguous(), group=pc.tp_group)
                t = tpl.unshard_param(parts, "vocab" if shard[0] == "vocab" else shard[0])
            out[name] = t.cpu().clone()
        return out

    @torch.no_grad()
    def load_logical_state(self, tensors: Dict[str, torch.Tensor], v: torch.Tensor, lo: int, hi: int, pc) -> None:
        """Inverse of :meth:`logical_state` for this rank's layout; padding elements are set to zero."""
        from ..parallel import tp as tpl
        v.zero_()
        for name, p, o in zip(self.names, self.params, self.offsets):
            if name not in tensors:
                raise KeyError(f"optimizer state is missing tensor '{name}'")
            full = tensors[name]
            shard = getattr(p, "tp_shard", None)
            if pc.tp_size > 1 and shard is not None:
                full = tpl.shard_param(full, shard[0], pc.tp_size, pc.tp_rank)
            if full.numel() != p.numel():
                raise ValueError(f"optimizer state '{name}': {full.numel()} elements, parameter has {p.numel()}")
            a, b = max(o, lo), min(o + p.numel(), hi)
            if a < b:
                v[a - lo:b - lo].copy_(full.reshape(-1)[a - o:b - o].to(v.device, v.dtype))
