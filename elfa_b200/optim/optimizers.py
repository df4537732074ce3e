"""AdamW, Lion, Muon and the Lion+Muon router on flat buffers, with ZeRO-1/2 sharding of the
optimizer state over the data-parallel group.

Math (reference): Lion ``v = b1*m + (1-b1)*g; m = b2*m + (1-b2)*g; p = p*(1 - lr*wd) - lr*sign(v)``
(``kernels/cuda/optim.cu:125-146``; CPU form ``src/optim/optimizer.zig:111-143``); AdamW
bias-corrected with decoupled decay ``p -= lr*(m_hat/(sqrt(v_hat)+eps) + wd*p)``
(``src/kernels/optim_kernels.zig:129-167``); Muon ``m = beta*m + g; Y = m/||m||_F;
Y <- 0.5*Y*(3I - Y^T Y)`` x ``iters`` on the smaller Gram side, ``p -= lr*Y``, no decay
(``src/optim/optimizer.zig:246-320``, ``kernels/cuda/optim.cu:378-398``); routing ``ndim == 2 →
Muon, else Lion`` (``optimizer.zig:361-369``). Moments and master weights are fp32 (the reference's
CUDA kernels keep bf16 moments).

One optimizer step on CUDA is: [DP reduce] → sum of squares → clip coefficient / non-finite guard
on the device → update kernels (which skip themselves when the guard fired) → [DP all-gather].
Nothing in the step reads back to the host.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..native import lib, stream_ptr
from ..ops.gemm import gemm
from ..parallel.mesh import ParallelContext
from .flat import FlatParams


def _ptype(t: torch.Tensor) -> int:
    return 0 if t.dtype == torch.float32 else 1


class _Base:
    """Common state: flat buffers, DP sharding, clipping scalars."""

    def __init__(self, flat: FlatParams, pc: Optional[ParallelContext], zero_stage: int, lr: float, weight_decay: float,
                 max_grad_norm: float):
        self.flat, self.pc = flat, pc or ParallelContext()
        # stage 3: `flat` holds only this rank's shards and reduces its gradients itself (parallel/zero3.py)
        self.presharded = bool(getattr(flat, "presharded", False))
        if self.presharded:
            zero_stage = 0
        self.zero_stage = zero_stage if self.pc.dp_size > 1 else 0
        self.lr, self.weight_decay, self.max_grad_norm = lr, weight_decay, max_grad_norm
        self.step_count = 0
        self.loss_scale = 1.0
        self.lr_on_device = False      # Lion / Muon kernels read the learning rate from scalars[4] (CUDA-graph replay)
        dev = flat.device
        self.sharded = self.zero_stage >= 1
        self.lo, self.hi = (flat.shard_lo, flat.shard_hi) if self.sharded else (0, flat.numel)
        n = self.hi - self.lo
        self.master_is_param = flat.dtype == torch.float32
        self.master = flat.flat[self.lo:self.hi] if self.master_is_param else flat.flat[self.lo:self.hi].float()
        self.scalars = torch.zeros(8, dtype=torch.float32, device=dev)     # sumsq, clip_coef, grad_norm, skip, lr (graph replay)
        self.part = torch.zeros(4096, dtype=torch.float32, device=dev)
        self.n_local = n
        self.last_grad_norm = 0.0
        # fused ZeRO path (peer-memory kernels): needs the flat buffers inside a symmetric arena
        self.zero_fused = None
        zf = getattr(flat, "symm", None)
        if self.sharded and zf is not None and flat.flat.is_cuda and self.pc.comm_backend == "fused":
            import ctypes
            arena, r_flat, r_grads = zf
            w = arena.world
            flags = arena.alloc(1024, "zero.barrier")
            self.zero_fused = {
                "arena": arena,
                "peer_params": (ctypes.c_uint64 * w)(*[arena.peer_address(r, r_flat) for r in range(w)]),
                "peer_grads": (ctypes.c_uint64 * w)(*[arena.peer_address(r, r_grads) for r in range(w)]),
                "peer_flags": (ctypes.c_uint64 * w)(*[arena.peer_address(r, flags) for r in range(w)]),
                "flags": flags, "epoch": 0,
            }
            self.gshard = torch.zeros(n, dtype=torch.float32, device=dev)
            arena.barrier()
        # unsharded data parallel with the gradient buffer in an arena that has a multicast mapping (ELFA_NVLS=1): the gradient
        # all-reduce is one in-switch reduction pass (parallel/nvls.py) instead of the library call
        self.nvls = None
        if (not self.sharded and not self.presharded and zf is not None and self.pc.dp_size > 1 and flat.flat.is_cuda
                and self.pc.comm_backend == "fused" and getattr(zf[0], "multicast_ptr", 0)):
            from ..parallel.nvls import MultimemGroup
            self.nvls = MultimemGroup(zf[0])

    # --------------------------------------------------------------- gradient synchronisation
    def _symm_barrier(self) -> None:
        import ctypes
        z = self.zero_fused
        z["epoch"] += 1
        lib.call("elfa_symm_barrier", ctypes.addressof(z["peer_flags"]), z["flags"].tensor, self.pc.dp_rank, self.pc.dp_size,
                 z["epoch"], 0, stream_ptr(self.flat.flat))

    def _grads(self, a: int, b: int) -> torch.Tensor:
        """Gradient values of the global index range [a, b) this rank updates."""
        if self.zero_fused is not None:
            return self.gshard[a - self.lo:b - self.lo]
        return self.flat.grads[a:b]

    def reduce_gradients(self) -> None:
        """TP: all-reduce the replicated prefix. DP: all-reduce (ZeRO-0) or reduce-scatter
        (ZeRO>=1) the whole buffer; gradients are averaged over DP."""
        pc, f = self.pc, self.flat
        if self.presharded:
            return
        red = getattr(f, "reduce_end", f.replicated_end)
        if pc.tp_size > 1 and red > 0:
            dist.all_reduce(f.grads[:red], group=pc.tp_group)
        if self.zero_fused is not None:
            import ctypes
            z = self.zero_fused
            self._symm_barrier()          # every rank's gradients are complete and visible
            lib.call("elfa_zero_reduce", ctypes.addressof(z["peer_grads"]), pc.dp_rank, pc.dp_size, self.lo, self.hi - self.lo,
                     self.gshard, 1.0 / pc.dp_size, self.part, self.scalars, stream_ptr(f.grads))
            return
        if pc.dp_size > 1 and self.nvls is not None:
            self.nvls.all_reduce_(f.symm[2], f.numel, torch.float32, 1.0 / pc.dp_size)
            return
        if pc.dp_size > 1:
            if self.sharded and f.grads.is_cuda:
                shard = f.grads[self.lo:self.hi]
                dist.reduce_scatter_tensor(shard, f.grads, op=dist.ReduceOp.AVG, group=pc.dp_group)
            else:
                dist.all_reduce(f.grads, group=pc.dp_group)
                f.grads.div_(pc.dp_size)

    def gather_params(self) -> None:
        if self.zero_fused is not None:
            if not getattr(self, "_fused_gather_done", False):
                # the update kernel did not broadcast (non-AdamW optimizers): library all-gather
                dist.all_gather_into_tensor(self.flat.flat, self.flat.flat[self.lo:self.hi], group=self.pc.dp_group)
            self._fused_gather_done = False
            self._symm_barrier()          # all parameter stores have landed before the next forward
            return
        if self.sharded:
            f, pc = self.flat, self.pc
            if f.flat.is_cuda:
                dist.all_gather_into_tensor(f.flat, f.flat[self.lo:self.hi], group=pc.dp_group)
            else:
                parts = [torch.empty_like(f.flat[self.lo:self.hi]) for _ in range(pc.dp_size)]
                dist.all_gather(parts, f.flat[self.lo:self.hi].contiguous(), group=pc.dp_group)
                f.flat.copy_(torch.cat(parts))

    # --------------------------------------------------------------------------- norm / clip
    def _norm_and_clip(self) -> None:
        """Fills ``self.scalars`` (device). The squared norm counts TP-replicated gradients once."""
        f, pc = self.flat, self.pc
        g = self._grads(self.lo, self.hi)
        inv_scale = 1.0 / self.loss_scale
        if g.is_cuda:
            st = stream_ptr(g)
            distributed = (pc.tp_size > 1) or self.sharded or (self.presharded and pc.dp_size > 1)
            if not distributed:
                lib.call("elfa_sumsq", g, _ptype(g), g.numel(), self.part, self.scalars, 0, st)
            else:
                # replicated prefix counted on tp_rank 0 only
                rep_hi = min(max(f.replicated_end, self.lo), self.hi)
                self.scalars[0].zero_()
                acc = 0
                if rep_hi > self.lo and pc.tp_rank == 0:
                    lib.call("elfa_sumsq", self._grads(self.lo, rep_hi), _ptype(g), rep_hi - self.lo, self.part, self.scalars, 0, st)
                    acc = 1
                if self.hi > rep_hi:
                    lib.call("elfa_sumsq", self._grads(rep_hi, self.hi), _ptype(g), self.hi - rep_hi, self.part, self.scalars, acc, st)
                dist.all_reduce(self.scalars[0:1], group=pc.dp_group if self.presharded else (None if self.sharded else pc.tp_group))
            lib.call("elfa_clip_coef", self.scalars, float(self.max_grad_norm), float(inv_scale), st)
            return
        # CPU
        sq = float(g.double().pow(2).sum())
        if pc.tp_size > 1 or self.sharded or (self.presharded and pc.dp_size > 1):
            rep_hi = min(max(f.replicated_end, self.lo), self.hi)
            sq = float(f.grads[rep_hi:self.hi].double().pow(2).sum())
            if pc.tp_rank == 0:
                sq += float(f.grads[self.lo:rep_hi].double().pow(2).sum())
            t = torch.tensor([sq], dtype=torch.float64)
            dist.all_reduce(t, group=pc.dp_group if self.presharded else (None if self.sharded else pc.tp_group))
            sq = float(t)
        norm = (sq ** 0.5) * inv_scale
        finite = norm == norm and norm != float("inf")
        coef = 1.0
        if finite and self.max_grad_norm > 0 and norm > self.max_grad_norm and norm > 1e-8:
            coef = self.max_grad_norm / norm
        self.scalars[0], self.scalars[1], self.scalars[2], self.scalars[3] = sq, coef * inv_scale if finite else 0.0, norm, 0.0 if finite else 1.0

    def grad_norm(self) -> float:
        """Host read of the last step's (unscaled, pre-clip) gradient norm."""
        return float(self.scalars[2])

    def skipped(self) -> bool:
        return bool(self.scalars[3] != 0)

    # ------------------------------------------------------------------------------ stepping
    def step(self, lr: Optional[float] = None) -> None:
        if lr is not None:
            self.lr = lr
        self.flat.fold_autograd_grads()
        self.reduce_gradients()
        self._norm_and_clip()
        self.step_count += 1
        self._update()
        self.gather_params()
        if self.presharded:
            self.flat.after_step()       # full-size copies of the parameters are stale now
        from ..quant.qat import new_weight_epoch
        new_weight_epoch()

    def zero_grad(self) -> None:
        self.flat.zero_grad()

    def _update(self) -> None:
        raise NotImplementedError

    def _param_out(self):
        """(tensor, type) of the working-precision copy to write, or (None, 0) when the master
        weights are the parameters themselves."""
        if self.master_is_param:
            return None, 0
        return self.flat.flat[self.lo:self.hi], 1

    # ---------------------------------------------------------------------------- checkpoint
    def state_tensors(self) -> Dict[str, torch.Tensor]:
        raise NotImplementedError

    def state_dict(self) -> Dict[str, object]:
        """Every state buffer as full per-parameter ("logical") host tensors: the shards are gathered over the data-parallel
        group and the tensor-parallel slices re-assembled, so the saved state does not depend on the parallel layout and a
        run may resume at another data- or tensor-parallel size. Collective: every rank must call."""
        out: Dict[str, object] = {"step": self.step_count, "lr": self.lr, "format": "logical"}
        out["tensors"] = {k: self.flat.logical_state(v, self.lo, self.hi, self.pc) for k, v in self.state_tensors().items()}
        return out

    def load_state_dict(self, sd) -> None:
        self.step_count = int(sd["step"])
        if sd.get("format") != "logical":
            # files written before the layout-independent form: flat shards, valid for the layout that wrote them only
            for k, v in self.state_tensors().items():
                t = sd["tensors"][k]
                if sd.get("stacked_over_dp"):
                    t = t[self.pc.dp_rank]
                v.copy_(t.to(v.device))
            return
        for k, v in self.state_tensors().items():
            self.flat.load_logical_state(sd["tensors"][k], v, self.lo, self.hi, self.pc)


class AdamW(_Base):
    def __init__(self, flat, pc=None, zero_stage=0, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_grad_norm=1.0):
        super().__init__(flat, pc, zero_stage, lr, weight_decay, max_grad_norm)
        self.betas, self.eps = betas, eps
        self.m = torch.zeros(self.n_local, dtype=torch.float32, device=flat.device)
        self.v = torch.zeros(self.n_local, dtype=torch.float32, device=flat.device)

    def _update(self) -> None:
        f = self.flat
        b1, b2 = self.betas
        pout, ptype = self._param_out()
        for a, b, wd in f.wd_ranges(self.lo, self.hi):
            s, e = a - self.lo, b - self.lo
            g = self._grads(a, b)
            wdv = self.weight_decay if wd else 0.0
            if self.zero_fused is not None and not self.master_is_param:
                import ctypes
                z = self.zero_fused
                lib.call("elfa_zero_adamw_allgather", ctypes.addressof(z["peer_params"]), self.pc.dp_rank, self.pc.dp_size, a, b - a,
                         self.master[s:e], self.m[s:e], self.v[s:e], g, float(self.lr), float(b1), float(b2), float(self.eps),
                         float(wdv), self.step_count, self.scalars, 0, 1 << 62, stream_ptr(g))
                self._fused_gather_done = True
                continue
            if g.is_cuda:
                lib.call("elfa_adamw", pout[s:e] if pout is not None else None, ptype, self.master[s:e], self.m[s:e], self.v[s:e], g,
                         _ptype(g), e - s, float(self.lr), float(b1), float(b2), float(self.eps), float(wdv), self.step_count,
                         self.scalars, stream_ptr(g))
            else:
                if self.skipped():
                    continue
                gg = g.float() * float(self.scalars[1])
                m, v, p = self.m[s:e], self.v[s:e], self.master[s:e]
                m.mul_(b1).add_(gg, alpha=1 - b1)
                v.mul_(b2).addcmul_(gg, gg, value=1 - b2)
                mh = m / (1 - b1 ** self.step_count)
                vh = v / (1 - b2 ** self.step_count)
                p.sub_(self.lr * (mh / (vh.sqrt() + self.eps) + wdv * p))
                if pout is not None:
                    pout[s:e].copy_(p.to(pout.dtype))

    def state_tensors(self):
        d = {"m": self.m, "v": self.v}
        if not self.master_is_param:
            d["master"] = self.master
        return d


class Lion(_Base):
    def __init__(self, flat, pc=None, zero_stage=0, lr=1e-4, betas=(0.95, 0.98), weight_decay=0.1, max_grad_norm=1.0,
                 ranges=None):
        super().__init__(flat, pc, zero_stage, lr, weight_decay, max_grad_norm)
        self.betas = betas
        self.m = torch.zeros(self.n_local, dtype=torch.float32, device=flat.device)
        self.ranges = ranges      # optional list of (start, end, wd) restricting the update (Lion+Muon)

    def _update(self) -> None:
        f = self.flat
        b1, b2 = self.betas
        pout, ptype = self._param_out()
        rngs = self.ranges if self.ranges is not None else f.wd_ranges(self.lo, self.hi)
        for a, b, wd in rngs:
            a, b = max(a, self.lo), min(b, self.hi)
            if a >= b:
                continue
            s, e = a - self.lo, b - self.lo
            g = self._grads(a, b)
            wdv = self.weight_decay if wd else 0.0
            if g.is_cuda:
                lib.call("elfa_lion", pout[s:e] if pout is not None else None, ptype, self.master[s:e], self.m[s:e], g, _ptype(g),
                         e - s, -1.0 if self.lr_on_device else float(self.lr), float(b1), float(b2), float(wdv), self.scalars,
                         stream_ptr(g))
            else:
                if self.skipped():
                    continue
                gg = g.float() * float(self.scalars[1])
                m, p = self.m[s:e], self.master[s:e]
                u = b1 * m + (1 - b1) * gg
                p.mul_(1 - self.lr * wdv).sub_(self.lr * torch.sign(u))
                m.mul_(b2).add_(gg, alpha=1 - b2)
                if pout is not None:
                    pout[s:e].copy_(p.to(pout.dtype))

    def state_tensors(self):
        d = {"m": self.m}
        if not self.master_is_param:
            d["master"] = self.master
        return d


def newton_schulz(y: torch.Tensor, iters: int) -> torch.Tensor:
    """``Y <- 0.5 * Y (3I - Y^T Y)`` (or the left form when rows < cols) for a Frobenius-normalised
    matrix. CUDA bf16 matrices run on the tcgen05 GEMM with the 0.5 folded into ``alpha`` and ``3I -`` into the
    epilogue (``alpha = -1`` plus an additive ``3I`` term): two launches per iteration."""
    rows, cols = y.shape
    right = cols <= rows
    if not y.is_cuda:
        yf = y.float()
        for _ in range(iters):
            if right:
                g = 3 * torch.eye(cols) - yf.t() @ yf
                yf = 0.5 * yf @ g
            else:
                g = 3 * torch.eye(rows) - yf @ yf.t()
                yf = 0.5 * g @ yf
        return yf.to(y.dtype)
    eye3 = _three_eye(cols if right else rows, y.device)
    for _ in range(iters):
        if right:
            g = gemm(y, y, a_mn=True, b_mn=True, alpha=-1.0, aux=eye3, add_aux=True)     # 3I - Y^T Y  [cols, cols], one launch
            y = gemm(y, g, b_mn=True, alpha=0.5)                 # Y G
        else:
            g = gemm(y, y, alpha=-1.0, aux=eye3, add_aux=True)   # 3I - Y Y^T  [rows, rows]
            y = gemm(g, y, b_mn=True, alpha=0.5)                 # G Y
    return y


_EYE3: Dict[tuple, torch.Tensor] = {}


def _three_eye(n: int, device) -> torch.Tensor:
    """``3 I`` in bf16, kept per size: the additive term of the Newton-Schulz product's epilogue."""
    key = (n, str(device))
    t = _EYE3.get(key)
    if t is None:
        t = (3.0 * torch.eye(n, device=device)).to(torch.bfloat16)
        _EYE3[key] = t
    return t


class Muon(_Base):
    """Momentum + Newton-Schulz orthogonalisation for the 2-D parameters listed in ``indices``."""

    def __init__(self, flat, pc=None, zero_stage=0, lr=1e-4, momentum=0.95, iterations=5, max_grad_norm=1.0, indices=None):
        super().__init__(flat, pc, 0, lr, 0.0, max_grad_norm)      # matrices are updated whole: no state sharding
        self.momentum, self.iterations = momentum, iterations
        self.indices = list(range(len(flat.params))) if indices is None else list(indices)
        self.m = torch.zeros(flat.numel, dtype=torch.float32, device=flat.device)

    def _update(self) -> None:
        f = self.flat
        for i in self.indices:
            p = f.params[i]
            o, n = f.offsets[i], p.numel()
            g = f.grads[o:o + n]
            m = self.m[o:o + n]
            master = self.master[o:o + n]
            rows, cols = p.shape[0], p.numel() // p.shape[0]
            if g.is_cuda:
                st = stream_ptr(g)
                y = torch.empty(n, dtype=torch.bfloat16, device=g.device)
                lib.call("elfa_muon_momentum", m, g, _ptype(g), y, n, float(self.momentum), self.scalars, self.part, None, st)
                if rows % 8 == 0 and cols % 8 == 0:
                    y2 = newton_schulz(y.view(rows, cols), self.iterations)
                else:
                    # the tensor-core GEMM wants multiples of 8: zero rows / columns change nothing (they stay zero through
                    # every Y <- 0.5 Y (3I - Y^T Y) step and add nothing to Y^T Y)
                    pr, pc_ = (rows + 7) // 8 * 8, (cols + 7) // 8 * 8
                    yp = torch.zeros((pr, pc_), dtype=torch.bfloat16, device=g.device)
                    yp[:rows, :cols] = y.view(rows, cols)
                    y2 = newton_schulz(yp, self.iterations)[:rows, :cols]
                pout = None if self.master_is_param else p.data.view(-1)
                lib.call("elfa_muon_apply", pout, 0 if pout is None else 1, master, y2.contiguous(), n,
                         -1.0 if self.lr_on_device else float(self.lr), self.scalars, st)
            else:
                if self.skipped():
                    continue
                m.mul_(self.momentum).add_(g.float() * float(self.scalars[1]))
                nrm = float(m.norm())
                if nrm < 1e-8:
                    master.sub_(self.lr * m)
                else:
                    y = newton_schulz((m / nrm).view(rows, cols), self.iterations)
                    master.sub_(self.lr * y.reshape(-1))
                if not self.master_is_param:
                    p.data.view(-1).copy_(master.to(p.dtype))

    def state_tensors(self):
        d = {"m": self.m}
        if not self.master_is_param:
            d["master"] = self.master
        return d


class LionMuon:
    """The reference's default optimizer: 2-D parameters → Muon, everything else → Lion."""

    def __init__(self, flat, pc=None, zero_stage=0, lr=1e-4, lion_betas=(0.95, 0.98), weight_decay=0.1, muon_momentum=0.95,
                 muon_iterations=5, max_grad_norm=1.0):
        idx2d = [i for i, p in enumerate(flat.params) if p.dim() == 2]
        lion_ranges = []
        for i, p in enumerate(flat.params):
            if p.dim() != 2:
                o = flat.offsets[i]
                lion_ranges.append((o, o + p.numel(), not getattr(p, "no_decay", False) and p.dim() >= 2))
        self.muon = Muon(flat, pc, 0, lr, muon_momentum, muon_iterations, max_grad_norm, idx2d)
        self.lion = Lion(flat, pc, 0, lr, lion_betas, weight_decay, max_grad_norm, ranges=lion_ranges)
        # both halves share the master copy and the clip scalars
        self.lion.master, self.lion.scalars = self.muon.master, self.muon.scalars
        self.flat, self.pc = flat, self.muon.pc
        self.step_count = 0
        self.lr = lr
        self._graph = None

    @property
    def loss_scale(self):
        return self.muon.loss_scale

    @loss_scale.setter
    def loss_scale(self, v):
        self.muon.loss_scale = v
        self.lion.loss_scale = v

    @property
    def scalars(self):
        return self.muon.scalars

    def _updates(self) -> None:
        self.muon._update()
        self.lion._update()

    def step(self, lr: Optional[float] = None) -> None:
        """The update itself is hundreds to thousands of small launches (momentum, 2 x iterations Newton-Schulz products and
        an apply per matrix). On a GPU it is captured once into a CUDA graph - after one eager step that has loaded every
        kernel and filled the caches - and replayed afterwards; the learning rate travels through the device scalars.
        ``ELFA_OPT_GRAPH=0`` keeps it eager."""
        if lr is not None:
            self.lr = lr
        self.muon.lr = self.lion.lr = self.lr
        self.flat.fold_autograd_grads()
        self.muon.reduce_gradients()
        self.muon._norm_and_clip()
        self.step_count += 1
        self.muon.step_count = self.lion.step_count = self.step_count
        import os
        use_graph = self.flat.flat.is_cuda and os.environ.get("ELFA_OPT_GRAPH", "1") not in ("0", "")
        if not use_graph or self.step_count == 1:
            self._updates()
        else:
            self.muon.scalars[4] = float(self.lr)
            if self._graph is None:
                self.muon.lr_on_device = self.lion.lr_on_device = True
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._updates()
                self._graph = g
            self._graph.replay()
        from ..quant.qat import new_weight_epoch
        new_weight_epoch()

    def zero_grad(self):
        self.flat.zero_grad()

    def grad_norm(self):
        return self.muon.grad_norm()

    def skipped(self):
        return self.muon.skipped()

    def state_dict(self):
        return {"step": self.step_count, "muon": self.muon.state_dict(), "lion": self.lion.state_dict()}

    def load_state_dict(self, sd):
        self.step_count = int(sd["step"])
        self.muon.load_state_dict(sd["muon"])
        self.lion.load_state_dict(sd["lion"])
        self.lion.master = self.muon.master


def build_optimizer(cfg, flat: FlatParams, pc: Optional[ParallelContext] = None):
    """Optimizer selected by ``training.optimizer`` (lion | muon | lion_muon | adamw)."""
    t = cfg.training
    z = cfg.runtime.zero_stage
    if getattr(flat, "presharded", False) and t.optimizer in ("muon", "lion_muon"):
        raise ValueError("ZeRO stage 3 shards parameters element-wise: use the adamw or lion optimizer (Muon needs whole matrices)")
    if t.optimizer == "adamw":
        return AdamW(flat, pc, z, t.learning_rate, (t.adam_beta1, t.adam_beta2), t.adam_eps, t.weight_decay, t.gradient_clip)
    if t.optimizer == "lion":
        return Lion(flat, pc, z, t.learning_rate, (t.lion_beta1, t.lion_beta2), t.weight_decay, t.gradient_clip)
    if t.optimizer == "muon":
        idx = [i for i, p in enumerate(flat.params) if p.dim() == 2]
        return Muon(flat, pc, z, t.learning_rate, t.muon_momentum, t.muon_iterations, t.gradient_clip, idx)
    return LionMuon(flat, pc, z, t.learning_rate, (t.lion_beta1, t.lion_beta2), t.weight_decay, t.muon_momentum, t.muon_iterations,
                    t.gradient_clip)
