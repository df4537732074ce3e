"""Library baseline arm: the benchmark GPT written in eager PyTorch, with every GEMM a ``torch.matmul`` (cuBLAS / cuBLASLt),
attention through ``scaled_dot_product_attention``, norms / GELU / cross-entropy through ``torch.nn.functional``, AdamW through
``torch.optim.AdamW(fused=True)`` and every collective an NCCL call of ``torch.distributed``.

It restates, without this framework's kernels or engine, the unfused sequences the reference's parallel code describes
(reference: ``src/distributed/tensor_parallel.zig:77-170`` all-gather → GEMM and GEMM → all-reduce;
``src/distributed/sequence_parallel.zig:79-200`` sequence split / gather / reduce-scatter;
``src/distributed/zero_sharding.zig:115-181`` reduce-scatter gradients → scale → optimizer → all-gather parameters;
``kernels/cuda/gemm.cu:212-232`` ``cublasGemmEx``; ``src/quantization/stable_qat.zig:52-106`` fake-quant before the GEMM).
Same model, initial weights, data, parallel layout (tensor + sequence parallel groups of neighbouring ranks, data parallel
across them, ZeRO stage from the file) and hyper-parameters as the product arm; selected with ``bench.py --impl baseline``.

Quantisation-aware training is fake-quant in plain PyTorch ops (``elfa_b200.quant.formats``) followed by the bf16 matmul,
which is what the reference's StableQAT + cuBLAS path amounts to. ZeRO stage 3 uses ``torch.distributed.fsdp.fully_shard``.
"""
from __future__ import annotations

import math
import os
import sys
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from elfa_b200.parallel import tp as tpl  # noqa: E402  (shard_param only: pure tensor slicing)
from elfa_b200.quant import formats  # noqa: E402


# ----------------------------------------------------------------------------------------- collectives with autograd
def _ag0(x, group):
    n = dist.get_world_size(group)
    out = torch.empty((x.shape[0] * n, *x.shape[1:]), dtype=x.dtype, device=x.device)
    if x.is_cuda:
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    else:
        parts = [torch.empty_like(x) for _ in range(n)]
        dist.all_gather(parts, x.contiguous(), group=group)
        out = torch.cat(parts, 0)
    return out


def _rs0(x, group):
    n = dist.get_world_size(group)
    r = dist.get_rank(group)
    m = x.shape[0] // n
    x = x.contiguous()
    if x.is_cuda:
        out = torch.empty((m, *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x, group=group)
        return out
    dist.all_reduce(x, group=group)
    return x[r * m:(r + 1) * m].clone()


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _ag0(x, group)

    @staticmethod
    def backward(ctx, g):
        return _rs0(g, ctx.group), None


class _ScatterSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _rs0(x, group)

    @staticmethod
    def backward(ctx, g):
        return _ag0(g, ctx.group), None


# ----------------------------------------------------------------------------------------- quantisation-aware linear
_wcache: Dict[tuple, torch.Tensor] = {}


def _fq(x, fmt, axis):
    if fmt == "mxfp8":
        return formats.mxfp8_fake_quant_ref(x, axis)
    if fmt == "nvfp4":
        return formats.nvfp4_fake_quant_ref(x, axis)
    raise ValueError(f"baseline arm: quantisation format '{fmt}' is not restated here")


def _fq_weight(w, fmt, axis):
    key = (id(w), fmt, axis)
    hit = _wcache.get(key)
    if hit is None:
        hit = _fq(w.detach(), fmt, axis)
        _wcache[key] = hit
    return hit


class _QatLinear(torch.autograd.Function):
    """``fq(x) @ fq(w)`` with straight-through gradients; with ``bwd`` the output gradient and the weight's output axis are
    MXFP8-quantised for the input gradient, as ``quant.backward: mxfp8`` does in the product arm."""

    @staticmethod
    def forward(ctx, x2, w, fmt, bwd):
        xq = _fq(x2, fmt, 1)
        wq = _fq_weight(w, fmt, 0)
        ctx.save_for_backward(xq, wq)
        ctx.w, ctx.bwd = w, bwd
        return torch.matmul(xq, wq)

    @staticmethod
    def backward(ctx, dy):
        xq, wq = ctx.saved_tensors
        if ctx.bwd:
            dy = _fq(dy, "mxfp8", 1)
            wq = _fq_weight(ctx.w, "mxfp8", 1)
        return torch.matmul(dy, wq.t()), torch.matmul(xq.t(), dy), None, None


def linear(x2, w, fmt, bwd):
    return torch.matmul(x2, w) if fmt == "none" else _QatLinear.apply(x2, w, fmt, bwd)


# ----------------------------------------------------------------------------------------- vocabulary-parallel loss
class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, group, vocab_lo, denom):
        lf = logits.float()
        m = lf.max(-1).values
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        e = torch.exp(lf - m.unsqueeze(-1))
        s = e.sum(-1)
        Vl = lf.shape[-1]
        lt = targets - vocab_lo
        mine = (lt >= 0) & (lt < Vl)
        tl = torch.where(mine, lf.gather(-1, lt.clamp(0, Vl - 1).unsqueeze(-1)).squeeze(-1), torch.zeros_like(m))
        pack = torch.stack([s, tl], 0)
        dist.all_reduce(pack, group=group)
        s, tl = pack[0], pack[1]
        loss = (torch.log(s) + m - tl).sum() / denom
        p = e / s.unsqueeze(-1)
        p[mine, lt[mine]] -= 1.0
        ctx.save_for_backward((p / denom).to(logits.dtype))
        return loss

    @staticmethod
    def backward(ctx, g):
        (p,) = ctx.saved_tensors
        return p * g, None, None, None, None


# ----------------------------------------------------------------------------------------- model
class BaselineBlock(nn.Module):
    def __init__(self, D, F_local, H_local, hd, norm, dtype, device):
        super().__init__()
        mk = lambda *s: nn.Parameter(torch.empty(*s, dtype=dtype, device=device))
        self.ln1_w, self.ln2_w = nn.Parameter(torch.ones(D, dtype=dtype, device=device)), nn.Parameter(torch.ones(D, dtype=dtype, device=device))
        self.ln1_b = nn.Parameter(torch.zeros(D, dtype=dtype, device=device)) if norm == "layernorm" else None
        self.ln2_b = nn.Parameter(torch.zeros(D, dtype=dtype, device=device)) if norm == "layernorm" else None
        self.w_qkv, self.w_o = mk(D, 3 * H_local * hd), mk(H_local * hd, D)
        self.up, self.down = mk(D, F_local), mk(F_local, D)
        self.H, self.hd, self.norm = H_local, hd, norm


class BaselineGPT(nn.Module):
    def __init__(self, cfg, tp_group, tp_size: int, tp_rank: int, device):
        super().__init__()
        m = cfg.model
        if m.activation != "gelu" or not cfg.bench.learned_positions or not m.tie_embeddings:
            raise ValueError("baseline arm: restated for the benchmark family (GELU MLP, learned positions, tied embeddings)")
        self.cfg, self.tp_group, self.tp, self.r = cfg, tp_group, tp_size, tp_rank
        dtype = {"fp32": torch.float32, "bf16": torch.bfloat16}[m.dtype]
        D, Fd, V = m.hidden_dim, m.intermediate_dim, m.vocab_size
        self.Vl = V // tp_size
        self.vocab_lo = tp_rank * self.Vl
        self.embed = nn.Parameter(torch.empty(self.Vl, D, dtype=dtype, device=device))
        self.pos = nn.Parameter(torch.empty(min(m.max_seq_len, max(cfg.data.seq_len, 1)), D, dtype=dtype, device=device))
        self.blocks = nn.ModuleList([BaselineBlock(D, Fd // tp_size, m.num_heads // tp_size, m.head_dim, m.norm_type, dtype, device)
                                     for _ in range(m.num_layers)])
        self.fn_w = nn.Parameter(torch.ones(D, dtype=dtype, device=device))
        self.fn_b = nn.Parameter(torch.zeros(D, dtype=dtype, device=device)) if m.norm_type == "layernorm" else None
        self.q_attn, self.q_mlp, self.q_bwd = cfg.quant.attention, cfg.quant.mlp, cfg.quant.backward == "mxfp8"
        self._init(cfg.runtime.seed, device)
        for p in self.replicated():
            p.tp_replicated = True

    def replicated(self) -> List[nn.Parameter]:
        out = [self.pos, self.fn_w] + ([self.fn_b] if self.fn_b is not None else [])
        for b in self.blocks:
            out += [p for p in (b.ln1_w, b.ln1_b, b.ln2_w, b.ln2_b) if p is not None]
        return out

    @torch.no_grad()
    def _init(self, seed, device):
        """The product arm's initial weights: full tensors drawn in the same order from the same generator, then sliced."""
        m, tp, r = self.cfg.model, self.tp, self.r
        g = torch.Generator(device=device).manual_seed(seed)
        std = self.cfg.bench.init_std
        D, Fd = m.hidden_dim, m.intermediate_dim
        draw = lambda shape, sigma: torch.randn(shape, generator=g, dtype=torch.float32, device=device) * sigma
        emb = draw((m.vocab_size, D), std if std > 0 else math.sqrt(1.0 / D))
        self.embed.copy_(emb[self.vocab_lo:self.vocab_lo + self.Vl])
        self.pos.copy_(draw(tuple(self.pos.shape), std if std > 0 else math.sqrt(1.0 / D)))
        s_in = std if std > 0 else math.sqrt(2.0 / D)
        for b in self.blocks:
            b.w_qkv.copy_(tpl.shard_param(draw((D, 3 * D), s_in), "col_qkv", tp, r))
            b.w_o.copy_(tpl.shard_param(draw((D, D), s_in), "row", tp, r))
            b.up.copy_(tpl.shard_param(draw((D, Fd), s_in), "col", tp, r))
            b.down.copy_(tpl.shard_param(draw((Fd, D), std if std > 0 else math.sqrt(2.0 / Fd)), "row", tp, r))

    def _norm(self, x, w, b):
        if b is not None:
            return F.layer_norm(x, (x.shape[-1],), w, b, 1e-5)
        return F.rms_norm(x, (x.shape[-1],), w, 1e-6)

    def forward(self, ids, targets, denom):
        """ids, targets ``[B, S]`` → mean cross-entropy. Activations are ``[S(/tp), B, D]`` (sequence parallel between blocks)."""
        tp, grp = self.tp, self.tp_group
        B, S = ids.shape
        ids_sb = ids.t()
        if tp > 1:
            lt = ids_sb - self.vocab_lo
            mine = (lt >= 0) & (lt < self.Vl)
            x = F.embedding(lt.clamp(0, self.Vl - 1), self.embed) * mine.unsqueeze(-1).to(self.embed.dtype)
            x = _ScatterSum.apply(x, grp)                                    # [S/tp, B, D]
            Sl = S // tp
            x = x + self.pos[self.r * Sl:(self.r + 1) * Sl].unsqueeze(1)
        else:
            x = F.embedding(ids_sb, self.embed) + self.pos[:S].unsqueeze(1)
        D = x.shape[-1]
        for b in self.blocks:
            n = self._norm(x, b.ln1_w, b.ln1_b)
            if tp > 1:
                n = _GatherSeq.apply(n, grp)                                 # [S, B, D]
            qkv = linear(n.reshape(-1, D), b.w_qkv, self.q_attn, self.q_bwd).view(S, B, 3, b.H, b.hd)
            q, k, v = (qkv[:, :, i].permute(1, 2, 0, 3) for i in range(3))   # [B, H, S, hd]
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True).permute(2, 0, 1, 3).reshape(S * B, b.H * b.hd)
            a = linear(o, b.w_o, self.q_attn, self.q_bwd).view(S, B, D)
            x = x + (_ScatterSum.apply(a, grp) if tp > 1 else a)
            n = self._norm(x, b.ln2_w, b.ln2_b)
            if tp > 1:
                n = _GatherSeq.apply(n, grp)
            h = F.gelu(linear(n.reshape(-1, D), b.up, self.q_mlp, self.q_bwd), approximate="tanh")
            f = linear(h, b.down, self.q_mlp, self.q_bwd).view(S, B, D)
            x = x + (_ScatterSum.apply(f, grp) if tp > 1 else f)
        n = self._norm(x, self.fn_w, self.fn_b)
        t_sb = targets.t().reshape(-1)
        if tp > 1:
            n = _GatherSeq.apply(n, grp)
            logits = torch.matmul(n.reshape(-1, D), self.embed.t())
            return _VocabParallelCE.apply(logits, t_sb, grp, self.vocab_lo, denom)
        logits = torch.matmul(n.reshape(-1, D), self.embed.t())
        return F.cross_entropy(logits.float(), t_sb, reduction="sum") / denom


# ----------------------------------------------------------------------------------------- trainer
class BaselineTrainer:
    """Same step protocol as ``elfa_b200.trainer.Trainer``: ``train_step(batches) -> device loss``, ``finish_step -> float``."""

    def __init__(self, cfg, device):
        self.cfg, self.device = cfg, device
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        tp = min(cfg.runtime.tensor_parallel_size, world)
        dp = world // tp
        self.world, self.rank, self.tp, self.dp = world, rank, tp, dp
        self.tp_rank, self.dp_rank = rank % tp, rank // tp
        self.tp_group = self.dp_group = None
        if world > 1:
            for d in range(dp):      # neighbouring ranks form a tensor-parallel group
                g = dist.new_group([d * tp + t for t in range(tp)])
                if d == self.dp_rank:
                    self.tp_group = g
            for t in range(tp):
                g = dist.new_group([d * tp + t for d in range(dp)])
                if t == self.tp_rank:
                    self.dp_group = g
        torch.manual_seed(cfg.runtime.seed)
        self.model = BaselineGPT(cfg, self.tp_group, tp, self.tp_rank, device)
        self.stage = cfg.runtime.zero_stage if dp > 1 else 0
        t = cfg.training
        self.lr, self.clip = t.learning_rate, t.gradient_clip
        self.accum = cfg.accumulation_steps()
        self.step = 0
        if self.stage == 3:
            self._init_fsdp(t)
        else:
            self._init_flat(t)

    # ---- ZeRO 0 / 1 / 2: flat buffers, fp32 gradient accumulation, sharded fused AdamW on fp32 master weights
    def _init_flat(self, t):
        params = [p for p in self.model.parameters()]
        rep = [p for p in params if getattr(p, "tp_replicated", False)]
        rest = [p for p in params if not getattr(p, "tp_replicated", False)]
        order = [p for p in rep if p.dim() >= 2] + [p for p in rep if p.dim() < 2] + [p for p in rest if p.dim() >= 2] + [p for p in rest if p.dim() < 2]
        self.params = order
        self.rep_numel = sum(p.numel() for p in rep)
        n = sum(p.numel() for p in order)
        q = self.dp * 256
        self.numel = (n + q - 1) // q * q
        dev, dt = self.device, order[0].dtype
        self.pflat = torch.zeros(self.numel, dtype=dt, device=dev)
        self.gflat = torch.zeros(self.numel, dtype=torch.float32, device=dev)
        off = 0
        self.decay_mask_ranges = []
        for p in order:
            k = p.numel()
            self.pflat[off:off + k].copy_(p.data.reshape(-1))
            p.data = self.pflat[off:off + k].view(p.shape)
            gview = self.gflat[off:off + k].view(p.shape)

            def hook(param, gview=gview):
                gview.add_(param.grad)          # fp32 accumulation across micro-batches
                param.grad = None
            p.register_post_accumulate_grad_hook(hook)
            self.decay_mask_ranges.append((off, off + k, p.dim() >= 2))
            off += k
        sharded = self.stage >= 1
        shard = self.numel // self.dp
        self.lo, self.hi = (self.dp_rank * shard, (self.dp_rank + 1) * shard) if sharded else (0, self.numel)
        self.master = self.pflat[self.lo:self.hi].float()
        groups = []
        self._opt_views = []
        for a, b, wd in self._runs(self.lo, self.hi):
            mp = nn.Parameter(self.master[a - self.lo:b - self.lo])
            mp.grad = self.gflat[a:b]
            self._opt_views.append((mp, a, b))
            groups.append({"params": [mp], "weight_decay": t.weight_decay if wd else 0.0})
        self.opt = torch.optim.AdamW(groups, lr=t.learning_rate, betas=(t.adam_beta1, t.adam_beta2), eps=t.adam_eps,
                                     fused=self.device.type == "cuda")

    def _runs(self, lo, hi):
        out = []
        for a, b, wd in self.decay_mask_ranges + [(sum(p.numel() for p in self.params), self.numel, False)]:
            a, b = max(a, lo), min(b, hi)
            if a >= b:
                continue
            if out and out[-1][2] == wd and out[-1][1] == a:
                out[-1] = (out[-1][0], b, wd)
            else:
                out.append((a, b, wd))
        return out

    def _init_fsdp(self, t):
        from torch.distributed.device_mesh import init_device_mesh
        from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
        if self.tp != 1:
            raise ValueError("baseline arm: ZeRO stage 3 (fully_shard) is restated for pure data parallelism")
        self.model = self.model.float()        # fp32 master parameters, bf16 compute / fp32 reduction by policy
        mesh = init_device_mesh(self.device.type, (self.world,))
        mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16 if self.cfg.model.dtype == "bf16" else None, reduce_dtype=torch.float32)
        for b in self.model.blocks:
            fully_shard(b, mesh=mesh, mp_policy=mp)
        fully_shard(self.model, mesh=mesh, mp_policy=mp)
        decay = [p for p in self.model.parameters() if p.dim() >= 2]
        nodecay = [p for p in self.model.parameters() if p.dim() < 2]
        self.opt = torch.optim.AdamW([{"params": decay, "weight_decay": t.weight_decay}, {"params": nodecay, "weight_decay": 0.0}],
                                     lr=t.learning_rate, betas=(t.adam_beta1, t.adam_beta2), eps=t.adam_eps, fused=self.device.type == "cuda")

    def make_loader(self):
        """The product arm's synthetic data stream (same seed, same sharding over the data-parallel ranks)."""
        from elfa_b200.data import DataLoader, SyntheticDataset
        cfg = self.cfg
        S, mb = cfg.data.seq_len, cfg.training.micro_batch_size
        kind = cfg.bench.synthetic if cfg.bench.synthetic != "none" else "uniform"
        need = S * mb * self.accum * self.dp * 4 + 1
        ds = SyntheticDataset(cfg.model.vocab_size, max(need, S * 64 + 1), kind, cfg.bench.data_seed, cfg.bench.zipf_s)
        return DataLoader(ds, mb, S, shuffle=False, seed=cfg.runtime.seed, dp_rank=self.dp_rank, dp_size=self.dp)

    # ---- one optimizer step
    def train_step(self, batches) -> torch.Tensor:
        _wcache.clear()
        total = None
        n_micro = len(batches)
        if self.stage == 3:
            self.opt.zero_grad(set_to_none=True)
        else:
            self.gflat.zero_()
        for b in batches:
            ids = b.input.to(self.device, non_blocking=True)
            tgt = b.target.to(self.device, non_blocking=True)
            loss = self.model(ids, tgt, float(tgt.numel() * n_micro))
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        if self.stage == 3:
            if self.clip > 0:
                torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.clip)
            self.opt.step()
            self.step += 1
            return total
        g = self.gflat
        if self.tp > 1 and self.rep_numel:
            dist.all_reduce(g[:self.rep_numel], group=self.tp_group)
        if self.dp > 1:
            if self.stage >= 1 and g.is_cuda:
                dist.reduce_scatter_tensor(g[self.lo:self.hi], g, op=dist.ReduceOp.AVG, group=self.dp_group)
            else:
                dist.all_reduce(g, group=self.dp_group)
                g.div_(self.dp)
        gs = g[self.lo:self.hi]
        rep_hi = min(max(self.rep_numel, self.lo), self.hi)
        sq = torch.linalg.vector_norm(gs[rep_hi - self.lo:]).double() ** 2          # no full-size temporaries
        if self.tp_rank == 0 and rep_hi > self.lo:
            sq = sq + torch.linalg.vector_norm(gs[:rep_hi - self.lo]).double() ** 2
        if self.world > 1 and (self.tp > 1 or self.stage >= 1):
            dist.all_reduce(sq, group=None if self.stage >= 1 else self.tp_group)
        norm = sq.sqrt().float()
        if self.clip > 0:
            gs.mul_(torch.clamp(self.clip / (norm + 1e-6), max=1.0))
        self.opt.step()
        self.pflat[self.lo:self.hi].copy_(self.master)
        if self.stage >= 1:
            dist.all_gather_into_tensor(self.pflat, self.pflat[self.lo:self.hi].clone(), group=self.dp_group)
        self.step += 1
        return total

    def finish_step(self, loss_dev: torch.Tensor) -> float:
        loss = float(loss_dev)
        if self.dp > 1:
            t = torch.tensor([loss], device=self.device)
            dist.all_reduce(t, group=self.dp_group)
            loss = float(t) / self.dp
        return loss
