"""The reference's own model family: pre-RMSNorm decoder whose token mixer is EFLA followed by
PRISM, then a GELU MLP.

Block (reference ``src/model/model.zig:229-272``)::

    n = norm1(x); e = EFLA(n); q = PRISM(n, e); r = x + q; out = r + W_down gelu(W_up norm2(r))

Model: token embedding → blocks → final norm → logits (``lm_head`` or tied embedding).
Parameter names and shapes follow the reference checkpoint layout (``model.zig:512-537``):
``embed_tokens.weight [V, D]``, per block ``blocks.{i}.ln1.weight``, ``.efla.w_k / .w_v [D, H*d]``,
``.efla.w_o [H*d, D]``, ``.efla.beta_param [1] (fp32)``, ``.prism.w_beta.{j} / .w_k.{j} / .w_p.{j} [D, d]``,
``.prism.shortconv.weight [D, W]`` (``.bias``), ``.ln2.weight``, ``.mlp_up.weight [D, I]``,
``.mlp_down.weight [I, D]``, then ``final_norm.weight`` and ``lm_head.weight`` when untied.
Initialisation uses the reference's He-style sigmas (``src/model/efla.zig:148``, ``prism.zig:163,889``,
``src/nn/layers.zig:336,446``) unless ``bench.init_std`` overrides them.

``forward_with_states`` streams a long sequence block by block, carrying the EFLA state (and the
ShortConv tail) per layer - the reference's route to very long contexts
(``model.zig:415-454``, ``efla.zig:681-733``).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn as nn

from .. import ops
from ..config import Config
from ..ops import efla as eops
from ..parallel import tp as tpl
from ..parallel.mesh import ParallelContext
from .gpt import Norm, _dtype


def _identical(*params):
    """Marks parameters that every tensor-parallel rank holds in full and differentiates on the same activations."""
    for p in params:
        if p is not None:
            p.tp_identical = True


class EflaLayer(nn.Module):
    """Tensor parallel over the heads: ``w_k`` / ``w_v`` column shards (this rank's heads), ``w_o`` the matching row shard whose
    partial products are summed over the group; the scan runs on the local heads only (reference: per-head weights
    ``src/model/efla.zig:149-156``, layer shard dims ``src/tensor/sharding.zig:183-222``). ``beta`` is shared by all heads:
    replicated, its gradient summed over the group."""

    def __init__(self, cfg: Config, dtype, device, pc: Optional[ParallelContext] = None):
        super().__init__()
        m = cfg.model
        self.pc = pc or ParallelContext()
        tp = self.pc.tp_size
        self.H, self.d = m.num_heads // tp, m.head_dim
        D = m.hidden_dim
        self.w_k = nn.Parameter(torch.empty(D, self.H * self.d, dtype=dtype, device=device))
        self.w_v = nn.Parameter(torch.empty(D, self.H * self.d, dtype=dtype, device=device))
        self.w_o = nn.Parameter(torch.empty(self.H * self.d, D, dtype=dtype, device=device))
        self.learned_beta = m.efla.learned_beta
        self.beta_param = nn.Parameter(torch.full((1,), float(m.efla.initial_beta), dtype=torch.float32, device=device),
                                       requires_grad=m.efla.learned_beta)
        self.beta_param.no_decay = True
        if tp > 1:
            self.w_k.tp_shard = self.w_v.tp_shard = ("col", tp)
            self.w_o.tp_shard = ("row", tp)
            self.beta_param.tp_replicated = True
        self.chunk = max(1, min(m.efla.chunk_size, 16)) if m.efla.use_chunked_scan else 16

    def forward(self, x, state=None, sp_group=None):
        B, T, D = x.shape
        k = tpl.column_parallel_linear(x, self.w_k, self.pc).view(B, T, self.H, self.d)
        v = tpl.column_parallel_linear(x, self.w_v, self.pc).view(B, T, self.H, self.d)
        if sp_group is not None:
            # sequence parallel: the state at the start of this rank's token block is the composition of the
            # affine maps of the ranks before it (exact for the delta rule)
            from ..parallel import sp
            state = sp.efla_cross_rank_state(k, v, self.beta_param, sp_group)
        o, s = eops.efla_scan(k, v, self.beta_param, state, self.chunk)
        return tpl.row_parallel_linear(o.reshape(B, T, self.H * self.d).to(x.dtype), self.w_o, self.pc), s


class PrismLayer(nn.Module):
    def __init__(self, cfg: Config, dtype, device):
        super().__init__()
        m = cfg.model
        D, d, L = m.hidden_dim, m.head_dim, m.prism.num_iterations
        self.d, self.L, self.forget = d, L, m.prism.forget_factor
        self.w_beta = nn.ParameterList([nn.Parameter(torch.empty(D, d, dtype=dtype, device=device)) for _ in range(L)])
        self.w_k = nn.ParameterList([nn.Parameter(torch.empty(D, d, dtype=dtype, device=device)) for _ in range(L)])
        self.w_p = nn.ParameterList([nn.Parameter(torch.empty(D, d, dtype=dtype, device=device)) for _ in range(L)])
        self.conv_weight = nn.Parameter(torch.empty(D, m.prism.shortconv_window, dtype=dtype, device=device))
        self.conv_bias = nn.Parameter(torch.zeros(D, dtype=dtype, device=device))
        self.conv_bias.no_decay = True
        # small per-channel work on the full hidden state: replicated under tensor parallelism
        _identical(self.conv_weight, self.conv_bias, *self.w_beta, *self.w_k, *self.w_p)

    def forward(self, x, v, carry_state: Optional[torch.Tensor] = None, conv_tail: Optional[torch.Tensor] = None, sp_group=None):
        """x: normed hidden ``[B, T, D]``, v: EFLA output. Returns (y, new_state or None, new conv tail)."""
        W = self.conv_weight.shape[1]
        if sp_group is not None and W > 1:
            from ..parallel import sp
            conv_tail = sp.halo_from_left(x, W - 1, sp_group)      # the left neighbour's last W-1 positions (zeros on rank 0)
        xin = x if conv_tail is None else torch.cat([conv_tail, x], dim=1)
        u = eops.shortconv(xin, self.conv_weight, self.conv_bias)
        if conv_tail is not None:
            u = u[:, conv_tail.shape[1]:]
        new_tail = xin[:, -(W - 1):].detach() if W > 1 else None
        ps = [torch.sigmoid(ops.linear(u, self.w_p[l]).float()) for l in range(self.L)]
        y = eops.prism_refine(u, v, ps, self.d)
        new_state = None
        if carry_state is not None:
            with torch.no_grad():
                B, T, D = u.shape
                G = D // self.d
                r = (v.float() - u.float()).view(B, T, G, self.d)
                deltas, betas, ks = [], [], []
                for l in range(self.L):
                    delta = ops.gelu_tanh_ref(ps[l].unsqueeze(2) * r)
                    r = r - delta
                    deltas.append(delta)
                    betas.append(torch.sigmoid(ops.linear(u, self.w_beta[l]).float().mean(-1)))
                    kk = ops.linear(u, self.w_k[l]).float()
                    nrm = kk.norm(dim=-1, keepdim=True)
                    ks.append(kk / torch.where(nrm < 1e-12, torch.ones_like(nrm), nrm))
                new_state = eops.prism_state_update(carry_state, deltas, betas, ks, self.forget)
        return y, new_state, new_tail


class EflaBlock(nn.Module):
    def __init__(self, cfg: Config, dtype, device, pc: Optional[ParallelContext] = None):
        super().__init__()
        m = cfg.model
        self.pc = pc or ParallelContext()
        tp = self.pc.tp_size
        self.ln1 = Norm(m.hidden_dim, m.norm_type, dtype, device)
        self.efla = EflaLayer(cfg, dtype, device, self.pc)
        self.prism = PrismLayer(cfg, dtype, device) if m.prism.enabled else None
        self.ln2 = Norm(m.hidden_dim, m.norm_type, dtype, device)
        self.mlp_up = nn.Parameter(torch.empty(m.hidden_dim, m.intermediate_dim // tp, dtype=dtype, device=device))
        self.mlp_down = nn.Parameter(torch.empty(m.intermediate_dim // tp, m.hidden_dim, dtype=dtype, device=device))
        if tp > 1:
            self.mlp_up.tp_shard, self.mlp_down.tp_shard = ("col", tp), ("row", tp)
        for n_ in (self.ln1, self.ln2):        # every rank normalises all tokens: identical gradients, no reduction
            n_.weight.tp_replicated = False
            if n_.bias is not None:
                n_.bias.tp_replicated = False
            _identical(n_.weight, n_.bias)
        self.act = "gelu" if m.activation in ("gelu", "swiglu") else m.activation

    def forward(self, x, states=None, sp_group=None):
        n, _ = self.ln1(x)
        e_state = states["efla"] if states is not None else None
        e, e_state = self.efla(n, e_state, sp_group)
        if self.prism is not None:
            q, p_state, tail = self.prism(n, e, states["prism"] if states is not None else None,
                                          states.get("conv_tail") if states is not None else None, sp_group)
        else:
            q, p_state, tail = e, None, None
        n2, r = self.ln2(q, x)                 # fused: r = x + q, n2 = norm2(r)
        if self.act == "gelu":
            h = tpl.column_parallel_linear(n2, self.mlp_up, self.pc, act="gelu")
        else:
            h = ops.activation(tpl.column_parallel_linear(n2, self.mlp_up, self.pc), self.act)
        out = r + tpl.row_parallel_linear(h, self.mlp_down, self.pc)
        new_states = None
        if states is not None:
            new_states = {"efla": e_state, "prism": p_state, "conv_tail": tail}
        return out, new_states


class EflaModel(nn.Module):
    def __init__(self, cfg: Config, pc: Optional[ParallelContext] = None, device=None):
        super().__init__()
        self.cfg = cfg
        pc = pc or ParallelContext()
        # tensor parallel without sequence parallelism: activations [B, T, D] are whole on every rank (the scan and the
        # ShortConv need every token of a sequence), heads / MLP columns / vocabulary rows are sharded
        import dataclasses
        self.pc = dataclasses.replace(pc, sequence_parallel=False) if pc.tp_size > 1 else pc
        m = cfg.model
        tp = self.pc.tp_size
        if m.num_heads % tp or m.intermediate_dim % tp or m.vocab_size % tp:
            raise ValueError("num_heads, intermediate_dim and vocab_size must be divisible by the tensor-parallel size")
        dtype = _dtype(m.dtype)
        self.dtype = dtype
        self.vocab_local = m.vocab_size // tp
        self.vocab_lo = self.pc.tp_rank * self.vocab_local
        self.embed_tokens = nn.Parameter(torch.empty(self.vocab_local, m.hidden_dim, dtype=dtype, device=device))
        self.blocks = nn.ModuleList([EflaBlock(cfg, dtype, device, self.pc) for _ in range(m.num_layers)])
        self.final_norm = Norm(m.hidden_dim, m.norm_type, dtype, device)
        self.final_norm.weight.tp_replicated = False
        if self.final_norm.bias is not None:
            self.final_norm.bias.tp_replicated = False
        _identical(self.final_norm.weight, self.final_norm.bias)
        self.lm_head = None if m.tie_embeddings else nn.Parameter(torch.empty(self.vocab_local, m.hidden_dim, dtype=dtype, device=device))
        if tp > 1:
            self.embed_tokens.tp_shard = ("vocab", tp)
            if self.lm_head is not None:
                self.lm_head.tp_shard = ("vocab", tp)
        self.reset_parameters(cfg.runtime.seed)

    def reset_parameters(self, seed: int) -> None:
        """Full (unsharded) tensors are drawn from one generator in a fixed order and sliced, so a tensor-parallel run
        starts from the weights of the single-rank run."""
        m = self.cfg.model
        tp, r = self.pc.tp_size, self.pc.tp_rank
        dev = self.embed_tokens.device
        g = torch.Generator(device=dev).manual_seed(seed)
        std = self.cfg.bench.init_std
        D, I, Hd = m.hidden_dim, m.intermediate_dim, m.num_heads * m.head_dim

        def fill(p, sigma, full_shape=None):
            shape = tuple(full_shape) if full_shape is not None else tuple(p.shape)
            full = torch.randn(shape, generator=g, dtype=torch.float32, device=dev) * (std if std > 0 else sigma)
            shard = getattr(p, "tp_shard", None)
            if shard is not None and tp > 1:
                full = tpl.shard_param(full, shard[0], tp, r)
            with torch.no_grad():
                p.copy_(full.to(p.dtype))

        fill(self.embed_tokens, math.sqrt(1.0 / D), (m.vocab_size, D))
        for b in self.blocks:
            for w in (b.efla.w_k, b.efla.w_v):
                fill(w, math.sqrt(2.0 / D), (D, Hd))
            fill(b.efla.w_o, math.sqrt(2.0 / D), (Hd, D))
            if b.prism is not None:
                for lst in (b.prism.w_beta, b.prism.w_k, b.prism.w_p):
                    for w in lst:
                        fill(w, math.sqrt(2.0 / D))
                fill(b.prism.conv_weight, math.sqrt(1.0 / b.prism.conv_weight.shape[1]))
            fill(b.mlp_up, math.sqrt(2.0 / D), (D, I))
            fill(b.mlp_down, math.sqrt(2.0 / I), (I, D))
        if self.lm_head is not None:
            fill(self.lm_head, math.sqrt(2.0 / D), (m.vocab_size, D))

    def named_checkpoint_parameters(self):
        yield "embed_tokens.weight", self.embed_tokens
        for i, b in enumerate(self.blocks):
            yield f"blocks.{i}.ln1.weight", b.ln1.weight
            if b.ln1.bias is not None:
                yield f"blocks.{i}.ln1.bias", b.ln1.bias
            yield f"blocks.{i}.efla.w_k", b.efla.w_k
            yield f"blocks.{i}.efla.w_v", b.efla.w_v
            yield f"blocks.{i}.efla.w_o", b.efla.w_o
            if b.efla.learned_beta:
                yield f"blocks.{i}.efla.beta_param", b.efla.beta_param
            if b.prism is not None:
                for j, w in enumerate(b.prism.w_beta):
                    yield f"blocks.{i}.prism.w_beta.{j}", w
                for j, w in enumerate(b.prism.w_k):
                    yield f"blocks.{i}.prism.w_k.{j}", w
                for j, w in enumerate(b.prism.w_p):
                    yield f"blocks.{i}.prism.w_p.{j}", w
                yield f"blocks.{i}.prism.shortconv.weight", b.prism.conv_weight
                yield f"blocks.{i}.prism.shortconv.bias", b.prism.conv_bias
            yield f"blocks.{i}.ln2.weight", b.ln2.weight
            if b.ln2.bias is not None:
                yield f"blocks.{i}.ln2.bias", b.ln2.bias
            yield f"blocks.{i}.mlp_up.weight", b.mlp_up
            yield f"blocks.{i}.mlp_down.weight", b.mlp_down
        yield "final_norm.weight", self.final_norm.weight
        if self.final_norm.bias is not None:
            yield "final_norm.bias", self.final_norm.bias
        if self.lm_head is not None:
            yield "lm_head.weight", self.lm_head

    def count_parameters(self) -> int:
        """Parameters of the full (unsharded) model."""
        return sum(p.numel() * (p.tp_shard[1] if hasattr(p, "tp_shard") else 1) for _, p in self.named_checkpoint_parameters())

    def init_states(self, batch: int) -> List[dict]:
        m = self.cfg.model
        dev = self.embed_tokens.device
        G = m.hidden_dim // m.head_dim
        return [{"efla": torch.zeros(batch, m.num_heads // self.pc.tp_size, m.head_dim, m.head_dim, device=dev),
                 "prism": torch.zeros(batch, G, m.head_dim, m.head_dim, device=dev) if m.prism.enabled else None,
                 "conv_tail": None} for _ in self.blocks]

    def _embed(self, ids: torch.Tensor) -> torch.Tensor:
        x = ops.embedding(ids, self.embed_tokens, None, 0, self.vocab_lo, seq_first=False, vocab_total=self.cfg.model.vocab_size)
        return tpl.embedding_reduce(x, self.pc)           # sum of the vocabulary shards' partial embeddings

    def _logits(self, n: torch.Tensor, gather: bool) -> torch.Tensor:
        head = self.lm_head if self.lm_head is not None else self.embed_tokens
        return tpl.vocab_parallel_logits(n, head, self.pc, gather=gather)

    def hidden_states(self, ids: torch.Tensor, states: Optional[List[dict]] = None, sp_group=None):
        x = self._embed(ids)
        new_states = [] if states is not None else None
        for i, blk in enumerate(self.blocks):
            x, ns = blk(x, states[i] if states is not None else None, sp_group)
            if new_states is not None:
                new_states.append(ns)
        n, _ = self.final_norm(x)
        return n, new_states

    def forward_sequence_parallel(self, ids_local: torch.Tensor, group=None) -> torch.Tensor:
        """Long-context forward with the sequence split over ``group``: ``ids_local [B, T / world]`` is this rank's
        contiguous token block; returns its logits. Per layer the ranks exchange the ShortConv halo (window - 1 normed
        positions from the left neighbour) and the EFLA state as an affine prefix, so the result equals the
        single-rank forward of the whole sequence. Both exchanges are differentiable: ``forward(..., sp_group=...)`` trains
        through them (``runtime.context_parallel_size`` in the trainer).
        reference: ``src/distributed/sequence_parallel.zig:54-77,202-240`` (split, boundary exchange); the reference never
        connects them to its model."""
        x = self._embed(ids_local)
        for blk in self.blocks:
            x, _ = blk(x, None, group if group is not None else torch.distributed.group.WORLD)
        n, _ = self.final_norm(x)
        return self._logits(n, gather=True)

    def forward_with_states(self, ids: torch.Tensor, states: Optional[List[dict]] = None):
        """ids ``[B, T]`` → (logits ``[B, T, V]``, per-layer states) for streaming / generation."""
        if states is None:
            states = self.init_states(ids.shape[0])
        n, states = self.hidden_states(ids, states)
        return self._logits(n, gather=True), states

    def forward(self, ids: torch.Tensor, targets: Optional[torch.Tensor] = None, pos0: int = 0,
                loss_denominator: Optional[float] = None, grad_scale: float = 1.0, sp_group=None):
        """``sp_group``: ``ids`` is this rank's contiguous block of a sequence split over the group (sequence-parallel
        training: the EFLA state and the ShortConv halo cross the ranks, forward and backward)."""
        n, _ = self.hidden_states(ids, None, sp_group)
        if targets is None:
            return self._logits(n, gather=True)
        logits = self._logits(n, gather=False)
        return tpl.vocab_parallel_cross_entropy(logits, targets, self.pc, self.vocab_lo, self.cfg.model.vocab_size,
                                                self.cfg.training.label_smoothing, loss_denominator, grad_scale)
