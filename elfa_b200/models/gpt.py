"""Pre-norm GPT decoder: learned positions, causal softmax attention, GELU MLP, tied embeddings.

This is the attention-mixer family selected by ``model.efla.enabled: false`` (the reference's
gen-1 distributed/quantisation code operates on exactly this QKVO + FFN parameter set:
reference ``src/distributed/zero_sharding.zig:73-99``, ``src/quantization/stable_qat.zig:36-50``;
attention math: ``src/futhark/attention.fut:28-51``). Block structure mirrors the reference block
(``src/model/model.zig:229-272``): norm → mixer → residual → norm → MLP → residual.

Tensor parallelism (Megatron style, with sequence parallelism): QKV and MLP-up are column
parallel, attention-out and MLP-down are row parallel, embeddings are vocabulary parallel, and the
residual stream / norms hold ``S/tp`` tokens per rank. Internal activation layout is
``[S, B, D]`` (sequence first) so that sequence shards are contiguous.

Parameter names (checkpoint keys) extend the reference's naming style
(``src/model/model.zig:512-537``): ``embed_tokens.weight``, ``pos_embed.weight``,
``blocks.{i}.ln1.{weight,bias}``, ``blocks.{i}.attn.w_qkv``, ``blocks.{i}.attn.w_o``,
``blocks.{i}.ln2.{weight,bias}``, ``blocks.{i}.mlp_up.weight``, ``blocks.{i}.mlp_down.weight``,
``final_norm.{weight,bias}``, ``lm_head.weight`` (untied only). Linear weights are ``[in, out]``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..config import Config
from ..parallel.mesh import ParallelContext
from ..parallel import tp as tpl
from ..quant.qat import QuantSpec


def _dtype(name: str) -> torch.dtype:
    return {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16, "fp8_e4m3": torch.bfloat16}[name]


class Norm(nn.Module):
    def __init__(self, dim: int, kind: str, dtype, device):
        super().__init__()
        self.kind = ops.LAYERNORM if kind == "layernorm" else ops.RMSNORM
        self.eps = 1e-5 if kind == "layernorm" else 1e-6
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device)) if kind == "layernorm" else None
        self.weight.no_decay = True
        self.weight.tp_replicated = True
        if self.bias is not None:
            self.bias.no_decay = True
            self.bias.tp_replicated = True

    def forward(self, x, residual=None):
        return ops.norm(x, self.weight, self.bias, eps=self.eps, kind=self.kind, residual=residual)


def _attend_cached(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """``q [s, B, H, hd]`` (the last ``s`` positions) against ``k, v [t, B, H, hd]`` (all positions so far), causal;
    fp32 math on a handful of rows. Returns ``[s, B, H * hd]``."""
    s_, B, H, hd = q.shape
    t = k.shape[0]
    sc = torch.einsum("sbhd,tbhd->bhst", q.float(), k.float()) / math.sqrt(hd)
    if s_ > 1:
        future = torch.arange(t, device=q.device)[None, :] > (torch.arange(s_, device=q.device)[:, None] + (t - s_))
        sc = sc.masked_fill(future, float("-inf"))
    o = torch.einsum("bhst,tbhd->sbhd", torch.softmax(sc, -1), v.float())
    return o.reshape(s_, B, H * hd).to(q.dtype)


class Attention(nn.Module):
    def __init__(self, cfg: Config, pc: ParallelContext, dtype, device, init_std: float, out_std: float):
        super().__init__()
        m = cfg.model
        self.pc = pc
        self.n_heads = m.num_heads // pc.tp_size
        self.n_kv_heads = m.num_kv_heads // pc.tp_size          # grouped-query attention when smaller than n_heads
        self.gqa = m.num_kv_heads != m.num_heads
        self.head_dim = m.head_dim
        D = m.hidden_dim
        local = self.n_heads * self.head_dim
        self.w_qkv = nn.Parameter(torch.empty(D, (self.n_heads + 2 * self.n_kv_heads) * self.head_dim, dtype=dtype, device=device))
        self.w_o = nn.Parameter(torch.empty(local, D, dtype=dtype, device=device))
        self.w_qkv.tp_shard = (f"col_gqa:{m.num_heads}:{m.num_kv_heads}:{m.head_dim}" if self.gqa else "col_qkv", pc.tp_size)
        self.w_o.tp_shard = ("row", pc.tp_size)
        self.init_std, self.out_std = init_std, out_std
        self.quant = QuantSpec.from_config(cfg.quant.attention, cfg.quant)

    def forward(self, x, cache: Optional[dict] = None, doc_start: Optional[torch.Tensor] = None):   # x: [S(/tp), B, D]
        h = tpl.column_parallel_linear(x, self.w_qkv, self.pc, quant=self.quant)      # [S, B, (H + 2 Hkv) * hd]
        S, B = h.shape[0], h.shape[1]
        H, Hkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        if self.gqa:
            qkv = h.view(S, B, H + 2 * Hkv, hd)                   # heads [query | key | value]
            q, k, v = qkv[:, :, :H], qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:]
        else:
            qkv = h.view(S, B, 3, H, hd)
            q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        if cache is not None and cache.get("k") is not None:
            # incremental decoding: the new rows attend to the cached keys / values and, causally, to each other
            k_all = torch.cat((cache["k"], k), 0)
            v_all = torch.cat((cache["v"], v), 0)
            cache["k"], cache["v"] = k_all, v_all
            rep = H // Hkv
            o = _attend_cached(q, k_all.repeat_interleave(rep, 2) if rep > 1 else k_all, v_all.repeat_interleave(rep, 2) if rep > 1 else v_all)
            return tpl.row_parallel_linear(o, self.w_o, self.pc, quant=self.quant)
        if cache is not None:        # prefill: the ordinary kernel, and keep what decoding will need
            cache["k"], cache["v"] = k.contiguous(), v.contiguous()
        if self.pc.cp_size > 1:
            if self.gqa or doc_start is not None:
                raise ValueError("context parallelism is implemented for num_kv_heads == num_heads and unpacked sequences")
            if self.pc.cp_mode == "ulysses":     # all-to-all to whole sequences of H / cp heads and back
                from ..parallel.ulysses import ulysses_attention
                o = ulysses_attention(qkv, self.pc.cp_group, causal=True)
            else:                                # the sequence is split over the context-parallel group: keys / values travel the ring
                from ..parallel.ring_attention import ring_attention
                o = ring_attention(qkv, self.pc.cp_group, causal=True, seq_first=True, zigzag=self.pc.cp_mode == "zigzag")
        else:
            o = ops.attention(qkv, causal=True, seq_first=True, num_heads=H if self.gqa else None, doc_start=doc_start)   # [S, B, local]
        return tpl.row_parallel_linear(o, self.w_o, self.pc, quant=self.quant)        # [S(/tp), B, D]


class MLP(nn.Module):
    def __init__(self, cfg: Config, pc: ParallelContext, dtype, device):
        super().__init__()
        m = cfg.model
        self.pc = pc
        D, F = m.hidden_dim, m.intermediate_dim // pc.tp_size
        self.act = m.activation
        self.gated = m.activation == "swiglu"
        self.up = nn.Parameter(torch.empty(D, F * (2 if self.gated else 1), dtype=dtype, device=device))
        self.down = nn.Parameter(torch.empty(F, D, dtype=dtype, device=device))
        self.up.tp_shard = ("col", pc.tp_size)
        self.down.tp_shard = ("row", pc.tp_size)
        self.quant = QuantSpec.from_config(cfg.quant.mlp, cfg.quant)

    def forward(self, x):
        if self.gated:
            h = tpl.column_parallel_linear(x, self.up, self.pc, quant=self.quant)
            g, u = h.chunk(2, dim=-1)
            a = ops.activation(g.contiguous(), "silu") * u
        elif self.act == "gelu":
            a = tpl.column_parallel_linear(x, self.up, self.pc, act="gelu", quant=self.quant)
        else:
            a = ops.activation(tpl.column_parallel_linear(x, self.up, self.pc, quant=self.quant), self.act)
        return tpl.row_parallel_linear(a, self.down, self.pc, quant=self.quant)


class Block(nn.Module):
    def __init__(self, cfg: Config, pc: ParallelContext, dtype, device, init_std, out_std):
        super().__init__()
        m = cfg.model
        self.ln1 = Norm(m.hidden_dim, m.norm_type, dtype, device)
        self.attn = Attention(cfg, pc, dtype, device, init_std, out_std)
        self.ln2 = Norm(m.hidden_dim, m.norm_type, dtype, device)
        self.mlp = MLP(cfg, pc, dtype, device)
        self.dropout = m.dropout

    def gemm_weights(self):
        """The parameters that are read only as the right-hand operand of ``ops.linear`` (no tensor parallelism, no
        quantiser in front of them): under ZeRO stage 3 their forward product can fetch them itself."""
        a, m = self.attn, self.mlp
        plain = a.pc.tp_size == 1 and not (a.quant is not None and a.quant.enabled) and not (m.quant is not None and m.quant.enabled)
        return [a.w_qkv, a.w_o, m.up, m.down] if plain else []

    def forward(self, x, pending, cache: Optional[dict] = None, doc_start: Optional[torch.Tensor] = None):
        """``pending`` is the previous sub-layer's output that has not been added to the residual
        stream yet; the add is fused into the next norm kernel. ``cache``: this layer's key / value cache
        when decoding incrementally. ``doc_start``: packed sequences (see ``ops.attention``)."""
        n, x = self.ln1(x, pending)
        a = self.attn(n, cache, doc_start)
        if self.dropout > 0 and self.training:
            a = torch.nn.functional.dropout(a, self.dropout)
        n, x = self.ln2(x, a)
        f = self.mlp(n)
        if self.dropout > 0 and self.training:
            f = torch.nn.functional.dropout(f, self.dropout)
        return x, f


class GPTModel(nn.Module):
    def __init__(self, cfg: Config, pc: Optional[ParallelContext] = None, device=None):
        super().__init__()
        self.cfg = cfg
        self.pc = pc or ParallelContext()
        m = cfg.model
        dtype = _dtype(m.dtype)
        self.dtype = dtype
        tp = self.pc.tp_size
        if m.vocab_size % tp or m.num_heads % tp or m.intermediate_dim % tp:
            raise ValueError("vocab_size, num_heads and intermediate_dim must be divisible by the tensor-parallel size")
        if m.num_kv_heads <= 0 or m.num_heads % m.num_kv_heads or m.num_kv_heads % tp:
            raise ValueError(f"model.num_kv_heads ({m.num_kv_heads}) must divide model.num_heads ({m.num_heads}) and be divisible by the "
                             f"tensor-parallel size ({tp})")
        self.vocab_local = m.vocab_size // tp
        self.vocab_lo = self.pc.tp_rank * self.vocab_local
        D = m.hidden_dim
        std = cfg.bench.init_std
        self.embed_tokens = nn.Parameter(torch.empty(self.vocab_local, D, dtype=dtype, device=device))
        self.embed_tokens.tp_shard = ("vocab", tp)
        self.pos_embed = None
        if cfg.bench.learned_positions:
            self.pos_embed = nn.Parameter(torch.empty(min(m.max_seq_len, max(cfg.data.seq_len, 1)), D, dtype=dtype, device=device))
            self.pos_embed.tp_replicated = True
        out_std = std if std > 0 else math.sqrt(2.0 / D)
        self.blocks = nn.ModuleList([Block(cfg, self.pc, dtype, device, std, out_std) for _ in range(m.num_layers)])
        self.final_norm = Norm(D, m.norm_type, dtype, device)
        self.lm_head = None
        if not m.tie_embeddings:
            self.lm_head = nn.Parameter(torch.empty(self.vocab_local, D, dtype=dtype, device=device))
            self.lm_head.tp_shard = ("vocab", tp)
        if tp > 1 and not self.pc.sequence_parallel:
            # without sequence parallelism every rank normalises all tokens: the norm parameters get the same full gradient
            # everywhere (no reduction), unlike the position table, which only the first vocabulary shard adds
            for mod in self.modules():
                if isinstance(mod, Norm):
                    for p in (mod.weight, mod.bias):
                        if p is not None:
                            p.tp_replicated, p.tp_identical = False, True
        self.reset_parameters(cfg.runtime.seed)

    # ------------------------------------------------------------------ init
    def reset_parameters(self, seed: int) -> None:
        """N(0, init_std) when ``bench.init_std > 0``; otherwise the reference's He-style defaults
        (Linear sigma = sqrt(2/in), Embedding sigma = sqrt(1/dim): reference ``src/nn/layers.zig:336,446``).
        Full (unsharded) tensors are drawn from one generator and sliced, so a TP run starts from
        the same weights as a single-GPU run."""
        m, tp, r = self.cfg.model, self.pc.tp_size, self.pc.tp_rank
        dev = self.embed_tokens.device
        g = torch.Generator(device=dev).manual_seed(seed)
        std = self.cfg.bench.init_std
        D = m.hidden_dim

        def draw(shape, sigma):
            return torch.randn(shape, generator=g, dtype=torch.float32, device=dev) * sigma

        def put(p, full):
            with torch.no_grad():
                p.copy_(full.to(p.dtype))

        emb = draw((m.vocab_size, D), std if std > 0 else math.sqrt(1.0 / D))
        put(self.embed_tokens, emb[self.vocab_lo:self.vocab_lo + self.vocab_local])
        if self.pos_embed is not None:
            put(self.pos_embed, draw(tuple(self.pos_embed.shape), std if std > 0 else math.sqrt(1.0 / D)))
        F = m.intermediate_dim
        for blk in self.blocks:
            s_in = std if std > 0 else math.sqrt(2.0 / D)
            wqkv = draw((D, (m.num_heads + 2 * m.num_kv_heads) * m.head_dim), s_in)
            put(blk.attn.w_qkv, tpl.shard_param(wqkv, blk.attn.w_qkv.tp_shard[0], tp, r))
            put(blk.attn.w_o, tpl.shard_param(draw((m.num_heads * m.head_dim, D), s_in), "row", tp, r))
            gated = 2 if blk.mlp.gated else 1
            up = draw((D, F * gated), s_in)
            put(blk.mlp.up, tpl.shard_param(up, "col_gated" if blk.mlp.gated else "col", tp, r))
            put(blk.mlp.down, tpl.shard_param(draw((F, D), std if std > 0 else math.sqrt(2.0 / F)), "row", tp, r))
        if self.lm_head is not None:
            head = draw((m.vocab_size, D), std if std > 0 else math.sqrt(2.0 / D))
            put(self.lm_head, head[self.vocab_lo:self.vocab_lo + self.vocab_local])

    # ------------------------------------------------------------------ names
    def named_checkpoint_parameters(self):
        """Yields ``(checkpoint_name, parameter)`` in a fixed order."""
        yield "embed_tokens.weight", self.embed_tokens
        if self.pos_embed is not None:
            yield "pos_embed.weight", self.pos_embed
        for i, b in enumerate(self.blocks):
            yield f"blocks.{i}.ln1.weight", b.ln1.weight
            if b.ln1.bias is not None:
                yield f"blocks.{i}.ln1.bias", b.ln1.bias
            yield f"blocks.{i}.attn.w_qkv", b.attn.w_qkv
            yield f"blocks.{i}.attn.w_o", b.attn.w_o
            yield f"blocks.{i}.ln2.weight", b.ln2.weight
            if b.ln2.bias is not None:
                yield f"blocks.{i}.ln2.bias", b.ln2.bias
            yield f"blocks.{i}.mlp_up.weight", b.mlp.up
            yield f"blocks.{i}.mlp_down.weight", b.mlp.down
        yield "final_norm.weight", self.final_norm.weight
        if self.final_norm.bias is not None:
            yield "final_norm.bias", self.final_norm.bias
        if self.lm_head is not None:
            yield "lm_head.weight", self.lm_head

    def count_parameters(self) -> int:
        """Parameters of the full (unsharded) model."""
        n = 0
        for _, p in self.named_checkpoint_parameters():
            k = p.numel()
            if hasattr(p, "tp_shard"):
                k *= p.tp_shard[1]
            n += k
        return n

    # ---------------------------------------------------------------- forward
    def hidden_states(self, ids: torch.Tensor, pos0: int = 0, caches: Optional[list] = None,
                      doc_start: Optional[torch.Tensor] = None) -> torch.Tensor:
        """ids ``[B, S]`` → final-norm output ``[S(/tp), B, D]``. ``doc_start [B, S]`` int32 (packed sequences): positions
        restart at every document and attention stays inside a document."""
        pc = self.pc
        ids_sb = ids.t().contiguous()                        # [S, B]
        if doc_start is not None:
            x = ops.embedding(ids_sb, self.embed_tokens, None, 0, self.vocab_lo, seq_first=True, vocab_total=self.cfg.model.vocab_size)
            if self.pos_embed is not None and self.vocab_lo == 0:      # the vocabulary-parallel sum adds the positions once
                S = ids_sb.shape[0]
                pos = (torch.arange(S, device=ids.device)[None, :] - doc_start.long()).t().clamp_(0, self.pos_embed.shape[0] - 1)
                x = x + self.pos_embed[pos]
        elif isinstance(pos0, (tuple, list)):
            # the local sequence is several equal segments of the whole one (zig-zag context parallelism): one offset each
            n = ids_sb.shape[0] // len(pos0)
            x = torch.cat([ops.embedding(ids_sb[i * n:(i + 1) * n].contiguous(), self.embed_tokens, self.pos_embed, int(p0), self.vocab_lo,
                                         seq_first=True, vocab_total=self.cfg.model.vocab_size) for i, p0 in enumerate(pos0)], 0)
        else:
            x = ops.embedding(ids_sb, self.embed_tokens, self.pos_embed, pos0, self.vocab_lo, seq_first=True,
                              vocab_total=self.cfg.model.vocab_size)  # [S, B, D]
        x = tpl.embedding_reduce(x, pc)                      # sum over vocab shards → [S(/tp), B, D]
        pending = None
        for i, blk in enumerate(self.blocks):
            if caches is not None:
                x, pending = blk(x, pending, caches[i])
            elif self.cfg.bench.activation_checkpointing and self.training:
                x, pending = torch.utils.checkpoint.checkpoint(blk, x, pending, None, doc_start, use_reentrant=False)
            else:
                x, pending = blk(x, pending, None, doc_start)
        n, _ = self.final_norm(x, pending)
        return n

    @property
    def max_positions(self) -> int:
        return self.cfg.model.max_seq_len

    def forward_with_states(self, ids: torch.Tensor, states: Optional[dict] = None):
        """Incremental decoding on one rank: ids ``[B, T]`` (the prompt, then one or a few new tokens per call) →
        (logits ``[B, T, V]``, states). ``states`` holds the position reached and a key / value cache per layer; the
        first call (``states=None``) runs the ordinary attention kernel over the prompt, later calls attend to the
        cache. The learned positions end at ``max_positions``.
        (reference: ``src/eval/evaluator.zig:419-470`` generates by running the whole context again for every token.)"""
        assert self.pc.tp_size == 1 and self.pc.cp_size == 1, "incremental decoding runs on one rank"
        if states is None:
            states = {"pos": 0, "layers": [{"k": None, "v": None} for _ in self.blocks]}
        if states["pos"] + ids.shape[1] > self.max_positions:
            raise ValueError(f"position {states['pos'] + ids.shape[1]} is past the model's {self.max_positions} learned positions")
        n = self.hidden_states(ids, states["pos"], states["layers"])
        states["pos"] += ids.shape[1]
        head = self.lm_head if self.lm_head is not None else self.embed_tokens
        return tpl.vocab_parallel_logits(n, head, self.pc, gather=True).transpose(0, 1), states

    def forward(self, ids: torch.Tensor, targets: Optional[torch.Tensor] = None, pos0: int = 0,
                loss_denominator: Optional[float] = None, grad_scale: float = 1.0, doc_start: Optional[torch.Tensor] = None):
        """Returns logits ``[B, S, V]`` when ``targets`` is None (single-rank only), else the mean
        cross-entropy over ``targets`` ``[B, S]`` (label smoothing from the config). ``doc_start``: packed sequences."""
        n = self.hidden_states(ids, pos0, None, doc_start)
        head = self.lm_head if self.lm_head is not None else self.embed_tokens
        if targets is None:
            logits = tpl.vocab_parallel_logits(n, head, self.pc, gather=True)    # [S, B, V]
            return logits.transpose(0, 1)
        logits = tpl.vocab_parallel_logits(n, head, self.pc, gather=False)       # [S, B, V/tp]
        t_sb = targets.t().contiguous()
        return tpl.vocab_parallel_cross_entropy(logits, t_sb, self.pc, self.vocab_lo, self.cfg.model.vocab_size,
                                                self.cfg.training.label_smoothing, loss_denominator, grad_scale)
