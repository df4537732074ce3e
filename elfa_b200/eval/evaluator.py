"""Perplexity, long-context sweep, generation and the forward-throughput micro-benchmark.

reference: ``src/eval/evaluator.zig:269-319`` (perplexity = exp of the token-weighted mean loss over
non-shuffled windows of ``seq_len``), ``:321-377`` (sweep over context lengths), ``:419-470`` (greedy and
temperature / top-p generation, which re-runs the whole prefix for every token), ``:472-529``
(nucleus sampling: softmax(logits / T) in f64, sort descending, smallest prefix with mass >= top_p,
sample proportionally inside it), ``:532-590`` (2 warm-up + 10 timed forward passes → tokens/s).
Generation here reuses per-layer state for the EFLA family (constant cost per token) and falls
back to prefix recomputation for the attention family.
"""
from __future__ import annotations

import math
import time
from typing import Dict, List, Optional

import torch

from ..data import BinaryDataset, DataLoader


def sample_top_p(logits: torch.Tensor, temperature: float = 1.0, top_p: float = 0.9,
                 generator: Optional[torch.Generator] = None) -> int:
    """Nucleus sampling of one token id from a 1-D logits vector."""
    if temperature <= 0:
        return int(torch.argmax(logits))
    probs = torch.softmax(logits.double() / temperature, -1)
    sp, si = torch.sort(probs, descending=True)
    cum = torch.cumsum(sp, 0)
    cutoff = int(torch.searchsorted(cum, torch.tensor(top_p, dtype=cum.dtype, device=cum.device)).item()) + 1
    cutoff = max(1, min(cutoff, sp.numel()))
    head = sp[:cutoff] / sp[:cutoff].sum()
    idx = torch.multinomial(head, 1, generator=generator)
    return int(si[idx])


class Evaluator:
    def __init__(self, model, cfg, device):
        self.model, self.cfg, self.device = model, cfg, device

    @torch.no_grad()
    def _loss(self, ids: torch.Tensor, tgt: torch.Tensor) -> float:
        self.model.eval()
        loss = self.model(ids.to(self.device), tgt.to(self.device))
        return float(loss)

    def evaluate_perplexity(self, data_path_or_dataset, seq_len: Optional[int] = None, max_tokens: Optional[int] = None) -> Dict[str, float]:
        ds = BinaryDataset.open(data_path_or_dataset) if isinstance(data_path_or_dataset, str) else data_path_or_dataset
        S = seq_len or self.cfg.data.seq_len
        loader = DataLoader(ds, 1, S, shuffle=False, pin_memory=False)
        tot_loss, tot_tok = 0.0, 0
        for b in loader:
            tot_loss += self._loss(b.input, b.target) * b.num_tokens
            tot_tok += b.num_tokens
            if max_tokens is not None and tot_tok >= max_tokens:
                break
        mean = tot_loss / max(tot_tok, 1)
        return {"loss": mean, "perplexity": math.exp(min(mean, 50.0)), "tokens": tot_tok}

    def evaluate_long_context(self, dataset, lengths: List[int]) -> List[Dict[str, float]]:
        out = []
        for n in lengths:
            if n + 1 > len(dataset):
                break
            r = self.evaluate_perplexity(dataset, seq_len=n, max_tokens=n)
            r["context"] = n
            out.append(r)
        return out


class Generator:
    def __init__(self, model, tokenizer=None, device=None):
        self.model, self.tok = model, tokenizer
        self.device = device or next(model.parameters()).device

    @torch.no_grad()
    def generate_ids(self, prompt_ids: List[int], max_new_tokens: int = 256, temperature: float = 1.0, top_p: float = 0.9,
                     seed: Optional[int] = None, eos_id: Optional[int] = None) -> List[int]:
        self.model.eval()
        gen = None
        if seed is not None:
            gen = torch.Generator(device="cpu").manual_seed(seed)
        ids = list(prompt_ids) or [0]
        stateful = hasattr(self.model, "forward_with_states")
        if stateful and len(ids) + max_new_tokens > getattr(self.model, "max_positions", 1 << 62):
            stateful = False        # learned positions run out: slide a window over the context instead
        states = None
        if stateful:
            logits, states = self.model.forward_with_states(torch.tensor([ids], device=self.device), None)
            last = logits[0, -1]
        max_ctx = self.model.cfg.data.seq_len
        for _ in range(max_new_tokens):
            if not stateful:
                ctx = ids[-max_ctx:]
                last = self.model(torch.tensor([ctx], device=self.device))[0, -1]
            nxt = sample_top_p(last.float().cpu(), temperature, top_p, gen)
            ids.append(nxt)
            if eos_id is not None and nxt == eos_id:
                break
            if stateful:
                logits, states = self.model.forward_with_states(torch.tensor([[nxt]], device=self.device), states)
                last = logits[0, -1]
        return ids

    def generate_greedy(self, prompt_ids, max_new_tokens=256):
        return self.generate_ids(prompt_ids, max_new_tokens, temperature=0.0)

    def generate(self, prompt: str, max_new_tokens: int = 256, temperature: float = 1.0, top_p: float = 0.9, seed=None) -> str:
        if self.tok is None:
            raise ValueError("a tokenizer is required for text generation")
        ids = self.generate_ids(self.tok.encode(prompt), max_new_tokens, temperature, top_p, seed)
        return self.tok.decode(ids)


@torch.no_grad()
def benchmark_throughput(model, batch: int, seq_len: int, vocab: int, device, warmup: int = 2, iters: int = 10) -> float:
    """Forward-only tokens/s, timed on the device when it is a GPU."""
    model.eval()
    ids = torch.randint(0, vocab, (batch, seq_len), device=device)
    tgt = torch.randint(0, vocab, (batch, seq_len), device=device)
    for _ in range(warmup):
        model(ids, tgt)
    if device.type == "cuda":
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            model(ids, tgt)
        e1.record()
        torch.cuda.synchronize()
        dt = e0.elapsed_time(e1) / 1e3
    else:
        t0 = time.time()
        for _ in range(iters):
            model(ids, tgt)
        dt = time.time() - t0
    return batch * seq_len * iters / max(dt, 1e-9)
