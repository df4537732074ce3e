"""Evaluation harness: token accuracy, perplexity, needle-in-a-haystack recall / precision and
ROUGE-1/2/L for long-form summaries (reference: ``src/evaluation/harness.zig:43-448``)."""
from __future__ import annotations

import math
from collections import Counter
from typing import Dict, List, Sequence

import torch


def lcs_length(a: Sequence, b: Sequence) -> int:
    if not a or not b:
        return 0
    prev = [0] * (len(b) + 1)
    for x in a:
        cur = [0]
        for j, y in enumerate(b, 1):
            cur.append(prev[j - 1] + 1 if x == y else max(prev[j], cur[j - 1]))
        prev = cur
    return prev[-1]


def _f1(overlap: int, n_ref: int, n_hyp: int) -> Dict[str, float]:
    p = overlap / n_hyp if n_hyp else 0.0
    r = overlap / n_ref if n_ref else 0.0
    f = 2 * p * r / (p + r) if p + r > 0 else 0.0
    return {"precision": p, "recall": r, "f1": f}


def rouge_n(ref: Sequence, hyp: Sequence, n: int = 1) -> Dict[str, float]:
    def grams(s):
        return Counter(tuple(s[i:i + n]) for i in range(len(s) - n + 1))
    gr, gh = grams(ref), grams(hyp)
    overlap = sum((gr & gh).values())
    return _f1(overlap, sum(gr.values()), sum(gh.values()))


def rouge_l(ref: Sequence, hyp: Sequence) -> Dict[str, float]:
    return _f1(lcs_length(ref, hyp), len(ref), len(hyp))


class EvalHarness:
    def __init__(self, model, device):
        self.model, self.device = model, device

    @torch.no_grad()
    def token_accuracy(self, ids: torch.Tensor, targets: torch.Tensor) -> float:
        self.model.eval()
        logits = self.model(ids.to(self.device))
        pred = logits.argmax(-1).cpu()
        return float((pred == targets).float().mean())

    @torch.no_grad()
    def perplexity(self, ids: torch.Tensor, targets: torch.Tensor) -> float:
        self.model.eval()
        return math.exp(min(float(self.model(ids.to(self.device), targets.to(self.device))), 50.0))

    @torch.no_grad()
    def greedy_decode(self, prompt: List[int], n: int) -> List[int]:
        from .evaluator import Generator
        return Generator(self.model, None, self.device).generate_greedy(prompt, n)[len(prompt):]

    def needle_recall(self, cases) -> Dict[str, float]:
        """Each case: haystack token ids ending in the query, answer ids. Recall = fraction of answer
        tokens reproduced in order, precision = fraction of generated tokens that are answer tokens."""
        rec, prec = [], []
        for c in cases:
            out = self.greedy_decode(c.tokens, len(c.answer))
            hit = lcs_length(c.answer, out)
            rec.append(hit / max(len(c.answer), 1))
            prec.append(hit / max(len(out), 1))
        n = max(len(rec), 1)
        return {"recall": sum(rec) / n, "precision": sum(prec) / n, "cases": len(rec)}

    def summary_rouge(self, cases, max_new_tokens: int = 64) -> Dict[str, float]:
        agg = {"rouge1": 0.0, "rouge2": 0.0, "rougeL": 0.0}
        for c in cases:
            out = self.greedy_decode(c.document, max_new_tokens)
            agg["rouge1"] += rouge_n(c.reference, out, 1)["f1"]
            agg["rouge2"] += rouge_n(c.reference, out, 2)["f1"]
            agg["rougeL"] += rouge_l(c.reference, out)["f1"]
        n = max(len(cases), 1)
        return {k: v / n for k, v in agg.items()}
