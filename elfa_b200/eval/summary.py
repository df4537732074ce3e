"""Synthetic long-form summarisation cases and heuristic scores (reference:
``src/evaluation/long_form_summary.zig:16-224``: documents built from topic vocabularies with a
reference summary, scored for coherence, coverage and conciseness)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List

import numpy as np

N_TOPICS = 10


@dataclass
class SummaryCase:
    document: List[int]
    reference: List[int]
    topic: int


def generate_summary_case(length: int, vocab: int, seed: int, summary_len: int = 32) -> SummaryCase:
    """A document whose tokens come mostly from one topic's slice of the vocabulary; the reference
    summary is the topic's most frequent tokens in order of first appearance."""
    rng = np.random.default_rng(seed)
    topic = int(rng.integers(0, N_TOPICS))
    span = max((vocab - 4) // N_TOPICS, 8)
    lo = 4 + topic * span
    core = rng.integers(lo, lo + span, size=max(summary_len, 8))
    doc = np.where(rng.random(length) < 0.7, rng.choice(core, size=length), rng.integers(4, vocab, size=length))
    seen, ref = set(), []
    for t in doc.tolist():
        if lo <= t < lo + span and t not in seen:
            seen.add(t)
            ref.append(t)
        if len(ref) >= summary_len:
            break
    return SummaryCase(doc.tolist(), ref, topic)


def score_summary(case: SummaryCase, summary: List[int]) -> Dict[str, float]:
    if not summary:
        return {"coverage": 0.0, "conciseness": 0.0, "coherence": 0.0}
    ref = set(case.reference)
    coverage = len(ref & set(summary)) / max(len(ref), 1)
    conciseness = min(1.0, len(case.reference) / len(summary))
    repeats = sum(1 for a, b in zip(summary, summary[1:]) if a == b)
    coherence = 1.0 - repeats / max(len(summary) - 1, 1)
    return {"coverage": coverage, "conciseness": conciseness, "coherence": coherence}
