"""Synthetic needle-in-a-haystack cases (reference: ``src/evaluation/needle_haystack.zig:50-176``):
a haystack of filler tokens of a requested length with a key/value "needle" inserted at a seeded
depth, followed by a query for the key; the multi-needle variant hides several."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import numpy as np


@dataclass
class NeedleCase:
    tokens: List[int]       # haystack + query
    answer: List[int]
    depth: float            # relative position of the needle in [0, 1]
    position: int


def generate_needle_case(length: int, vocab: int, seed: int, depth: float | None = None, key_len: int = 2, value_len: int = 4,
                         marker: int = 1) -> NeedleCase:
    rng = np.random.default_rng(seed)
    lo = max(4, marker + 1)
    hay = rng.integers(lo, vocab, size=length).tolist()
    key = rng.integers(lo, vocab, size=key_len).tolist()
    val = rng.integers(lo, vocab, size=value_len).tolist()
    d = float(rng.random()) if depth is None else depth
    needle = [marker] + key + val
    pos = int(d * max(length - len(needle) - key_len - 1, 1))
    hay[pos:pos + len(needle)] = needle
    tokens = hay + [marker] + key
    return NeedleCase(tokens, val, d, pos)


def generate_multi_needle(length: int, vocab: int, seed: int, n: int = 3) -> List[NeedleCase]:
    return [generate_needle_case(length, vocab, seed * 1000 + i, depth=(i + 0.5) / n) for i in range(n)]


def depth_accuracy(results: List[tuple], bins: int = 10) -> List[float]:
    """results: (depth, correct) pairs → accuracy per depth bin."""
    tot = [0] * bins
    ok = [0] * bins
    for d, c in results:
        b = min(int(d * bins), bins - 1)
        tot[b] += 1
        ok[b] += int(bool(c))
    return [ok[i] / tot[i] if tot[i] else float("nan") for i in range(bins)]
