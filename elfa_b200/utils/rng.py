"""Deterministic random number generators with the reference's algorithms.

reference: ``src/util/rng.zig:3-91`` (``DeterministicRng``: PCG32 XSH-RR with multiplier
6364136223846793005 and increment ``(seed << 1) | 1``, Box-Muller normals, unbiased range, Fisher-Yates
shuffle, fork), ``:93-149`` (``DistributedRng``: four streams per rank, seed ``base.next() ^ rank*phi ^
stream*c``), ``:151-180`` (``PhiloxRng``: 10-round Philox 2x32). Model initialisation itself uses
``torch.Generator`` (the reference's live path uses Zig's xoshiro + ziggurat, which cannot be
reproduced outside Zig); these generators serve data shuffling, dropout seeds and tests.
"""
from __future__ import annotations

import math
from typing import List, Sequence

M64 = (1 << 64) - 1
M32 = (1 << 32) - 1
PCG_MULT = 6364136223846793005
PHI = 0x9E3779B97F4A7C15
STREAM_C = 0xBF58476D1CE4E5B9


class DeterministicRng:
    def __init__(self, seed: int):
        self.inc = ((seed << 1) | 1) & M64
        self.state = 0
        self.next_u32()
        self.state = (self.state + (seed & M64)) & M64
        self.next_u32()
        self._spare = None

    def next_u32(self) -> int:
        old = self.state
        self.state = (old * PCG_MULT + self.inc) & M64
        xorshifted = (((old >> 18) ^ old) >> 27) & M32
        rot = old >> 59
        return ((xorshifted >> rot) | (xorshifted << ((-rot) & 31))) & M32

    def next_u64(self) -> int:
        return (self.next_u32() << 32) | self.next_u32()

    def uniform(self) -> float:
        return self.next_u32() / 4294967296.0

    def range(self, n: int) -> int:
        """Unbiased integer in [0, n)."""
        if n <= 0:
            raise ValueError("n must be positive")
        threshold = (1 << 32) % n
        while True:
            r = self.next_u32()
            if r >= threshold:
                return r % n

    def normal(self) -> float:
        if self._spare is not None:
            v, self._spare = self._spare, None
            return v
        u1 = max(self.uniform(), 1e-12)
        u2 = self.uniform()
        r = math.sqrt(-2.0 * math.log(u1))
        self._spare = r * math.sin(2 * math.pi * u2)
        return r * math.cos(2 * math.pi * u2)

    def shuffle(self, items: List) -> None:
        for i in range(len(items) - 1, 0, -1):
            j = self.range(i + 1)
            items[i], items[j] = items[j], items[i]

    def fork(self) -> "DeterministicRng":
        return DeterministicRng(self.next_u64())


class DistributedRng:
    STREAMS = ("init", "dropout", "data", "noise")

    def __init__(self, seed: int, rank: int):
        base = DeterministicRng(seed)
        self.streams = {}
        for i, name in enumerate(self.STREAMS):
            s = base.next_u64() ^ ((rank * PHI) & M64) ^ ((i * STREAM_C) & M64)
            self.streams[name] = DeterministicRng(s)

    def __getitem__(self, name: str) -> DeterministicRng:
        return self.streams[name]


class PhiloxRng:
    """Philox 2x32 with 10 rounds: counter-based, so ``at(i)`` needs no state."""
    M = 0xD256D193
    W = 0x9E3779B9

    def __init__(self, key: int):
        self.key = key & M32
        self.counter = 0

    def at(self, counter: int) -> Sequence[int]:
        lo, hi = counter & M32, (counter >> 32) & M32
        k = self.key
        for _ in range(10):
            prod = self.M * lo
            lo, hi = ((prod >> 32) ^ k ^ hi) & M32, prod & M32
            k = (k + self.W) & M32
        return lo, hi

    def next(self) -> Sequence[int]:
        v = self.at(self.counter)
        self.counter += 1
        return v
