"""Sequence packing.

``pack_sequences`` concatenates variable-length sequences into one row and returns positions,
sequence ids and cumulative lengths (reference: ``src/data/dataset.zig:421-465``).
``StreamingPacker`` packs tokenised documents into fixed ``max_seq_len`` rows separated by an
end-of-document token and optionally shuffles the rows (reference: ``src/data_packer.zig:5-110``).
"""
from __future__ import annotations

from typing import Iterable, List, Sequence, Tuple

import numpy as np


def pack_sequences(seqs: Sequence[Sequence[int]]) -> Tuple[np.ndarray, np.ndarray, np.ndarray, np.ndarray]:
    """→ (tokens, positions, sequence_ids, cu_seqlens)."""
    total = sum(len(s) for s in seqs)
    tokens = np.empty(total, dtype=np.int64)
    positions = np.empty(total, dtype=np.int64)
    seq_ids = np.empty(total, dtype=np.int64)
    cu = np.zeros(len(seqs) + 1, dtype=np.int64)
    o = 0
    for i, s in enumerate(seqs):
        n = len(s)
        tokens[o:o + n] = np.asarray(s, dtype=np.int64)
        positions[o:o + n] = np.arange(n)
        seq_ids[o:o + n] = i
        o += n
        cu[i + 1] = o
    return tokens, positions, seq_ids, cu


class StreamingPacker:
    EOD = 4      # <eod> id of the gen-1 tokenizer (reference: src/tokenizer.zig:3-20)

    def __init__(self, max_seq_len: int, eod_token: int = EOD, shuffle: bool = False, seed: int = 0):
        self.max_seq_len, self.eod, self.shuffle, self.seed = max_seq_len, eod_token, shuffle, seed
        self._buf: List[int] = []
        self.rows: List[np.ndarray] = []

    def add_document(self, tokens: Iterable[int]) -> None:
        self._buf.extend(int(t) for t in tokens)
        self._buf.append(self.eod)
        while len(self._buf) >= self.max_seq_len:
            self.rows.append(np.asarray(self._buf[:self.max_seq_len], dtype=np.int64))
            del self._buf[:self.max_seq_len]

    def finish(self, pad_token: int = 0) -> np.ndarray:
        if self._buf:
            row = np.full(self.max_seq_len, pad_token, dtype=np.int64)
            row[:len(self._buf)] = self._buf
            self.rows.append(row)
            self._buf = []
        out = np.stack(self.rows) if self.rows else np.zeros((0, self.max_seq_len), dtype=np.int64)
        if self.shuffle:
            np.random.default_rng(self.seed).shuffle(out)
        return out


def document_starts(ends: np.ndarray) -> np.ndarray:
    """``ends [B, S]`` bool (True where a token closes its document) → ``[B, S]`` int32: for every position the index of
    the first token of its document. Row starts open a document; the token after an end opens the next one."""
    B, S = ends.shape
    opens = np.zeros((B, S), dtype=bool)
    opens[:, 0] = True
    opens[:, 1:] = ends[:, :-1]
    idx = np.where(opens, np.arange(S, dtype=np.int64)[None, :], 0)
    return np.maximum.accumulate(idx, axis=1).astype(np.int32)
