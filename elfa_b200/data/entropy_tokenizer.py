"""The first-generation ("entropy") tokenizer of the reference, for its packed-dataset tools.

reference: ``src/tokenizer.zig:3-356``. Six specials ``<pad> <unk> <bos> <eos> <eod> <mask>`` = ids 0..5,
byte fallback tokens ``<byte_0> .. <byte_255>`` = ids 6..261, learned merges with priorities. ``encode``
adds ``<bos>`` / ``<eos>``, splits the text at spaces and ``\\n \\t . , ! ? ; :`` (each separator is its own
word), turns every word into byte tokens and applies merges (highest priority first, all occurrences of
the chosen pair at once) until none applies; pieces that are not in the vocabulary become ``<unk>``.
File format (little endian): ``u32 n_vocab, n_vocab x (u32 id, u32 len, bytes)``, ``u32 n_merges,
n_merges x (u32 len, first, u32 len, second, u32 priority)``.

Two deliberate differences: a merge with priority 0 can win (the reference starts its search at
priority 0 with a strict comparison, so its first learned merge is never applied), and training counts
pairs inside words on the current segmentation instead of re-encoding every text with string ids.
"""
from __future__ import annotations

import struct
from collections import Counter
from dataclasses import dataclass
from typing import Dict, Iterable, List, Sequence, Tuple

SEPARATORS = b" \n\t.,!?;:"
PAD, UNK, BOS, EOS, EOD, MASK = range(6)
_SPECIALS = ("<pad>", "<unk>", "<bos>", "<eos>", "<eod>", "<mask>")


@dataclass
class TokenizedBatch:
    tokens: List[int]
    targets: List[int]
    seq_len: int


class EntropyTokenizer:
    def __init__(self, vocab_size: int = 32000):
        self.vocab_size = vocab_size
        self.vocab: Dict[bytes, int] = {s.encode(): i for i, s in enumerate(_SPECIALS)}
        for b in range(256):
            self.vocab[f"<byte_{b}>".encode()] = 6 + b
        self.merges: List[Tuple[bytes, bytes, int]] = []       # (first, second, priority)
        self._rank: Dict[Tuple[bytes, bytes], int] = {}
        self._rev: Dict[int, bytes] = {}

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _words(text: bytes) -> List[bytes]:
        out, start = [], 0
        for i, ch in enumerate(text):
            if ch in SEPARATORS:
                if i > start:
                    out.append(text[start:i])
                out.append(text[i:i + 1])
                start = i + 1
        if start < len(text):
            out.append(text[start:])
        return out

    def _segment(self, word: bytes) -> List[bytes]:
        parts = [f"<byte_{b}>".encode() for b in word]
        while len(parts) > 1:
            best, best_pr = None, -1
            for a, b in zip(parts, parts[1:]):
                pr = self._rank.get((a, b), -1)
                if pr > best_pr:
                    best, best_pr = (a, b), pr
            if best is None:
                break
            a, b = best
            merged, i = [], 0
            while i < len(parts):
                if i + 1 < len(parts) and parts[i] == a and parts[i + 1] == b:
                    merged.append(a + b)
                    i += 2
                else:
                    merged.append(parts[i])
                    i += 1
            parts = merged
        return parts

    # ------------------------------------------------------------------ API
    def encode(self, text) -> List[int]:
        data = text.encode("utf-8") if isinstance(text, str) else bytes(text)
        ids = [BOS]
        for w in self._words(data):
            ids.extend(self.vocab.get(p, UNK) for p in self._segment(w))
        ids.append(EOS)
        return ids

    def decode(self, ids: Iterable[int]) -> bytes:
        if len(self._rev) != len(self.vocab):
            self._rev = {v: k for k, v in self.vocab.items()}
        out = bytearray()
        for t in ids:
            if t in (BOS, EOS, PAD):
                continue
            s = self._rev.get(int(t))
            if s is None:
                continue
            out.extend(self._expand(s))
        return bytes(out)

    @staticmethod
    def _expand(piece: bytes) -> bytes:
        """A vocabulary string is a concatenation of ``<byte_N>`` names (or a special's name)."""
        if not piece.startswith(b"<byte_"):
            return piece
        out = bytearray()
        for tok in piece.split(b">")[:-1]:
            out.append(int(tok[len(b"<byte_"):]))
        return bytes(out)

    def train(self, texts: Sequence, num_merges: int) -> None:
        words = Counter()
        for t in texts:
            data = t.encode("utf-8") if isinstance(t, str) else bytes(t)
            words.update(self._words(data))
        seg = {w: self._segment(w) for w in words}
        for _ in range(num_merges):
            if len(self.vocab) >= self.vocab_size:
                break
            pairs = Counter()
            for w, n in words.items():
                p = seg[w]
                for a, b in zip(p, p[1:]):
                    pairs[(a, b)] += n
            if not pairs:
                break
            (a, b), _cnt = max(pairs.items(), key=lambda kv: (kv[1], kv[0]))   # deterministic tie-break
            self.vocab[a + b] = len(self.vocab)
            pr = len(self.merges)
            self.merges.append((a, b, pr))
            self._rank[(a, b)] = pr
            seg = {w: self._segment(w) for w in words}

    def save(self, path: str) -> None:
        with open(path, "wb") as f:
            f.write(struct.pack("<I", len(self.vocab)))
            for s, i in self.vocab.items():
                f.write(struct.pack("<II", i, len(s)) + s)
            f.write(struct.pack("<I", len(self.merges)))
            for a, b, pr in self.merges:
                f.write(struct.pack("<I", len(a)) + a + struct.pack("<I", len(b)) + b + struct.pack("<I", pr))

    def load(self, path: str) -> None:
        with open(path, "rb") as f:
            data = f.read()
        off = 0
        def u32():
            nonlocal off
            v = struct.unpack_from("<I", data, off)[0]
            off += 4
            return v
        def raw(n):
            nonlocal off
            v = data[off:off + n]
            off += n
            return v
        for _ in range(u32()):
            i = u32()
            s = raw(u32())
            self.vocab[s] = i
        self.merges, self._rank = [], {}
        for _ in range(u32()):
            a = raw(u32())
            b = raw(u32())
            pr = u32()
            self.merges.append((a, b, pr))
            self._rank[(a, b)] = pr
        self._rev = {}

    def eod_token(self) -> int:
        return EOD

    def batch(self, ids: Sequence[int], seq_len: int) -> TokenizedBatch:
        """Next-token pairs of one window: tokens ``ids[:seq_len]``, targets shifted by one (``<pad>`` past the end)."""
        toks = list(ids[:seq_len]) + [PAD] * max(0, seq_len - len(ids))
        tg = list(ids[1:seq_len + 1]) + [PAD] * max(0, seq_len - max(len(ids) - 1, 0))
        return TokenizedBatch(toks, tg[:seq_len], seq_len)
