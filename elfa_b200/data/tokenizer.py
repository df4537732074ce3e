"""Byte-level BPE tokenizer with the reference's file format.

ids 0..255 are raw bytes, 256..259 are ``<pad> <unk> <bos> <eos>``, merged tokens follow.
Training merges the most frequent adjacent pair, ties broken towards the lexicographically
smaller ``(first, second)``; encoding splits on the longest matching special token and applies the
merges in training order (reference: ``src/data/tokenizer.zig:28-29,129-141,178-268,371-433``).

File format (little endian, ``tokenizer.zig:273-358``)::

    u32 magic = 0x544B5A31 | u32 vocab_size | u32 special_count | u32 merge_count |
    vocab_size x { u32 len | bytes } | special_count x u32 id | merge_count x { u32 first, u32 second, u32 result }

``encode_file`` writes ``u64 n | u32 tokens[n]``.
"""
from __future__ import annotations

import struct
from collections import Counter
from typing import Dict, List, Tuple

import numpy as np

MAGIC = 0x544B5A31
SPECIALS = ("<pad>", "<unk>", "<bos>", "<eos>")
PAD, UNK, BOS, EOS = 256, 257, 258, 259


class Tokenizer:
    def __init__(self):
        self.vocab: List[bytes] = [bytes([i]) for i in range(256)] + [s.encode() for s in SPECIALS]
        self.special_ids: List[int] = [PAD, UNK, BOS, EOS]
        self.merges: List[Tuple[int, int, int]] = []
        self._rank: Dict[Tuple[int, int], Tuple[int, int]] = {}

    # ------------------------------------------------------------------ training
    @classmethod
    def train(cls, corpus: bytes, vocab_size: int) -> "Tokenizer":
        tok = cls()
        ids = list(corpus)
        while len(tok.vocab) < vocab_size and len(ids) >= 2:
            counts = Counter(zip(ids, ids[1:]))
            if not counts:
                break
            best_n = max(counts.values())
            if best_n < 2:
                break
            pair = min(p for p, n in counts.items() if n == best_n)
            new_id = len(tok.vocab)
            tok.vocab.append(tok.vocab[pair[0]] + tok.vocab[pair[1]])
            tok.merges.append((pair[0], pair[1], new_id))
            ids = _merge(ids, pair, new_id)
        tok._build()
        return tok

    @classmethod
    def train_from_text(cls, text: str, vocab_size: int) -> "Tokenizer":
        return cls.train(text.encode("utf-8"), vocab_size)

    def _build(self) -> None:
        self._rank = {(a, b): (i, r) for i, (a, b, r) in enumerate(self.merges)}

    @property
    def vocab_size(self) -> int:
        return len(self.vocab)

    # -------------------------------------------------------------------- coding
    def _encode_bytes(self, data: bytes) -> List[int]:
        ids = list(data)
        while len(ids) >= 2:
            best = None
            for p in set(zip(ids, ids[1:])):
                r = self._rank.get(p)
                if r is not None and (best is None or r[0] < best[0]):
                    best = (r[0], p, r[1])
            if best is None:
                break
            ids = _merge(ids, best[1], best[2])
        return ids

    def encode(self, text, add_bos: bool = False, add_eos: bool = False) -> List[int]:
        data = text.encode("utf-8") if isinstance(text, str) else bytes(text)
        specials = sorted(((self.vocab[i], i) for i in self.special_ids), key=lambda t: -len(t[0]))
        out: List[int] = [BOS] if add_bos else []
        pos, start = 0, 0
        n = len(data)
        while pos < n:
            hit = None
            if data[pos:pos + 1] == b"<":
                for sb, sid in specials:
                    if data.startswith(sb, pos):
                        hit = (sb, sid)
                        break
            if hit is None:
                pos += 1
                continue
            if start < pos:
                out.extend(self._encode_bytes(data[start:pos]))
            out.append(hit[1])
            pos += len(hit[0])
            start = pos
        if start < n:
            out.extend(self._encode_bytes(data[start:]))
        if add_eos:
            out.append(EOS)
        return out

    def decode_bytes(self, ids) -> bytes:
        return b"".join(self.vocab[i] if 0 <= i < len(self.vocab) else self.vocab[UNK] for i in ids)

    def decode(self, ids) -> str:
        return self.decode_bytes(ids).decode("utf-8", errors="replace")

    def encode_file(self, in_path: str, out_path: str) -> int:
        with open(in_path, "rb") as f:
            ids = self.encode(f.read())
        with open(out_path, "wb") as f:
            f.write(struct.pack("<Q", len(ids)))
            f.write(np.asarray(ids, dtype="<u4").tobytes())
        return len(ids)

    # ------------------------------------------------------------------------ io
    def save(self, path: str) -> None:
        with open(path, "wb") as f:
            f.write(struct.pack("<IIII", MAGIC, len(self.vocab), len(self.special_ids), len(self.merges)))
            for v in self.vocab:
                f.write(struct.pack("<I", len(v)) + v)
            for s in self.special_ids:
                f.write(struct.pack("<I", s))
            for a, b, r in self.merges:
                f.write(struct.pack("<III", a, b, r))

    @classmethod
    def load(cls, path: str) -> "Tokenizer":
        with open(path, "rb") as f:
            data = f.read()
        magic, nv, ns, nm = struct.unpack_from("<IIII", data, 0)
        if magic != MAGIC:
            raise ValueError(f"{path}: bad tokenizer magic 0x{magic:08x}")
        off = 16
        tok = cls()
        tok.vocab = []
        for _ in range(nv):
            (ln,) = struct.unpack_from("<I", data, off)
            off += 4
            tok.vocab.append(data[off:off + ln])
            off += ln
        tok.special_ids = list(struct.unpack_from(f"<{ns}I", data, off))
        off += 4 * ns
        tok.merges = [struct.unpack_from("<III", data, off + 12 * i) for i in range(nm)]
        tok._build()
        return tok


def _merge(ids: List[int], pair: Tuple[int, int], new_id: int) -> List[int]:
    out: List[int] = []
    i, n = 0, len(ids)
    a, b = pair
    while i < n:
        if i + 1 < n and ids[i] == a and ids[i + 1] == b:
            out.append(new_id)
            i += 2
        else:
            out.append(ids[i])
            i += 1
    return out
