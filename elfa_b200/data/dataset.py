"""Binary token dataset, shard writer/builder, synthetic generators and the batch loader.

File format (little endian), identical to the reference's
(``src/data/dataset.zig:24-58,260-283``; generator script ``scripts/run_local_smoke.sh:33-48``)::

    u32 magic = 0xEF1AD001 | u32 version = 1 | u64 num_tokens | u32 num_shards |
    num_shards x { u32 path_len | path bytes | u64 shard_tokens | u8[32] sha256 } |
    u32 tokens[num_tokens]

Sampling follows ``dataset.zig:301-375``: sample ``i`` is ``tokens[i*seq_len : i*seq_len+seq_len+1]``,
input = the first ``seq_len`` tokens, target = shifted by one; ``num_samples = num_tokens // seq_len``
(the last sample is dropped when it has no look-ahead token); indices are shuffled with a seeded
generator and reshuffled every epoch; incomplete batches are dropped. The token offset is computed
from the actual shard records (the reference estimates it with a fixed record size).

Data-parallel ranks read disjoint strided slices of the shuffled index list. Batches are staged
in pinned host memory so that the host→device copy can be asynchronous.
"""
from __future__ import annotations

import hashlib
import os
import struct
from dataclasses import dataclass
from typing import List, Optional, Tuple

import numpy as np
import torch

MAGIC = 0xEF1AD001
VERSION = 1


@dataclass
class Batch:
    input: torch.Tensor     # [B, S] int64
    target: torch.Tensor    # [B, S] int64 (-100: no loss at this position)
    doc_start: Optional[torch.Tensor] = None    # [B, S] int32, packed rows only: first position of each token's document

    @property
    def num_tokens(self) -> int:
        return int(self.input.numel())


def write_token_file(path: str, tokens: np.ndarray, shards: Optional[List[Tuple[str, int, bytes]]] = None) -> None:
    """Writes ``tokens`` (any integer dtype, stored as u32) in the dataset format."""
    tok = np.ascontiguousarray(tokens, dtype="<u4")
    shards = shards or []
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "wb") as f:
        f.write(struct.pack("<IIQI", MAGIC, VERSION, tok.size, len(shards)))
        for spath, ntok, digest in shards:
            b = spath.encode()
            f.write(struct.pack("<I", len(b)) + b + struct.pack("<Q", ntok) + digest)
        f.write(tok.tobytes())


class BinaryDataset:
    """Memory-mapped reader of the dataset format."""

    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            head = f.read(20)
            if len(head) < 20:
                raise ValueError(f"{path}: truncated header")
            magic, version, ntok, nshards = struct.unpack("<IIQI", head)
            if magic != MAGIC:
                raise ValueError(f"{path}: bad magic 0x{magic:08x}")
            if version != VERSION:
                raise ValueError(f"{path}: unsupported version {version}")
            self.shards = []
            for _ in range(nshards):
                (plen,) = struct.unpack("<I", f.read(4))
                spath = f.read(plen).decode()
                (stok,) = struct.unpack("<Q", f.read(8))
                digest = f.read(32)
                self.shards.append((spath, stok, digest))
            self.offset = f.tell()
        self.num_tokens = ntok
        size = os.path.getsize(path)
        if self.offset + 4 * ntok > size:
            raise ValueError(f"{path}: header claims {ntok} tokens but the file is too short")
        self.tokens = np.memmap(path, dtype="<u4", mode="r", offset=self.offset, shape=(ntok,))

    @classmethod
    def open(cls, path: str) -> "BinaryDataset":
        return cls(path)

    def get_tokens(self, start: int, count: int) -> np.ndarray:
        if start < 0 or start + count > self.num_tokens:
            raise IndexError("token range out of bounds")
        return np.asarray(self.tokens[start:start + count])

    def __len__(self) -> int:
        return self.num_tokens


class SyntheticDataset:
    """Seeded synthetic token stream: ``uniform`` over ``[0, vocab)`` or ``zipf`` with exponent ``s``
    (rank-frequency ``p(k) ~ 1/k^s`` over the vocabulary, ranks mapped to ids by a fixed permutation)."""

    def __init__(self, vocab_size: int, num_tokens: int, kind: str = "uniform", seed: int = 0, zipf_s: float = 1.1):
        rng = np.random.default_rng(seed)
        if kind == "uniform":
            tok = rng.integers(0, vocab_size, size=num_tokens, dtype=np.int64)
        elif kind == "zipf":
            ranks = np.arange(1, vocab_size + 1, dtype=np.float64)
            p = ranks ** (-zipf_s)
            cdf = np.cumsum(p / p.sum())
            cdf[-1] = 1.0
            perm = rng.permutation(vocab_size)
            tok = perm[np.searchsorted(cdf, rng.random(num_tokens), side="left")]
        else:
            raise ValueError(kind)
        self.tokens = tok.astype("<u4")
        self.num_tokens = num_tokens
        self.shards = []

    def get_tokens(self, start: int, count: int) -> np.ndarray:
        return self.tokens[start:start + count]

    def __len__(self) -> int:
        return self.num_tokens


class ShardWriter:
    """Writes one shard file: a 64-byte zero header followed by u32 tokens; tracks the SHA-256 of
    the token bytes (reference: ``src/data/dataset.zig:110-160``)."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "wb")
        self._f.write(b"\0" * 64)
        self._h = hashlib.sha256()
        self.num_tokens = 0

    def write(self, tokens) -> None:
        b = np.ascontiguousarray(tokens, dtype="<u4").tobytes()
        self._f.write(b)
        self._h.update(b)
        self.num_tokens += len(b) // 4

    def close(self) -> bytes:
        self._f.close()
        return self._h.digest()


class DatasetBuilder:
    """Accumulates tokens into ``shard_%06d.bin`` files of at most ``shard_tokens`` tokens and
    writes ``<name>.index`` (the dataset header with shard records) plus a merged ``<name>.bin``
    (reference: ``src/data/dataset.zig:162-284``)."""

    def __init__(self, out_dir: str, name: str = "dataset", shard_tokens: int = 1 << 24):
        self.out_dir, self.name, self.shard_tokens = out_dir, name, shard_tokens
        os.makedirs(out_dir, exist_ok=True)
        self.records: List[Tuple[str, int, bytes]] = []
        self._cur: Optional[ShardWriter] = None
        self._all: List[np.ndarray] = []

    def _roll(self):
        if self._cur is not None:
            digest = self._cur.close()
            self.records.append((os.path.basename(self._cur.path), self._cur.num_tokens, digest))
        self._cur = ShardWriter(os.path.join(self.out_dir, f"shard_{len(self.records):06d}.bin"))

    def add(self, tokens) -> None:
        tok = np.asarray(tokens, dtype="<u4")
        self._all.append(tok)
        pos = 0
        while pos < tok.size:
            if self._cur is None or self._cur.num_tokens >= self.shard_tokens:
                self._roll()
            take = min(tok.size - pos, self.shard_tokens - self._cur.num_tokens)
            self._cur.write(tok[pos:pos + take])
            pos += take

    def finish(self) -> str:
        if self._cur is not None:
            digest = self._cur.close()
            self.records.append((os.path.basename(self._cur.path), self._cur.num_tokens, digest))
            self._cur = None
        total = sum(r[1] for r in self.records)
        with open(os.path.join(self.out_dir, self.name + ".index"), "wb") as f:
            f.write(struct.pack("<IIQI", MAGIC, VERSION, total, len(self.records)))
            for spath, ntok, digest in self.records:
                b = spath.encode()
                f.write(struct.pack("<I", len(b)) + b + struct.pack("<Q", ntok) + digest)
        merged = os.path.join(self.out_dir, self.name + ".bin")
        write_token_file(merged, np.concatenate(self._all) if self._all else np.zeros(0, "<u4"), self.records)
        return merged


class DataLoader:
    """Yields :class:`Batch` es of ``[batch, seq_len]`` int64 tensors (pinned when CUDA exists)."""

    def __init__(self, dataset, batch_size: int, seq_len: int, shuffle: bool = True, seed: int = 0, dp_rank: int = 0,
                 dp_size: int = 1, pin_memory: Optional[bool] = None, pack_eos: Optional[int] = None):
        """``pack_eos``: rows are documents packed back to back, each ended by this token id (``data.pack_sequences``;
        reference: ``src/data/dataset.zig:421-465`` positions / sequence ids / cumulative lengths of packed rows,
        ``src/data_packer.zig:5-112``). Batches then carry ``doc_start`` (attention and positions restart at every document)
        and the target that would cross into the next document is masked out."""
        self.pack_eos = pack_eos
        self.ds, self.batch_size, self.seq_len = dataset, batch_size, seq_len
        self.shuffle, self.seed = shuffle, seed
        self.dp_rank, self.dp_size = dp_rank, dp_size
        n = len(dataset) // seq_len
        if n * seq_len + 1 > len(dataset):
            n -= 1                       # the last window has no look-ahead token for its target
        self.num_samples = max(n, 0)
        self.epoch = 0
        self.pin = torch.cuda.is_available() if pin_memory is None else pin_memory
        self._order = None
        self._pos = 0
        self.reset()

    def num_batches(self) -> int:
        return (self.num_samples // self.dp_size) // self.batch_size

    def reset(self) -> None:
        idx = np.arange(self.num_samples, dtype=np.int64)
        if self.shuffle:
            np.random.default_rng(self.seed + self.epoch).shuffle(idx)
        self._order = idx[self.dp_rank::self.dp_size]
        self._pos = 0

    def next(self) -> Optional[Batch]:
        if self._pos + self.batch_size > len(self._order):
            return None
        S = self.seq_len
        buf = np.empty((self.batch_size, S + 1), dtype=np.int64)
        for b in range(self.batch_size):
            i = int(self._order[self._pos + b])
            buf[b] = self.ds.get_tokens(i * S, S + 1)
        self._pos += self.batch_size
        t = torch.from_numpy(buf)
        inp, tgt = t[:, :S].contiguous(), t[:, 1:].contiguous()
        doc = None
        if self.pack_eos is not None:
            from .packing import document_starts
            ends = buf[:, :S] == self.pack_eos                # the end-of-sequence token closes its document
            doc = torch.from_numpy(document_starts(ends))
            tgt[torch.from_numpy(ends)] = -100                # no prediction across a document boundary
        if self.pin:
            inp, tgt = inp.pin_memory(), tgt.pin_memory()
            doc = doc.pin_memory() if doc is not None else None
        return Batch(inp, tgt, doc)

    def skip(self, n_batches: int) -> None:
        """Advances the read position by ``n_batches`` batches (rolling over epochs) without
        materialising them; used to resume a run at the right place in the data."""
        per_epoch = max(len(self._order) // self.batch_size, 1)
        for _ in range(n_batches // per_epoch):
            self.epoch += 1
        if n_batches >= per_epoch:
            self.reset()
        self._pos = (n_batches % per_epoch) * self.batch_size

    def next_cycling(self) -> Batch:
        """Like :meth:`next` but rolls over to the next epoch (reshuffle) when exhausted."""
        b = self.next()
        if b is None:
            self.epoch += 1
            self.reset()
            b = self.next()
            if b is None:
                raise RuntimeError("dataset too small for one batch")
        return b

    def __iter__(self):
        while True:
            b = self.next()
            if b is None:
                return
            yield b


class PrefetchLoader:
    """Assembles batches ahead of the training loop on a worker thread.

    Wraps a :class:`DataLoader`: ``next_cycling()`` hands out the batches in exactly the order the wrapped loader
    would, but up to ``depth`` of them (``data.prefetch_factor x data.num_workers``) are already read, shifted into
    input / target and pinned when they are asked for. ``epoch`` is the epoch of the batch handed out last, not of
    the one the worker is reading. ``skip`` (resume) must come before the first batch.

    reference: ``src/data/dataset.zig:288-340`` (``DataLoader``: batches are built inline in the training loop; the
    YAML keys ``data.prefetch_factor`` / ``data.num_workers`` are parsed and unused there).
    """

    def __init__(self, loader: DataLoader, depth: int = 2):
        import queue
        import threading
        self.loader = loader
        self.depth = max(1, depth)
        self.epoch = loader.epoch
        self._q: "queue.Queue" = queue.Queue(maxsize=self.depth)
        self._stop = threading.Event()
        self._thread: Optional["threading.Thread"] = None
        self._threading, self._queue = threading, queue

    # the attributes callers read from a plain loader
    @property
    def num_samples(self) -> int:
        return self.loader.num_samples

    def num_batches(self) -> int:
        return self.loader.num_batches()

    def skip(self, n_batches: int) -> None:
        assert self._thread is None, "skip() must be called before the first batch is taken"
        self.loader.skip(n_batches)
        self.epoch = self.loader.epoch

    def _work(self) -> None:
        try:
            while not self._stop.is_set():
                item = (self.loader.next_cycling(), self.loader.epoch)
                while not self._stop.is_set():
                    try:
                        self._q.put(item, timeout=0.1)
                        break
                    except self._queue.Full:
                        continue
        except BaseException as e:          # handed to the consumer, which re-raises it
            self._q.put(e)

    def next_cycling(self) -> Batch:
        if self._thread is None:
            self._thread = self._threading.Thread(target=self._work, name="elfa-data-prefetch", daemon=True)
            self._thread.start()
        item = self._q.get()
        if isinstance(item, BaseException):
            raise item
        batch, self.epoch = item
        return batch

    def close(self) -> None:
        self._stop.set()
        if self._thread is not None:
            while self._thread.is_alive():
                try:
                    self._q.get_nowait()
                except self._queue.Empty:
                    pass
                self._thread.join(timeout=0.05)
            self._thread = None
