"""Checkpoint directory format ``EFLATNS1`` (byte compatible with the reference's manager).

Layout (reference: ``src/checkpoint/manager.zig:46-63,88-176,244-413,498-578``)::

    <dir>/step_%08d/
      metadata.json   {"step","epoch","tokens_seen","loss","learning_rate","timestamp","git_revision","config_hash"}
      tensors.bin     "EFLATNS1" | u32 version=1 | u32 num_tensors |
                      index: per tensor u32 name_len | name | u32 ndim | ndim x u64 dims | u32 dtype | u64 offset | u64 size | u8[32] sha256
                      payload: raw little-endian tensor bytes in index order, no padding
      optimizer.bin   (optional) "EFLAOPT1" | u32 version=1 | u64 nbytes | opaque payload
      rng.bin         (optional) opaque bytes
      config.yaml     copy of the run configuration (evaluate / generate read it; the reference expects
                      the file but never writes it)

Publication is atomic: everything is written into ``.tmp_step_<step>_<ns>``, an existing final
directory is renamed to ``.bak``, the temp directory is renamed into place and the backup removed.
Every tensor carries a SHA-256 that is verified on load together with name / shape / dtype / size.
Only the newest ``keep_last_n`` step directories are kept.

dtype codes (``src/tensor/dtype.zig:3-13``): fp32=0 fp16=1 bf16=2 fp8_e4m3=3 fp8_e5m2=4 fp4=5 int8=6
int32=7 int64=8 bool=9.

Tensors are stored as *logical* (unsharded) tensors, so a checkpoint written by a TP / ZeRO run can
be loaded by a run with a different world size. ``async_save`` snapshots to host memory and writes
in a background thread; ``compression`` gzip-compresses ``optimizer.bin`` only (``tensors.bin`` stays
byte compatible).
"""
from __future__ import annotations

import gzip
import hashlib
import io
import json
import os
import re
import shutil
import struct
import threading
import time
from dataclasses import asdict, dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

TENSOR_MAGIC = b"EFLATNS1"
OPT_MAGIC = b"EFLAOPT1"
VERSION = 1

DTYPE_CODES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2, torch.float8_e4m3fn: 3, torch.float8_e5m2: 4,
               torch.int8: 6, torch.int32: 7, torch.int64: 8, torch.bool: 9}
CODE_DTYPES = {v: k for k, v in DTYPE_CODES.items()}
FP4_CODE = 5


@dataclass
class CheckpointMetadata:
    step: int = 0
    epoch: int = 0
    tokens_seen: int = 0
    loss: float = 0.0
    learning_rate: float = 0.0
    timestamp: int = 0
    git_revision: str = ""
    config_hash: str = "0" * 64

    FIELDS = ("step", "epoch", "tokens_seen", "loss", "learning_rate", "timestamp", "git_revision", "config_hash")

    def to_json(self) -> str:
        return json.dumps(asdict(self))

    @classmethod
    def from_json(cls, text: str) -> "CheckpointMetadata":
        if len(text) > (1 << 20):
            raise ValueError("metadata.json larger than 1 MiB")
        d = json.loads(text)
        if not isinstance(d, dict):
            raise ValueError("metadata.json must be an object")
        unknown = set(d) - set(cls.FIELDS)
        if unknown:
            raise ValueError(f"metadata.json: unknown fields {sorted(unknown)}")
        m = cls(**d)
        if not re.fullmatch(r"[0-9a-f]{64}", m.config_hash):
            raise ValueError("metadata.json: config_hash must be 64 lowercase hex characters")
        if len(m.git_revision) > 40:
            raise ValueError("metadata.json: git_revision longer than 40 characters")
        return m


def _tensor_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().tobytes()
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return t.view(torch.uint8).numpy().tobytes()
    return t.numpy().tobytes()


def _bytes_tensor(b: bytes, dtype: torch.dtype, shape) -> torch.Tensor:
    if dtype == torch.bfloat16:
        return torch.from_numpy(np.frombuffer(b, dtype="<i2").copy()).view(torch.bfloat16).reshape(shape)
    if dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return torch.from_numpy(np.frombuffer(b, dtype=np.uint8).copy()).view(dtype).reshape(shape)
    npdt = {torch.float32: "<f4", torch.float16: "<f2", torch.int8: "i1", torch.int32: "<i4", torch.int64: "<i8", torch.bool: "?"}[dtype]
    return torch.from_numpy(np.frombuffer(b, dtype=npdt).copy()).reshape(shape)


def write_tensors(path: str, tensors: List[Tuple[str, torch.Tensor]]) -> None:
    names = [n for n, _ in tensors]
    if any(not n for n in names) or len(set(names)) != len(names):
        raise ValueError("tensor names must be unique and non-empty")
    blobs = [_tensor_bytes(t) for _, t in tensors]
    index_size = sum(4 + len(n.encode()) + 4 + 8 * t.dim() + 4 + 8 + 8 + 32 for n, t in tensors)
    offset = 16 + index_size
    with open(path, "wb") as f:
        f.write(TENSOR_MAGIC + struct.pack("<II", VERSION, len(tensors)))
        for (name, t), blob in zip(tensors, blobs):
            nb = name.encode()
            f.write(struct.pack("<I", len(nb)) + nb)
            f.write(struct.pack("<I", t.dim()) + b"".join(struct.pack("<Q", int(d)) for d in t.shape))
            f.write(struct.pack("<IQQ", DTYPE_CODES[t.dtype], offset, len(blob)))
            f.write(hashlib.sha256(blob).digest())
            offset += len(blob)
        for blob in blobs:
            f.write(blob)


def read_index(f) -> List[dict]:
    head = f.read(16)
    if head[:8] != TENSOR_MAGIC:
        raise ValueError("tensors.bin: bad magic")
    version, n = struct.unpack("<II", head[8:])
    if version != VERSION:
        raise ValueError(f"tensors.bin: unsupported version {version}")
    out = []
    seen = set()
    for _ in range(n):
        (nl,) = struct.unpack("<I", f.read(4))
        name = f.read(nl).decode()
        if not name or name in seen:
            raise ValueError("tensors.bin: empty or duplicate tensor name")
        seen.add(name)
        (nd,) = struct.unpack("<I", f.read(4))
        dims = [struct.unpack("<Q", f.read(8))[0] for _ in range(nd)]
        dt, off, size = struct.unpack("<IQQ", f.read(20))
        sha = f.read(32)
        out.append({"name": name, "dims": dims, "dtype": dt, "offset": off, "size": size, "sha256": sha})
    return out


def read_tensors(path: str, verify: bool = True) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    with open(path, "rb") as f:
        for e in read_index(f):
            f.seek(e["offset"])
            blob = f.read(e["size"])
            if len(blob) != e["size"]:
                raise ValueError(f"tensors.bin: '{e['name']}' is truncated")
            if verify and hashlib.sha256(blob).digest() != e["sha256"]:
                raise ValueError(f"tensors.bin: SHA-256 mismatch for '{e['name']}'")
            if e["dtype"] not in CODE_DTYPES:
                raise ValueError(f"tensors.bin: unsupported dtype code {e['dtype']} for '{e['name']}'")
            dt = CODE_DTYPES[e["dtype"]]
            numel = int(np.prod(e["dims"])) if e["dims"] else 1
            if numel * torch.empty(0, dtype=dt).element_size() != e["size"]:
                raise ValueError(f"tensors.bin: size mismatch for '{e['name']}'")
            out[e["name"]] = _bytes_tensor(blob, dt, e["dims"])
    return out


def parse_step(name: str) -> Optional[int]:
    m = re.fullmatch(r"step_(\d{8})", name)
    return int(m.group(1)) if m else None


def list_checkpoints(directory: str) -> List[Tuple[int, str]]:
    if not os.path.isdir(directory):
        return []
    out = []
    for n in os.listdir(directory):
        s = parse_step(n)
        if s is not None and os.path.isdir(os.path.join(directory, n)):
            out.append((s, os.path.join(directory, n)))
    return sorted(out)


def resolve_checkpoint(path: str) -> str:
    """``path`` may be a step directory, a checkpoint root (→ ``latest`` link or the highest step),
    like the reference's launcher does (``cloud/modal/train.py:84-124``)."""
    if os.path.isfile(os.path.join(path, "tensors.bin")):
        return path
    latest = os.path.join(path, "latest")
    if os.path.exists(latest):
        return os.path.realpath(latest)
    cks = list_checkpoints(path)
    if not cks:
        raise FileNotFoundError(f"no checkpoint under {path}")
    return cks[-1][1]


def validate_checkpoint(path: str) -> CheckpointMetadata:
    with open(os.path.join(path, "metadata.json"), "r", encoding="utf-8") as f:
        meta = CheckpointMetadata.from_json(f.read())
    read_tensors(os.path.join(path, "tensors.bin"), verify=True)
    opt = os.path.join(path, "optimizer.bin")
    if os.path.exists(opt):
        read_optimizer(opt)
    return meta


def write_optimizer(path: str, payload: bytes) -> None:
    with open(path, "wb") as f:
        f.write(OPT_MAGIC + struct.pack("<IQ", VERSION, len(payload)) + payload)


def read_optimizer(path: str) -> bytes:
    with open(path, "rb") as f:
        head = f.read(20)
        if head[:8] != OPT_MAGIC:
            raise ValueError("optimizer.bin: bad magic")
        version, n = struct.unpack("<IQ", head[8:])
        if version != VERSION:
            raise ValueError("optimizer.bin: unsupported version")
        payload = f.read(n)
        if len(payload) != n:
            raise ValueError("optimizer.bin: truncated")
        return payload


def convert_checkpoint(src: str, dst: str, fmt: str = "efla_native") -> None:
    """``efla_native`` copies (re-validating); ``pytorch`` writes ``<dst>/model.pt`` with a plain state
    dict; ``safetensors`` writes the safetensors container (the reference rejects both with
    ``UnsupportedCheckpointFormat``, ``src/checkpoint/manager.zig:671-728``)."""
    validate_checkpoint(src)
    os.makedirs(dst, exist_ok=True)
    if fmt == "efla_native":
        for n in os.listdir(src):
            shutil.copy2(os.path.join(src, n), os.path.join(dst, n))
        return
    tensors = read_tensors(os.path.join(src, "tensors.bin"))
    if fmt == "pytorch":
        torch.save(tensors, os.path.join(dst, "model.pt"))
        return
    if fmt == "safetensors":
        names = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.int8: "I8", torch.int32: "I32",
                 torch.int64: "I64", torch.bool: "BOOL", torch.float8_e4m3fn: "F8_E4M3", torch.float8_e5m2: "F8_E5M2"}
        header, blobs, off = {}, [], 0
        for k, t in tensors.items():
            b = _tensor_bytes(t)
            header[k] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
            blobs.append(b)
            off += len(b)
        hb = json.dumps(header, separators=(",", ":")).encode()
        hb += b" " * ((8 - len(hb) % 8) % 8)
        with open(os.path.join(dst, "model.safetensors"), "wb") as f:
            f.write(struct.pack("<Q", len(hb)) + hb + b"".join(blobs))
        return
    raise ValueError(f"unsupported checkpoint format {fmt!r}")


class CheckpointManager:
    def __init__(self, directory: str, keep_last_n: int = 5, compression: bool = False, async_save: bool = False):
        self.dir, self.keep_last_n, self.compression, self.async_save = directory, keep_last_n, compression, async_save
        os.makedirs(directory, exist_ok=True)
        self._thread: Optional[threading.Thread] = None
        self._error: Optional[BaseException] = None

    # ------------------------------------------------------------------ save
    def save(self, step: int, tensors: List[Tuple[str, torch.Tensor]], meta: CheckpointMetadata,
             optimizer_state: Optional[dict] = None, rng_state: Optional[bytes] = None, config_yaml: Optional[str] = None) -> str:
        self.wait()
        # snapshot to host first so that training can continue while the files are written
        host = [(n, t.detach().to("cpu", copy=True)) for n, t in tensors]
        opt_payload = None
        if optimizer_state is not None:
            buf = io.BytesIO()
            torch.save(optimizer_state, buf)
            opt_payload = buf.getvalue()
            if self.compression:
                opt_payload = b"GZ01" + gzip.compress(opt_payload, compresslevel=1)
        final = os.path.join(self.dir, f"step_{step:08d}")

        def work():
            tmp = os.path.join(self.dir, f".tmp_step_{step:08d}_{time.time_ns()}")
            os.makedirs(tmp)
            try:
                with open(os.path.join(tmp, "metadata.json"), "w", encoding="utf-8") as f:
                    f.write(meta.to_json())
                write_tensors(os.path.join(tmp, "tensors.bin"), host)
                if opt_payload is not None:
                    write_optimizer(os.path.join(tmp, "optimizer.bin"), opt_payload)
                if rng_state is not None:
                    with open(os.path.join(tmp, "rng.bin"), "wb") as f:
                        f.write(rng_state)
                if config_yaml is not None:
                    with open(os.path.join(tmp, "config.yaml"), "w", encoding="utf-8") as f:
                        f.write(config_yaml)
                bak = final + ".bak"
                if os.path.exists(final):
                    if os.path.exists(bak):
                        shutil.rmtree(bak)
                    os.rename(final, bak)
                try:
                    os.rename(tmp, final)
                except OSError:
                    if os.path.exists(bak):
                        os.rename(bak, final)
                    raise
                if os.path.exists(bak):
                    shutil.rmtree(bak)
                latest = os.path.join(self.dir, "latest")
                try:
                    if os.path.islink(latest) or os.path.exists(latest):
                        os.remove(latest)
                    os.symlink(os.path.basename(final), latest)
                except OSError:
                    pass
                self._cleanup()
            except BaseException as e:      # noqa: BLE001 - reported by wait()
                shutil.rmtree(tmp, ignore_errors=True)
                self._error = e

        if self.async_save:
            self._thread = threading.Thread(target=work, daemon=True)
            self._thread.start()
        else:
            work()
            self.wait()
        return final

    def wait(self) -> None:
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self._error is not None:
            e, self._error = self._error, None
            raise e

    def _cleanup(self) -> None:
        if self.keep_last_n <= 0:
            return
        cks = list_checkpoints(self.dir)
        for _, p in cks[:-self.keep_last_n]:
            shutil.rmtree(p, ignore_errors=True)

    # ------------------------------------------------------------------ load
    def load(self, path: Optional[str] = None, expected: Optional[Dict[str, Tuple[tuple, torch.dtype]]] = None):
        """→ (metadata, tensors). ``expected`` maps name → (shape, dtype); every expected tensor must be
        present with exactly that shape and dtype (reference: ``manager.zig:471-494``)."""
        p = resolve_checkpoint(path or self.dir)
        with open(os.path.join(p, "metadata.json"), "r", encoding="utf-8") as f:
            meta = CheckpointMetadata.from_json(f.read())
        tensors = read_tensors(os.path.join(p, "tensors.bin"))
        if expected is not None:
            for name, (shape, dtype) in expected.items():
                if name not in tensors:
                    raise KeyError(f"checkpoint is missing tensor '{name}'")
                t = tensors[name]
                if tuple(t.shape) != tuple(shape) or t.dtype != dtype:
                    raise ValueError(f"tensor '{name}': checkpoint has {tuple(t.shape)} {t.dtype}, model needs {tuple(shape)} {dtype}")
        return meta, tensors

    def load_full(self, path: Optional[str] = None):
        """→ (metadata, tensors, optimizer_state or None, rng bytes or None, config yaml or None)."""
        p = resolve_checkpoint(path or self.dir)
        meta, tensors = self.load(p)
        opt = rng = cfg = None
        op = os.path.join(p, "optimizer.bin")
        if os.path.exists(op):
            payload = read_optimizer(op)
            if payload[:4] == b"GZ01":
                payload = gzip.decompress(payload[4:])
            opt = torch.load(io.BytesIO(payload), map_location="cpu", weights_only=False)
        rp = os.path.join(p, "rng.bin")
        if os.path.exists(rp):
            with open(rp, "rb") as f:
                rng = f.read()
        cp = os.path.join(p, "config.yaml")
        if os.path.exists(cp):
            with open(cp, "r", encoding="utf-8") as f:
                cfg = f.read()
        return meta, tensors, opt, rng, cfg
