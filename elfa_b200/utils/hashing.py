"""Hash helpers: SHA-256 of data / files with hex + verify, a 64-bit fast hash, struct hash, combine.

reference: ``src/util/hash.zig:7-101`` (SHA-256 data / file / hex / verify, XxHash3, Wyhash struct hash,
``combine``, string hash). The 64-bit fast hash here is XXH64 (public algorithm, implemented directly so
that checkpoints and caches do not depend on an extra package); it is used for cache keys, never for
integrity (integrity is SHA-256).
"""
from __future__ import annotations

import hashlib
import struct
from typing import Iterable

_M = (1 << 64) - 1
_P1, _P2, _P3, _P4, _P5 = 11400714785074694791, 14029467366897019727, 1609587929392839161, 9650029242287828579, 2870177450012600261


def sha256_bytes(data: bytes) -> bytes:
    return hashlib.sha256(data).digest()


def sha256_hex(data: bytes) -> str:
    return hashlib.sha256(data).hexdigest()


def sha256_file(path: str, chunk: int = 1 << 20) -> bytes:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        while True:
            b = f.read(chunk)
            if not b:
                break
            h.update(b)
    return h.digest()


def verify_sha256(data: bytes, expected: bytes) -> bool:
    return hashlib.sha256(data).digest() == bytes(expected)


def _rotl(x: int, r: int) -> int:
    return ((x << r) | (x >> (64 - r))) & _M


def _round(acc: int, lane: int) -> int:
    return (_rotl((acc + lane * _P2) & _M, 31) * _P1) & _M


def _merge(h: int, v: int) -> int:
    return ((h ^ _round(0, v)) * _P1 + _P4) & _M


def xxh64(data: bytes, seed: int = 0) -> int:
    n, i = len(data), 0
    if n >= 32:
        v1, v2, v3, v4 = (seed + _P1 + _P2) & _M, (seed + _P2) & _M, seed & _M, (seed - _P1) & _M
        while i + 32 <= n:
            a, b, c, d = struct.unpack_from("<QQQQ", data, i)
            v1, v2, v3, v4 = _round(v1, a), _round(v2, b), _round(v3, c), _round(v4, d)
            i += 32
        h = (_rotl(v1, 1) + _rotl(v2, 7) + _rotl(v3, 12) + _rotl(v4, 18)) & _M
        for v in (v1, v2, v3, v4):
            h = _merge(h, v)
    else:
        h = (seed + _P5) & _M
    h = (h + n) & _M
    while i + 8 <= n:
        h = (_rotl(h ^ _round(0, struct.unpack_from("<Q", data, i)[0]), 27) * _P1 + _P4) & _M
        i += 8
    if i + 4 <= n:
        h = (_rotl(h ^ (struct.unpack_from("<I", data, i)[0] * _P1 & _M), 23) * _P2 + _P3) & _M
        i += 4
    while i < n:
        h = (_rotl(h ^ (data[i] * _P5 & _M), 11) * _P1) & _M
        i += 1
    h ^= h >> 33
    h = (h * _P2) & _M
    h ^= h >> 29
    h = (h * _P3) & _M
    h ^= h >> 32
    return h


def hash_string(s: str, seed: int = 0) -> int:
    return xxh64(s.encode("utf-8"), seed)


def combine(a: int, b: int) -> int:
    """Order-dependent combination of two 64-bit hashes."""
    return (a ^ ((b + 0x9E3779B97F4A7C15 + ((a << 6) & _M) + (a >> 2)) & _M)) & _M


def hash_fields(fields: Iterable) -> int:
    """Hash of a flat record (ints, floats, strings, bytes), field by field."""
    h = 0
    for f in fields:
        if isinstance(f, bytes):
            v = xxh64(f)
        elif isinstance(f, str):
            v = hash_string(f)
        elif isinstance(f, float):
            v = xxh64(struct.pack("<d", f))
        else:
            v = xxh64(struct.pack("<q", int(f)))
        h = combine(h, v)
    return h
