"""ctypes binding of the native library.

The C prototypes are read from ``csrc/elfa_native.h`` so that the Python signatures can never
drift from the header. Pointer arguments accept ``torch.Tensor`` (its ``data_ptr()``), ``int`` or
``None``. Every call checks the return code and raises :class:`NativeError` with the library's
message; on a CUDA machine a missing library is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes
import os
import re
from pathlib import Path
from typing import Any, Dict, Optional

import torch

_PKG = Path(__file__).resolve().parent
# ELFA_BOUNDS=1 selects the checked variant of the library (see build.build(bounds=True)): in-kernel index checks that record
# a violation in the status word and skip the access
_BOUNDS = os.environ.get("ELFA_BOUNDS", "0") == "1"
_LIB_PATH = _PKG / "_native" / ("libelfa_b200_bounds.so" if _BOUNDS else "libelfa_b200.so")
_HEADER = _PKG / "csrc" / "elfa_native.h"

ST_MBAR_TIMEOUT = 1
ST_FLAG_TIMEOUT = 2
ST_BAD_TARGET = 4
ST_NONFINITE = 8
ST_BOUNDS = 16

EPI_BIAS, EPI_GELU, EPI_DGELU_AUX, EPI_ADD_AUX, EPI_ACCUM, EPI_OUT_F32, EPI_STORE_PREACT = 1, 2, 4, 8, 16, 32, 64


class NativeError(RuntimeError):
    pass


class CommTimeout(NativeError):
    """A bounded device-side wait ran out (peer flag or pipeline barrier)."""


def _ctype(decl: str):
    d = decl.strip()
    if "*" in d:
        return ctypes.c_void_p
    d = re.sub(r"\bconst\b", "", d).strip()
    base = " ".join(d.split()[:-1]) if len(d.split()) > 1 else d
    return {
        "int": ctypes.c_int, "unsigned": ctypes.c_uint, "unsigned int": ctypes.c_uint, "long long": ctypes.c_longlong,
        "float": ctypes.c_float, "double": ctypes.c_double, "size_t": ctypes.c_size_t, "uint64_t": ctypes.c_uint64,
        "uint32_t": ctypes.c_uint32, "unsigned long long": ctypes.c_ulonglong,
    }[base]


def _parse_header(text: str) -> Dict[str, list]:
    text = re.sub(r"//[^\n]*", "", text)
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    protos = {}
    for m in re.finditer(r"\b(int|const char\*)\s+(elfa_\w+)\s*\(([^)]*)\)\s*;", text):
        ret, name, args = m.group(1), m.group(2), m.group(3).strip()
        argt = [] if args in ("", "void") else [_ctype(a) for a in args.split(",")]
        protos[name] = (ret, argt)
    return protos


class _Lib:
    def __init__(self) -> None:
        self._dll: Optional[ctypes.CDLL] = None
        self._protos: Dict[str, Any] = {}

    def available(self) -> bool:
        return _LIB_PATH.exists()

    def load(self) -> ctypes.CDLL:
        if self._dll is not None:
            return self._dll
        self._check_fresh()
        if not _LIB_PATH.exists():
            raise NativeError(f"native library {_LIB_PATH} is missing: run `python -m elfa_b200.build`")
        dll = ctypes.CDLL(str(_LIB_PATH), mode=os.RTLD_GLOBAL if hasattr(os, "RTLD_GLOBAL") else ctypes.DEFAULT_MODE)
        self._protos = _parse_header(_HEADER.read_text())
        for name, (ret, argt) in self._protos.items():
            fn = getattr(dll, name, None)
            if fn is None:
                raise NativeError(f"symbol {name} declared in elfa_native.h is missing from the library")
            fn.argtypes = argt
            fn.restype = ctypes.c_char_p if ret != "int" else ctypes.c_int
        self._dll = dll
        return dll

    def _check_fresh(self) -> None:
        """The binary must come from the sources next to it. A stale library (sources edited, not rebuilt) is rebuilt when
        a compiler is at hand - one process at a time, the others wait on a file lock - and is an error otherwise."""
        if os.environ.get("ELFA_SKIP_HASH_CHECK", "0") == "1":
            return
        from . import build as b
        here = b.source_hash()

        def built() -> str:
            if not _LIB_PATH.exists():
                return ""
            try:
                probe = ctypes.CDLL(str(_LIB_PATH))
                probe.elfa_source_hash.restype = ctypes.c_char_p
                return (probe.elfa_source_hash() or b"").decode()
            except (OSError, AttributeError):
                return ""
        stamp = b.obj_dir(_BOUNDS) / "source_hash.txt"
        if _LIB_PATH.exists() and stamp.exists() and stamp.read_text().strip() == here:
            return              # the build step's own record says the library is current (no need to open it twice)
        if built() == here:
            return
        import fcntl
        b.OUT_DIR.mkdir(parents=True, exist_ok=True)
        with open(b.OUT_DIR / ".build.lock", "w") as lock:
            fcntl.flock(lock, fcntl.LOCK_EX)
            try:
                if not (stamp.exists() and stamp.read_text().strip() == here and _LIB_PATH.exists()):
                    try:
                        b.build(bounds=_BOUNDS)
                    except RuntimeError as e:
                        raise NativeError(f"native library {_LIB_PATH} is missing or was built from other sources and could not be "
                                          f"rebuilt: {e}") from e
            finally:
                fcntl.flock(lock, fcntl.LOCK_UN)


    def last_error(self) -> str:
        return (self.load().elfa_last_error() or b"").decode()

    def call(self, name: str, *args) -> None:
        dll = self.load()
        conv = []
        for a in args:
            if isinstance(a, torch.Tensor):
                conv.append(a.data_ptr())
            elif a is None:
                conv.append(None)
            else:
                conv.append(a)
        rc = getattr(dll, name)(*conv)
        if rc != 0:
            raise NativeError(f"{name} failed (code {rc}): {self.last_error()}")

    def raw(self, name: str):
        return getattr(self.load(), name)


lib = _Lib()


def stream_ptr(t: Optional[torch.Tensor] = None) -> int:
    return torch.cuda.current_stream(t.device if t is not None else None).cuda_stream


def status() -> int:
    """Reads and clears the device status word (synchronises the device)."""
    out = ctypes.c_uint(0)
    rc = lib.load().elfa_status(ctypes.addressof(out))
    if rc != 0:
        raise NativeError(f"elfa_status failed: {lib.last_error()}")
    return int(out.value)


_deterministic = False


def set_deterministic(on: bool) -> None:
    """``runtime.deterministic``: fixed summation orders only - the GEMM stops splitting contractions across CTAs (fp32
    atomics) and the embedding gradient is reduced over sorted token ids instead of scattered with atomics."""
    global _deterministic
    _deterministic = bool(on)
    if lib.available():
        lib.call("elfa_set_deterministic", int(bool(on)))


def deterministic() -> bool:
    return _deterministic


def check_status() -> None:
    st = status()
    if st & (ST_MBAR_TIMEOUT | ST_FLAG_TIMEOUT):
        raise CommTimeout(f"a device-side wait timed out (status 0x{st:x})")
    if st & ST_BAD_TARGET:
        raise NativeError("token or target id outside the vocabulary")
    if st & ST_BOUNDS:
        raise NativeError("a kernel of the checked build computed an index outside the extents it was given (the access was skipped)")


def require_native(t: torch.Tensor) -> bool:
    """True when ``t`` must be handled by the native kernels (CUDA tensor). Raises if they are
    not built: a GPU run never falls back to eager PyTorch silently."""
    if not t.is_cuda:
        return False
    lib.load()
    return True
