"""Builds the single native library ``elfa_b200/_native/libelfa_b200.so`` from ``elfa_b200/csrc``.

Every ``.cu`` file is compiled for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``) with
``nvcc`` (no GPU needed: nvcc cross-compiles) and linked into one shared object that the Python
side loads with ``ctypes``. Objects are rebuilt only when their source or a header is newer.

    python -m elfa_b200.build [--force] [--verbose]

reference: ``scripts/build_kernels.sh:55-118`` builds one ``libcuda_<stem>.so`` per ``.cu`` with
``-arch=sm_100``; ``build.zig:42-69`` links them. Here there is one library and one arch.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT_DIR = PKG / "_native"
OBJ_DIR = OUT_DIR / "obj"
LIB = OUT_DIR / "libelfa_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def find_nvcc() -> str:
    cand = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found (set CUDA_HOME)")
    return cand


def source_hash() -> str:
    """SHA-256 over the names and contents of every native source and header: the identity of the sources a library was
    built from. It is compiled into the library (``elfa_source_hash``) and checked when the library is loaded."""
    import hashlib
    h = hashlib.sha256()
    for p in sorted(q for pat in ("*.cu", "*.cpp", "*.h", "*.hpp", "*.cuh") for q in CSRC.glob(pat)):
        h.update(p.name.encode())
        h.update(b"\0")
        h.update(p.read_bytes())
        h.update(b"\0")
    return h.hexdigest()


def _compile(nvcc: str, src: Path, obj: Path, verbose: bool, extra=()) -> str:
    cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return r.stderr


def lib_path(bounds: bool = False) -> Path:
    return OUT_DIR / "libelfa_b200_bounds.so" if bounds else LIB


def obj_dir(bounds: bool = False) -> Path:
    return OUT_DIR / "obj_bounds" if bounds else OBJ_DIR


def build(force: bool = False, verbose: bool = False, bounds: bool = False) -> Path:
    """Compile and link the native library. ``bounds``: the checked variant (``-DELFA_BOUNDS``): kernels test the tile
    coordinates, ring-slot offsets and push ranges they compute against the extents they were given, record a violation in
    the device status word (``ELFA_ST_BOUNDS``) and skip the access instead of making it. It is a separate library beside
    the normal one, loaded when ``ELFA_BOUNDS=1``."""
    if bounds:
        return _build_variant(force, verbose, lib_path(True), obj_dir(True), ("-DELFA_BOUNDS",))
    return _build_variant(force, verbose, LIB, OBJ_DIR, ())


def object_keys(csrc: Path, extra_flags=(), digest: str = "") -> dict:
    """``{source stem: key}``: an object file is current when the key recorded beside it equals the hash of its source, of
    every header it may include and of the extra compiler flags (file times do not survive a copy of the tree to another
    machine). ``runtime.cu`` also carries ``digest``, the hash of all sources, which is compiled into it."""
    import hashlib
    hdr = hashlib.sha256()
    for h in sorted(q for pat in ("*.h", "*.hpp", "*.cuh") for q in csrc.glob(pat)):
        hdr.update(h.name.encode() + b"\0" + h.read_bytes() + b"\0")
    hdr.update(" ".join(extra_flags).encode())
    keys = {}
    for src in sorted(csrc.glob("*.cu")) + sorted(csrc.glob("*.cpp")):
        key = hashlib.sha256(hdr.digest() + src.read_bytes()).hexdigest()
        if src.name == "runtime.cu":
            key = hashlib.sha256((key + digest).encode()).hexdigest()
        keys[src.stem] = key
    return keys


def _build_variant(force: bool, verbose: bool, LIB: Path, OBJ_DIR: Path, extra_flags) -> Path:
    nvcc = find_nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp"))
    if not sources:
        raise RuntimeError("no native sources found")
    digest = source_hash()
    stamp = OBJ_DIR / "source_hash.txt"
    jobs = []
    want = object_keys(CSRC, extra_flags, digest)
    for src in sources:
        obj = OBJ_DIR / (src.stem + ".o")
        rec = OBJ_DIR / (src.stem + ".hash")
        if force or not obj.exists() or not rec.exists() or rec.read_text().strip() != want[src.stem]:
            jobs.append((src, obj))
    if jobs:
        def flags(src):
            return tuple(extra_flags) + ((f'-DELFA_SOURCE_HASH="{digest}"',) if src.name == "runtime.cu" else ())
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for log in ex.map(lambda j: _compile(nvcc, j[0], j[1], verbose, flags(j[0])), jobs):
                if verbose and log:
                    print(log, file=sys.stderr)
        for src, _ in jobs:
            (OBJ_DIR / (src.stem + ".hash")).write_text(want[src.stem] + "\n")
    objs = [OBJ_DIR / (s.stem + ".o") for s in sources]
    if jobs or not LIB.exists():
        cmd = [nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart", "-Xcompiler", "-fPIC"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    stamp.write_text(digest + "\n")
    return LIB


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--bounds", action="store_true", help="build the checked variant (-DELFA_BOUNDS) beside the normal library")
    a = ap.parse_args(argv)
    print(build(force=a.force, verbose=a.verbose, bounds=a.bounds))
    return 0


if __name__ == "__main__":
    sys.exit(main())
