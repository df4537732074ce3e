"""Layout helpers: padding, tensor-core tile constants and a best-fit host memory pool.

reference: ``src/tensor/layout.zig:3-48`` (``Layout`` enum), ``:50-91`` (``PaddingStrategy`` with 128-byte
alignment and ``optimalLeadingDimension``), ``:93-105`` (``TensorCoreTiles``), ``:107-247`` (best-fit
host ``MemoryPool`` with defragmentation). The tile constants are the ones this library's tcgen05
kernels actually use.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

LAYOUTS = ("row_major", "col_major", "aligned", "nchw", "nhwc", "tensor_core_a", "tensor_core_b", "tensor_core_c")


@dataclass(frozen=True)
class TensorCoreTiles:
    block_m: int = 128          # rows of one tcgen05.mma (cta_group::1)
    block_n: int = 256          # widest accumulator tile of the GEMM (also 128 and 64)
    block_k: int = 64           # one 128-byte swizzle span of bf16
    mma_k: int = 16             # K of one tcgen05.mma.kind::f16 instruction
    tmem_columns: int = 512


@dataclass
class PaddingStrategy:
    alignment: int = 128        # bytes

    def padded_bytes(self, nbytes: int) -> int:
        a = self.alignment
        return (nbytes + a - 1) // a * a

    def optimal_leading_dimension(self, cols: int, elem_bytes: int) -> int:
        """Smallest leading dimension >= cols whose row pitch is a multiple of the alignment."""
        per = max(self.alignment // elem_bytes, 1)
        return (cols + per - 1) // per * per


class HostMemoryPool:
    """Best-fit allocator over one address range (offsets, not pointers) with coalescing free."""

    def __init__(self, capacity: int, alignment: int = 128):
        self.capacity, self.alignment = capacity, alignment
        self.free: List[Tuple[int, int]] = [(0, capacity)]     # (offset, size), sorted by offset
        self.used: Dict[int, int] = {}

    def alloc(self, size: int) -> int:
        size = (size + self.alignment - 1) // self.alignment * self.alignment
        best = None
        for i, (off, sz) in enumerate(self.free):
            if sz >= size and (best is None or sz < self.free[best][1]):
                best = i
        if best is None:
            raise MemoryError(f"pool exhausted: {size} bytes requested, largest free block {max((s for _, s in self.free), default=0)}")
        off, sz = self.free.pop(best)
        if sz > size:
            self.free.insert(best, (off + size, sz - size))
        self.used[off] = size
        return off

    def release(self, offset: int) -> None:
        size = self.used.pop(offset)
        self.free.append((offset, size))
        self.defragment()

    def defragment(self) -> None:
        self.free.sort()
        merged: List[Tuple[int, int]] = []
        for off, sz in self.free:
            if merged and merged[-1][0] + merged[-1][1] == off:
                merged[-1] = (merged[-1][0], merged[-1][1] + sz)
            else:
                merged.append((off, sz))
        self.free = merged

    def bytes_in_use(self) -> int:
        return sum(self.used.values())
