"""Block-scaled MXFP8 GEMM (``tcgen05.mma.kind::mxf8f6f4.block_scale``) and its quantiser.

An operand is a pair ``(payload, scales)``: ``payload [rows, K]`` e4m3 bytes (K contiguous) and
``scales`` ue8m0 bytes, one per 32 K-elements, stored in 512-byte atoms of 128 rows x 4 K-blocks
(byte ``(r % 32) * 16 + (r % 128 // 32) * 4 + kb % 4`` of an atom) - the layout the tensor core copies
into tensor memory with one instruction per atom. Atoms of a left operand are ordered
``[r // 128][kb // 4]``, atoms of a right operand ``[kb // 4][r // 128]`` with one atom of padding per
K tile, so that the atoms one output tile needs are contiguous in both cases.

``y = gemm_mxfp8(xq, wq)`` multiplies ``x [M, K]`` by ``w^T`` with ``w`` given as ``[N, K]``; the
result equals the bf16 GEMM of the fake-quantised operands up to fp32 summation order (the products
of e4m3 values and power-of-two scales are exact in fp32).

reference: the MX block format of ``src/tensor/dtype.zig:117-147`` / ``src/optimizer/stable_qat.zig:52-130``;
the reference has no block-scaled GEMM (``kernels/cuda/gemm_sm100.cu:74-112`` is a scalar-scale fp8
kernel, ``src/ptx/tcgen05_kernels.ptx:183,482`` are stubs).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from ..native import EPI_BIAS, EPI_GELU, EPI_STORE_PREACT, lib, stream_ptr


@dataclass
class Mxfp8Operand:
    payload: torch.Tensor      # uint8 [rows, K]
    scales: torch.Tensor       # uint8 [ceil(rows/128) * ceil(K/128) * 512]
    rows: int
    cols: int
    right: bool = False        # right-hand operand (the ``[N, K]`` matrix): different atom order


def sf_numel(rows: int, cols: int, right: bool = False) -> int:
    return ((rows + 127) // 128 + (1 if right else 0)) * ((cols + 127) // 128) * 512


def quantize_mxfp8(x: torch.Tensor, dequantized: bool = False, right: bool = False) -> Tuple[Mxfp8Operand, Optional[torch.Tensor]]:
    """``x [rows, K]`` bf16 (last dim contiguous) → operand for :func:`gemm_mxfp8` (``right`` for the
    ``[N, K]`` matrix), plus (optionally) the bf16 tensor of dequantised values, bit-identical to
    ``fake_quant(x, mxfp8)``."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    rows, cols = x.shape
    if cols % 32:
        raise ValueError("mxfp8: the contraction dimension must be a multiple of 32")
    payload = torch.empty((rows, cols), dtype=torch.uint8, device=x.device)
    n_sf = sf_numel(rows, cols, right)
    padded = right or rows % 128 != 0 or cols % 128 != 0
    sf = (torch.zeros if padded else torch.empty)(n_sf, dtype=torch.uint8, device=x.device)
    deq = torch.empty((rows, cols), dtype=torch.bfloat16, device=x.device) if dequantized else None
    lib.call("elfa_mxfp8_quantize_gemm", x, x.stride(0), payload, sf, deq, rows, cols, int(right), stream_ptr(x))
    return Mxfp8Operand(payload, sf, rows, cols, right), deq


def gemm_mxfp8(a: Mxfp8Operand, b: Mxfp8Operand, *, bias: Optional[torch.Tensor] = None, gelu: bool = False,
               preact: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, force_bn: int = 0) -> torch.Tensor:
    """``out[M, N] = epilogue(a[M, K] @ b[N, K]^T)`` in bf16. Epilogue order: ``+bias`` → store ``preact`` → GELU."""
    assert a.cols == b.cols, f"gemm_mxfp8: contraction mismatch {a.cols} vs {b.cols}"
    assert not a.right and b.right, "gemm_mxfp8: quantise the [N, K] matrix with right=True and the [M, K] matrix without"
    M, N, K = a.rows, b.rows, a.cols
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.payload.device)
    flags = (EPI_BIAS if bias is not None else 0) | (EPI_GELU if gelu else 0) | (EPI_STORE_PREACT if preact is not None else 0)
    lib.call("elfa_gemm_mxfp8", a.payload, a.scales, b.payload, b.scales, out, M, N, K, out.stride(0), bias, preact,
             preact.stride(0) if preact is not None else 0, flags, force_bn, stream_ptr(a.payload))
    return out


def dequantize_mxfp8(op: Mxfp8Operand, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 tensor of the values an operand stands for (exact), by the native kernel."""
    if out is None:
        out = torch.empty((op.rows, op.cols), dtype=torch.bfloat16, device=op.payload.device)
    lib.call("elfa_mxfp8_dequantize", op.payload, op.scales, out, op.rows, op.cols, int(op.right), stream_ptr(op.payload))
    return out


def dequantize_ref(op: Mxfp8Operand) -> torch.Tensor:
    """fp32 values of an operand, decoded with plain PyTorch (test oracle)."""
    rows, cols = op.rows, op.cols
    vals = op.payload.view(torch.float8_e4m3fn).float()
    r = torch.arange(rows, device=vals.device).unsqueeze(1)
    kb = torch.arange(cols // 32, device=vals.device).unsqueeze(0)
    kt = (cols + 127) // 128
    atom = (kb // 4) * ((rows + 127) // 128 + 1) + r // 128 if op.right else (r // 128) * kt + kb // 4
    idx = atom * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4
    e = op.scales[idx.reshape(-1)].reshape(rows, cols // 32).to(torch.int32) - 127
    scale = torch.pow(torch.tensor(2.0, device=vals.device, dtype=torch.float64), e.double()).float()
    return vals * scale.repeat_interleave(32, dim=1)
