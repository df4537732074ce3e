"""Block-scaled NVFP4 GEMM (``tcgen05.mma.kind::mxf4nvf4.block_scale``) and its quantiser.

An operand is ``(payload, scales, amax)``: ``payload [rows, K / 2]`` bytes holding two e2m1 values
each (even element in the low nibble), ``scales`` ue4m3 bytes, one per 16 K-elements, in 512-byte
atoms of 128 rows x 4 blocks (same byte order inside an atom as the MXFP8 operands; left operands
ordered ``[row block][K / 64]``, right operands ``[K / 64][row block + 1 pad]``), and the tensor-level
``amax`` (device scalar): a value is ``e2m1 * scale * amax / (448 * 6)``.

The product differs from ``fake_quant(nvfp4)`` → bf16 GEMM only by the bf16 rounding that the
fake-quantised operands go through (their dequantised values have more than 8 mantissa bits).

reference: the NVFP4 format of ``src/tensor/dtype.zig:117-147`` / ``src/optimizer/stable_qat.zig:52-130``;
``src/ptx/tcgen05_kernels.ptx:482`` (``tensor_parallel_matmul_fp4``) is a stub without tensor-core code.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from ..native import EPI_BIAS, EPI_GELU, EPI_STORE_PREACT, lib, stream_ptr


@dataclass
class Nvfp4Operand:
    payload: torch.Tensor      # uint8 [rows, K / 2]
    scales: torch.Tensor       # uint8 atoms
    amax: torch.Tensor         # fp32 [1] on the device
    rows: int
    cols: int
    right: bool = False


def sf_numel(rows: int, cols: int, right: bool = False) -> int:
    return ((rows + 127) // 128 + (1 if right else 0)) * ((cols + 255) // 256 * 4) * 512


def quantize_nvfp4(x: torch.Tensor, dequantized: bool = False, right: bool = False,
                   amax: Optional[torch.Tensor] = None) -> Tuple[Nvfp4Operand, Optional[torch.Tensor]]:
    """``x [rows, K]`` bf16 → operand for :func:`gemm_nvfp4` plus (optionally) the bf16 tensor of
    dequantised values (bit-identical to ``fake_quant(x, nvfp4)``). ``amax``: precomputed max |x|."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    rows, cols = x.shape
    if cols % 32:
        raise ValueError("nvfp4: the contraction dimension must be a multiple of 32")
    st = stream_ptr(x)
    if amax is None:
        amax = torch.zeros(1, dtype=torch.float32, device=x.device)
        xc = x if x.is_contiguous() else x.contiguous()
        lib.call("elfa_amax", xc, xc.numel(), amax, st)
    payload = torch.empty((rows, cols // 2), dtype=torch.uint8, device=x.device)
    sf = torch.zeros(sf_numel(rows, cols, right), dtype=torch.uint8, device=x.device)
    deq = torch.empty((rows, cols), dtype=torch.bfloat16, device=x.device) if dequantized else None
    lib.call("elfa_nvfp4_quantize_gemm", x, x.stride(0), payload, sf, deq, rows, cols, int(right), amax, st)
    return Nvfp4Operand(payload, sf, amax, rows, cols, right), deq


def gemm_nvfp4(a: Nvfp4Operand, b: Nvfp4Operand, *, bias: Optional[torch.Tensor] = None, gelu: bool = False,
               preact: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, force_bn: int = 0) -> torch.Tensor:
    """``out[M, N] = epilogue(a[M, K] @ b[N, K]^T)`` in bf16. Epilogue order: ``+bias`` → store ``preact`` → GELU."""
    assert a.cols == b.cols, f"gemm_nvfp4: contraction mismatch {a.cols} vs {b.cols}"
    assert not a.right and b.right, "gemm_nvfp4: quantise the [N, K] matrix with right=True and the [M, K] matrix without"
    M, N, K = a.rows, b.rows, a.cols
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.payload.device)
    flags = (EPI_BIAS if bias is not None else 0) | (EPI_GELU if gelu else 0) | (EPI_STORE_PREACT if preact is not None else 0)
    lib.call("elfa_gemm_nvfp4", a.payload, a.scales, a.amax, b.payload, b.scales, b.amax, out, M, N, K, out.stride(0), bias, preact,
             preact.stride(0) if preact is not None else 0, flags, force_bn, stream_ptr(a.payload))
    return out


_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def dequantize_ref(op: Nvfp4Operand) -> torch.Tensor:
    """fp32 values of an operand, decoded with plain PyTorch (test oracle)."""
    rows, cols = op.rows, op.cols
    dev = op.payload.device
    lut = torch.tensor(_E2M1 + tuple(-v for v in _E2M1), dtype=torch.float32, device=dev)
    lo = (op.payload & 0xF).long()
    hi = (op.payload >> 4).long()
    vals = torch.stack([lut[lo], lut[hi]], dim=-1).reshape(rows, cols)
    r = torch.arange(rows, device=dev).unsqueeze(1)
    kb = torch.arange(cols // 16, device=dev).unsqueeze(0)
    k64 = (cols + 255) // 256 * 4
    atom = (kb // 4) * ((rows + 127) // 128 + 1) + r // 128 if op.right else (r // 128) * k64 + kb // 4
    idx = atom * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4
    sb = op.scales[idx.reshape(-1)].reshape(rows, cols // 16).view(torch.float8_e4m3fn).float()
    ts = op.amax.float() / (448.0 * 6.0) if float(op.amax) > 0 else torch.ones((), device=dev)
    return vals * (sb * ts).repeat_interleave(16, dim=1)
