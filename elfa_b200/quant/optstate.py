"""Optimizer-state and gradient quantisation (memory savers).

reference: ``src/quantization/optimizer_quant.zig:27-85`` (state fake-quant to ``optimizer_state_bits``,
int8 momentum with absmax/127), ``:87-177`` (blockwise 4/8-bit with a scale and zero point per
block, nibble packed), ``:179-250`` (dynamic per-tensor u8, int8 gradients).
"""
from __future__ import annotations

from typing import Tuple

import torch


def quantize_int8_absmax(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Symmetric int8: ``q = round(x / s)``, ``s = absmax / 127``."""
    amax = x.abs().max().clamp_min(1e-12)
    s = amax / 127.0
    return torch.clamp(torch.round(x / s), -127, 127).to(torch.int8), s


def dequantize_int8_absmax(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    return q.float() * s


def quantize_blockwise(x: torch.Tensor, bits: int = 8, block_size: int = 256):
    """Affine per-block quantisation to ``bits`` (4 or 8). Returns (codes uint8 - nibble packed for 4
    bits, scale [nblocks], zero_point [nblocks], numel)."""
    assert bits in (4, 8)
    flat = x.reshape(-1).float()
    n = flat.numel()
    pad = (-n) % block_size
    if pad:
        flat = torch.nn.functional.pad(flat, (0, pad))
    b = flat.view(-1, block_size)
    lo, hi = b.min(1).values, b.max(1).values
    qmax = float(2 ** bits - 1)
    scale = ((hi - lo) / qmax).clamp_min(1e-12)
    zp = -lo / scale
    q = torch.clamp(torch.round(b / scale[:, None] + zp[:, None]), 0, qmax).to(torch.uint8)
    if bits == 4:
        q = q.view(-1, 2)
        q = (q[:, 0] | (q[:, 1] << 4)).contiguous()
    return q.reshape(-1), scale, zp, n


def dequantize_blockwise(q: torch.Tensor, scale: torch.Tensor, zp: torch.Tensor, numel: int, bits: int = 8,
                         block_size: int = 256) -> torch.Tensor:
    if bits == 4:
        q = torch.stack([q & 0xF, q >> 4], -1).reshape(-1)
    b = q.view(-1, block_size).float()
    return ((b - zp[:, None]) * scale[:, None]).reshape(-1)[:numel]


def fake_quantize_state(x: torch.Tensor, bits: int) -> torch.Tensor:
    """Round-trip of an optimizer state tensor through ``bits``-bit symmetric quantisation."""
    if bits >= 32:
        return x
    qmax = float(2 ** (bits - 1) - 1)
    s = x.abs().max().clamp_min(1e-12) / qmax
    return torch.clamp(torch.round(x / s), -qmax, qmax) * s


def quantize_dynamic_u8(x: torch.Tensor):
    lo, hi = x.min(), x.max()
    s = ((hi - lo) / 255.0).clamp_min(1e-12)
    return torch.clamp(torch.round((x - lo) / s), 0, 255).to(torch.uint8), s, lo


def dequantize_dynamic_u8(q, s, lo):
    return q.float() * s + lo
