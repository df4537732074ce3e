"""Software codecs of the low-precision formats (the bit-exact oracle of the CUDA kernels).

reference: ``src/tensor/dtype.zig:192-303`` (e4m3: bias 7, max 448, min subnormal 2^-9, NaN =
S.1111.111, overflow saturates to 448), ``:305-416`` (e5m2: bias 15, max 57344, overflow → inf),
``:418-455`` (bf16 round-to-nearest-even), ``:587-642`` (fp4 e2m1: {0, .5, 1, 1.5, 2, 3, 4, 6},
low nibble = even index), ``:85-148`` (``ScaleFactor``: delayed scaling over a 16-deep amax
history), ``:150-190`` (``BlockScale``).

The block formats are the Blackwell-native realisations of ``BlockScale``:
* MXFP8: 32-element blocks, one ue8m0 (power-of-two) scale, e4m3 values;
* NVFP4: 16-element blocks, one e4m3 scale per block, one fp32 scale per tensor, e2m1 values.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Tuple

import torch

E4M3_MAX = 448.0
E5M2_MAX = 57344.0
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.float().to(torch.bfloat16).float()


def e4m3_round(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even into e4m3 with saturation to +-448 (NaN stays NaN)."""
    xf = x.float()
    return xf.clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).float()


def e5m2_round(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even into e5m2; overflow becomes infinity."""
    return x.float().to(torch.float8_e5m2).float()


def e2m1_round(x: torch.Tensor) -> torch.Tensor:
    """Round to the nearest e2m1 value, ties to the even mantissa, saturating at +-6."""
    xf = x.float()
    a = xf.abs().clamp_max(6.0)
    # below 2 the grid step is 0.5, below 4 it is 1, else 2; torch.round is round-half-to-even
    r = torch.where(a < 2.0, torch.round(a * 2.0) / 2.0, torch.where(a < 4.0, torch.round(a), torch.round(a / 2.0) * 2.0))
    return torch.copysign(r, xf)


def e2m1_index(x: torch.Tensor) -> torch.Tensor:
    """4-bit code (sign bit 3, magnitude index 0..7) of already-rounded e2m1 values."""
    vals = torch.tensor(E2M1_VALUES, dtype=torch.float32, device=x.device)
    idx = (x.abs().unsqueeze(-1) - vals).abs().argmin(-1)
    return (idx + 8 * (x < 0).long()).to(torch.uint8)


def pack_fp4(x: torch.Tensor) -> torch.Tensor:
    """Packs e2m1 values two per byte, element 2i in the low nibble (flattened last dim must be even)."""
    codes = e2m1_index(e2m1_round(x)).reshape(-1, 2)
    return (codes[:, 0] | (codes[:, 1] << 4)).to(torch.uint8)


def unpack_fp4(packed: torch.Tensor) -> torch.Tensor:
    vals = torch.tensor(E2M1_VALUES + tuple(-v for v in E2M1_VALUES), dtype=torch.float32, device=packed.device)
    lo, hi = packed & 0xF, packed >> 4
    return torch.stack([vals[lo.long()], vals[hi.long()]], -1).reshape(-1)


def _mx_exponent(amax: torch.Tensor, emax_elem: int) -> torch.Tensor:
    e = torch.floor(torch.log2(amax.clamp_min(2.0 ** -126))) - emax_elem
    e = torch.where(amax > 0, e, torch.full_like(e, -127.0))
    return e.clamp(-127, 127)


def mxfp8_quantize_ref(x: torch.Tensor, axis: int = -1) -> Tuple[torch.Tensor, torch.Tensor]:
    """→ (values rounded to e4m3 (as fp32), ue8m0 exponents as int (unbiased)) with 32-element
    blocks along ``axis`` (padded with zeros to a multiple of 32 for the scale computation)."""
    xf = x.float().movedim(axis, -1)
    n = xf.shape[-1]
    pad = (-n) % 32
    if pad:
        xf = torch.nn.functional.pad(xf, (0, pad))
    blocks = xf.reshape(*xf.shape[:-1], -1, 32)
    e = _mx_exponent(blocks.abs().amax(-1), 8)
    scale = torch.pow(2.0, e).unsqueeze(-1)
    q = e4m3_round(blocks / scale)
    return q, e


def mxfp8_fake_quant_ref(x: torch.Tensor, axis: int = -1) -> torch.Tensor:
    q, e = mxfp8_quantize_ref(x, axis)
    deq = (q * torch.pow(2.0, e).unsqueeze(-1)).reshape(*q.shape[:-2], -1)
    n = x.movedim(axis, -1).shape[-1]
    return deq[..., :n].movedim(-1, axis).to(x.dtype)


def nvfp4_fake_quant_ref(x: torch.Tensor, axis: int = -1, tensor_amax: float | None = None) -> torch.Tensor:
    xf = x.float().movedim(axis, -1)
    n = xf.shape[-1]
    pad = (-n) % 16
    if pad:
        xf = torch.nn.functional.pad(xf, (0, pad))
    ta = float(xf.abs().max()) if tensor_amax is None else float(tensor_amax)
    ts = ta / (448.0 * 6.0) if ta > 0 else 1.0
    blocks = xf.reshape(*xf.shape[:-1], -1, 16)
    sb = e4m3_round(blocks.abs().amax(-1) / (6.0 * ts))
    full = (sb * ts).unsqueeze(-1)
    inv = torch.where(full > 0, 1.0 / full, torch.zeros_like(full))
    deq = (e2m1_round(blocks * inv) * full).reshape(*blocks.shape[:-2], -1)
    return deq[..., :n].movedim(-1, axis).to(x.dtype)


@dataclass
class ScaleFactor:
    """Per-tensor delayed scaling: ``scale = target_max / max(amax history)``."""
    target_max: float = E4M3_MAX
    history_len: int = 16
    history: List[float] = field(default_factory=list)
    scale: float = 1.0

    def update(self, amax: float) -> float:
        self.history.append(abs(float(amax)))
        if len(self.history) > self.history_len:
            self.history.pop(0)
        m = max(self.history)
        if m > 0 and math.isfinite(m):
            self.scale = self.target_max / m
        return self.scale


@dataclass
class BlockScale:
    """Generic block scaling descriptor: ``block_size`` elements share one scale."""
    block_size: int = 32
    scale_format: str = "ue8m0"     # or "e4m3" (NVFP4)

    def num_blocks(self, n: int) -> int:
        return (n + self.block_size - 1) // self.block_size
