"""Quantisation-aware training: fake-quant of GEMM operands with surrogate gradients.

Modes (``quant.attention`` / ``quant.mlp`` in the YAML):

* ``mxfp8``      - e4m3 values, 1x32 ue8m0 block scales along the contraction dimension;
* ``nvfp4``      - e2m1 values, 16-element e4m3 block scales and one fp32 tensor scale;
* ``fp8_tensor`` - per-tensor e4m3 with delayed scaling (16-deep amax history);
* ``int_affine`` - min/max affine to ``weight_bits`` bits (the reference's "StableQAT").

Backward is the straight-through estimator by default; the reference's sigmoid-tempered and
piecewise-linear surrogates are available for ``int_affine`` weights
(reference: ``src/quantization/stable_qat.zig:12-16,52-106``).

``fake_quant`` is called inside the linear autograd functions (which implement the
straight-through backward themselves); :func:`fake_quant_ste` is the standalone autograd op.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import formats

SURROGATE = {"straight_through": 0, "sigmoid_tempered": 1, "piecewise_linear": 2}


@dataclass
class QuantSpec:
    fmt: str = "none"
    bits: int = 8
    surrogate: str = "straight_through"
    temperature: float = 0.1
    threshold: float = 1.0
    outside_slope: float = 0.1
    block_scaled_gemm: bool = True
    backward: str = "none"        # "mxfp8": output gradients and the weights' other axis are quantised for the input-gradient GEMMs

    @property
    def quant_backward(self) -> bool:
        return self.fmt != "none" and self.backward == "mxfp8"

    @property
    def enabled(self) -> bool:
        return self.fmt != "none"

    @classmethod
    def from_config(cls, fmt: str, qcfg) -> "QuantSpec":
        return cls(fmt=fmt, bits=qcfg.weight_bits, surrogate=qcfg.surrogate,
                   block_scaled_gemm=bool(getattr(qcfg, "block_scaled_gemm", True)), backward=getattr(qcfg, "backward", "none"))


_amax_buf = {}
_scale_state = {}

# Fake-quantised weights are reused by every micro-batch of an optimizer step: the cache is keyed on
# the parameter and invalidated by `new_weight_epoch()` (called after each optimizer update).
_weight_cache = {}
_weight_epoch = 0


def new_weight_epoch() -> None:
    global _weight_epoch
    _weight_epoch += 1
    _weight_cache.clear()


def cached_weight_quant(w: torch.Tensor, spec: "QuantSpec") -> torch.Tensor:
    key = (id(w), spec.fmt, spec.bits)
    hit = _weight_cache.get(key)
    if hit is not None and hit[0] is w:
        return hit[1]
    wq = fake_quant(w.detach(), spec, weight=True)
    _weight_cache[key] = (w, wq)
    return wq


def cached_weight_operand(w: torch.Tensor, spec: "QuantSpec"):
    """Block-scaled tensor-core operand (MXFP8 or NVFP4) of a ``[K, N]`` weight: payload ``[N, K]`` with
    scales along K, the same blocks as ``fake_quant(w, weight=True)``. Cached like the bf16 copy."""
    key = (id(w), spec.fmt + "_operand")
    hit = _weight_cache.get(key)
    if hit is not None and hit[0] is w:
        return hit[1]
    wt = w.detach().t().contiguous()
    if spec.fmt == "nvfp4":
        from ..ops.gemm_nvfp4 import quantize_nvfp4
        op, _ = quantize_nvfp4(wt, right=True)
    else:
        from ..ops.gemm_mxfp8 import quantize_mxfp8
        op, _ = quantize_mxfp8(wt, right=True)
    _weight_cache[key] = (w, op)
    return op


def cached_weight_quant_bwd(w: torch.Tensor, spec: "QuantSpec") -> torch.Tensor:
    """``[K, N]`` weight fake-quantised (MXFP8) with blocks along N, the contraction dimension of ``dx = dy @ w^T``."""
    key = (id(w), "mxfp8_bwd")
    hit = _weight_cache.get(key)
    if hit is not None and hit[0] is w:
        return hit[1]
    wq = fake_quant(w.detach(), QuantSpec(fmt="mxfp8"), weight=False)
    _weight_cache[key] = (w, wq)
    return wq


def cached_weight_operand_bwd(w: torch.Tensor, spec: "QuantSpec"):
    """Right-hand MXFP8 operand of the input-gradient GEMM: the ``[K, N]`` weight as it lies in memory (rows of N
    contiguous elements), scales along N. Same blocks as :func:`cached_weight_quant_bwd`."""
    key = (id(w), "mxfp8_bwd_operand")
    hit = _weight_cache.get(key)
    if hit is not None and hit[0] is w:
        return hit[1]
    from ..ops.gemm_mxfp8 import quantize_mxfp8
    wd = w.detach()
    op, _ = quantize_mxfp8(wd if wd.is_contiguous() else wd.contiguous(), right=True)
    _weight_cache[key] = (w, op)
    return op


def use_block_scaled_bwd(dy2: torch.Tensor, w: torch.Tensor, spec: Optional["QuantSpec"]) -> bool:
    """True when ``dx = dy2 [T, N] @ w[K, N]^T`` runs on the block-scaled tensor-core path."""
    return (spec is not None and spec.quant_backward and spec.block_scaled_gemm and dy2.is_cuda and dy2.dtype == torch.bfloat16
            and w.dtype == torch.bfloat16 and dy2.shape[1] % 32 == 0 and w.shape[0] % 8 == 0)


def quantize_grad(dy2: torch.Tensor):
    """MXFP8 quantisation of an output gradient ``[T, N]`` (blocks along N). Returns ``(operand or None, dyq)``:
    the tensor-core operand (CUDA bf16 only) and the tensor of dequantised values in ``dy2``'s dtype."""
    if dy2.is_cuda and dy2.dtype == torch.bfloat16 and dy2.shape[1] % 32 == 0:
        from ..ops.gemm_mxfp8 import quantize_mxfp8
        return quantize_mxfp8(dy2 if dy2.is_contiguous() else dy2.contiguous(), dequantized=True)
    return None, fake_quant(dy2, QuantSpec(fmt="mxfp8"), weight=False)


def use_block_scaled_gemm(x2: torch.Tensor, w: torch.Tensor, spec: Optional["QuantSpec"]) -> bool:
    """True when the forward GEMM ``x2 [T, K] @ w [K, N]`` can run on a block-scaled tensor-core path
    (MXFP8: exactly the fake-quantised product; NVFP4: the same up to the bf16 rounding of the
    fake-quantised operands)."""
    return (spec is not None and spec.fmt in ("mxfp8", "nvfp4") and spec.block_scaled_gemm and x2.is_cuda and x2.dtype == torch.bfloat16
            and w.dtype == torch.bfloat16 and x2.shape[1] % 32 == 0 and w.shape[1] % 8 == 0)


def _scratch(device, n):
    b = _amax_buf.get(device)
    if b is None or b.numel() < n:
        b = torch.zeros(max(n, 8192), dtype=torch.float32, device=device)
        _amax_buf[device] = b
    return b


def fake_quant(x: torch.Tensor, spec: Optional[QuantSpec], weight: bool = False) -> torch.Tensor:
    """Quantise-dequantise ``x`` (2-D). Activations ``[tokens, K]`` use blocks along the last
    dimension; weights ``[K, N]`` (``weight=True``) use blocks along dim 0 - in both cases the
    contraction dimension of the GEMM that consumes them."""
    if spec is None or not spec.enabled:
        return x
    assert x.dim() == 2
    axis = 0 if weight else 1
    if not x.is_cuda:
        if spec.fmt == "mxfp8":
            return formats.mxfp8_fake_quant_ref(x, axis)
        if spec.fmt == "nvfp4":
            return formats.nvfp4_fake_quant_ref(x, axis)
        if spec.fmt == "fp8_tensor":
            amax = float(x.abs().max())
            sc = formats.E4M3_MAX / amax if amax > 0 else 1.0
            return (formats.e4m3_round(x.float() * sc) / sc).to(x.dtype)
        if spec.fmt == "int_affine":
            lo, hi = float(x.min()), float(x.max())
            qmax = float(2 ** spec.bits - 1)
            sc = (hi - lo) / qmax if hi > lo else 1.0
            zp = -lo / sc
            q = torch.clamp(torch.round(x.float() / sc + zp), 0, qmax)
            return ((q - zp) * sc).to(x.dtype)
        raise ValueError(spec.fmt)
    from ..native import lib, stream_ptr
    xc = x if x.is_contiguous() else x.contiguous()
    out = torch.empty_like(xc)
    rows, cols = xc.shape
    st = stream_ptr(xc)
    if spec.fmt == "mxfp8":
        if axis == 1 and cols % 32:
            raise ValueError("mxfp8: the contraction dimension must be a multiple of 32")
        lib.call("elfa_mxfp8_fake_quant", xc, out, rows, cols, axis, st)
    elif spec.fmt == "nvfp4":
        amax = torch.zeros(1, dtype=torch.float32, device=x.device)
        lib.call("elfa_amax", xc, xc.numel(), amax, st)
        lib.call("elfa_nvfp4_fake_quant", xc, out, rows, cols, axis, amax, st)
    elif spec.fmt == "fp8_tensor":
        # current-tensor scaling on the device (no host sync): scale = 448 / amax
        amax = torch.zeros(1, dtype=torch.float32, device=x.device)
        lib.call("elfa_amax", xc, xc.numel(), amax, st)
        scale = torch.where(amax > 0, formats.E4M3_MAX / amax, torch.ones_like(amax))
        lib.call("elfa_fp8_tensor_fake_quant", xc, out, xc.numel(), scale, 0, st)
    elif spec.fmt == "int_affine":
        mm = torch.empty(2, dtype=torch.float32, device=x.device)
        lib.call("elfa_int_affine_fake_quant", xc, out, xc.numel(), spec.bits, mm, _scratch(x.device, 8192), st)
    else:
        raise ValueError(spec.fmt)
    return out


class _FakeQuantSTE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, spec, weight):
        ctx.spec = spec
        ctx.save_for_backward(x)
        return fake_quant(x, spec, weight)

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        spec = ctx.spec
        mode = SURROGATE[spec.surrogate]
        if mode == 0:
            return g, None, None
        p0 = spec.temperature if mode == 1 else spec.threshold
        if not x.is_cuda:
            xf, gf = x.float(), g.float()
            if mode == 1:
                s = torch.sigmoid(xf / p0)
                return (gf * s * (1 - s) / p0).to(g.dtype), None, None
            return torch.where(xf.abs() <= p0, gf, gf * spec.outside_slope).to(g.dtype), None, None
        from ..native import lib, stream_ptr
        out = torch.empty_like(g)
        lib.call("elfa_qat_surrogate_bwd", x.contiguous(), g.contiguous(), out, x.numel(), mode, float(p0), float(spec.outside_slope),
                 stream_ptr(x))
        return out, None, None


def fake_quant_ste(x: torch.Tensor, spec: QuantSpec, weight: bool = False) -> torch.Tensor:
    """Autograd version: forward quantise-dequantise, backward per ``spec.surrogate``."""
    return _FakeQuantSTE.apply(x, spec, weight)
