"""Gradient clipping (global L2 norm or value) and loss scaling.

reference: ``src/optim/optimizer.zig:524-593`` (``GradientClipper`` with norm / value modes: global
L2 in f64, scale by ``max_norm / norm`` when ``norm > max_norm`` and ``> 1e-8``, returns the
pre-clip norm); YAML knobs ``training.loss_scale`` / ``dynamic_loss_scale``
(``src/util/config.zig:419-423``) which the reference parses but never uses.

On CUDA the norm and the clip coefficient are computed by kernels inside the optimizer step (no
host round trip); this class is the host/CPU form and the public API for standalone use.
"""
from __future__ import annotations

import math
from typing import Iterable

import torch


class GradientClipper:
    def __init__(self, mode: str = "norm", max_value: float = 1.0):
        if mode not in ("norm", "value"):
            raise ValueError(mode)
        self.mode, self.max_value = mode, float(max_value)

    @staticmethod
    def global_norm(grads: Iterable[torch.Tensor]) -> float:
        tot = 0.0
        for g in grads:
            tot += float(g.double().pow(2).sum())
        return math.sqrt(tot)

    def clip(self, grads: Iterable[torch.Tensor]) -> float:
        grads = [g for g in grads if g is not None]
        norm = self.global_norm(grads)
        if self.mode == "value":
            for g in grads:
                g.clamp_(-self.max_value, self.max_value)
            return norm
        if self.max_value > 0 and norm > self.max_value and norm > 1e-8:
            s = self.max_value / norm
            for g in grads:
                g.mul_(s)
        return norm


class LossScaler:
    """Static or dynamic loss scale. Dynamic: halve on a skipped (non-finite) step, double after
    ``growth_interval`` good steps."""

    def __init__(self, init_scale: float = 1.0, dynamic: bool = False, growth_interval: int = 1000, min_scale: float = 1.0,
                 max_scale: float = 2.0 ** 24):
        self.scale, self.dynamic = float(init_scale), bool(dynamic)
        self.growth_interval, self.min_scale, self.max_scale = growth_interval, min_scale, max_scale
        self.good_steps = 0
        self.skipped_steps = 0

    def update(self, skipped: bool) -> None:
        if skipped:
            self.skipped_steps += 1
        if not self.dynamic:
            return
        if skipped:
            self.scale = max(self.scale * 0.5, self.min_scale)
            self.good_steps = 0
        else:
            self.good_steps += 1
            if self.good_steps >= self.growth_interval:
                self.scale = min(self.scale * 2.0, self.max_scale)
                self.good_steps = 0

    def state_dict(self):
        return {"scale": self.scale, "good_steps": self.good_steps, "skipped_steps": self.skipped_steps}

    def load_state_dict(self, sd):
        self.scale, self.good_steps = float(sd["scale"]), int(sd["good_steps"])
        self.skipped_steps = int(sd.get("skipped_steps", 0))
