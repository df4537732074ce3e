"""Learning-rate schedules.

reference: ``src/optim/optimizer.zig:443-521`` (constant, linear_warmup, cosine,
linear_warmup_cosine) and the gen-1 trainer's linear / polynomial(2) decays
(``src/trainer.zig:36-61``). Warm-up is ``lr * max(1, step) / warmup``; the cosine part is
``min + (lr - min) * 0.5 * (1 + cos(pi * clamp((step - warmup) / (total - warmup))))``.
"""
from __future__ import annotations

import math


class LRScheduler:
    KINDS = ("constant", "linear_warmup", "cosine", "linear_warmup_cosine", "linear", "polynomial")

    def __init__(self, kind: str, base_lr: float, min_lr: float = 0.0, warmup_steps: int = 0, total_steps: int = 1):
        if kind not in self.KINDS:
            raise ValueError(f"unknown lr schedule {kind!r}")
        self.kind, self.base_lr, self.min_lr = kind, float(base_lr), float(min_lr)
        self.warmup_steps, self.total_steps = int(warmup_steps), max(int(total_steps), 1)
        self.step_count = 0

    def _progress(self, step: int, start: int) -> float:
        span = max(self.total_steps - start, 1)
        return min(max((step - start) / span, 0.0), 1.0)

    def lr_at(self, step: int) -> float:
        k = self.kind
        warm = k in ("linear_warmup", "linear_warmup_cosine") and self.warmup_steps > 0
        if warm and step < self.warmup_steps:
            return self.base_lr * max(1, step) / self.warmup_steps
        if k in ("constant", "linear_warmup"):
            return self.base_lr
        start = self.warmup_steps if warm else 0
        t = self._progress(step, start)
        if k in ("cosine", "linear_warmup_cosine"):
            return self.min_lr + (self.base_lr - self.min_lr) * 0.5 * (1.0 + math.cos(math.pi * t))
        if k == "linear":
            return self.base_lr + (self.min_lr - self.base_lr) * t
        return self.min_lr + (self.base_lr - self.min_lr) * (1.0 - t) ** 2      # polynomial(2)

    def get_lr(self) -> float:
        return self.lr_at(self.step_count)

    def step(self) -> float:
        self.step_count += 1
        return self.get_lr()

    def state_dict(self):
        return {"step": self.step_count}

    def load_state_dict(self, sd):
        self.step_count = int(sd["step"])
