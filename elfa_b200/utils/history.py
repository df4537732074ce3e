"""Training book-keeping: loss history, moving average, early-stop test, run manifest.

reference: ``src/trainer.zig:36-322`` (the first-generation trainer: loss history, ``manifest.json`` next to
``checkpoint_N.bin``, evaluation result log, moving-average loss, early-stop test with patience).
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional


@dataclass
class LossHistory:
    losses: List[float] = field(default_factory=list)
    steps: List[int] = field(default_factory=list)
    evals: List[Dict[str, float]] = field(default_factory=list)

    def record(self, step: int, loss: float) -> None:
        self.steps.append(int(step))
        self.losses.append(float(loss))

    def record_eval(self, step: int, **metrics: float) -> None:
        self.evals.append({"step": int(step), **{k: float(v) for k, v in metrics.items()}})

    def moving_average(self, window: int = 100) -> float:
        """Mean of the last ``window`` finite losses (NaN when there is none)."""
        xs = [x for x in self.losses[-max(window, 1):] if x == x and x not in (float("inf"), float("-inf"))]
        return sum(xs) / len(xs) if xs else float("nan")

    def best(self) -> float:
        xs = [x for x in self.losses if x == x]
        return min(xs) if xs else float("inf")

    def should_stop_early(self, patience: int, min_delta: float = 0.0, window: int = 1) -> bool:
        """True when the (windowed) loss has not improved by more than ``min_delta`` for ``patience`` records."""
        if patience <= 0 or len(self.losses) <= patience:
            return False
        def avg(i):       # windowed loss ending at record i (inclusive)
            lo = max(0, i - window + 1)
            xs = [x for x in self.losses[lo:i + 1] if x == x]
            return sum(xs) / len(xs) if xs else float("inf")
        n = len(self.losses)
        best_before = min(avg(i) for i in range(0, n - patience))
        best_recent = min(avg(i) for i in range(n - patience, n))
        return best_recent > best_before - min_delta

    def write_manifest(self, directory: str, extra: Optional[Dict[str, object]] = None) -> str:
        """``manifest.json`` in ``directory``: steps, losses, evaluation log, best loss, moving average."""
        os.makedirs(directory, exist_ok=True)
        path = os.path.join(directory, "manifest.json")
        doc = {"written": int(time.time()), "num_steps": len(self.steps), "best_loss": self.best(),
               "moving_average_100": self.moving_average(100), "steps": self.steps, "losses": self.losses, "evals": self.evals}
        if extra:
            doc.update(extra)
        tmp = path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(doc, f)
        os.replace(tmp, path)
        return path
