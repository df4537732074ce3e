"""Tracing: NVTX ranges for external profilers and an in-process phase timer.

* :func:`nvtx_range` marks a region for ``nsys`` / ``ncu --nvtx`` (a no-op without CUDA or when tracing is off).
* :class:`PhaseTimer` times named phases of a training step on the device (CUDA events on the current
  stream, read back only when a summary is asked for, so nothing synchronises inside the step) or on the
  host clock for CPU runs, keeps per-phase totals and can write a Chrome ``trace_event`` file of the host
  ranges. The trainer wraps forward / backward / optimizer with it when ``ELFA_TRACE=1``.

reference: ``scripts/profile.sh:11-42`` (``nsys --trace=cuda,nvtx,...``: NVTX is requested there, but no
range exists in the code), ``src/runtime/cuda.zig:318-341`` (``CudaEvent.elapsedTime``), ``build.zig:59-62``
(``-Denable-profiling``).
"""
from __future__ import annotations

import contextlib
import json
import os
import time
from typing import Dict, List, Optional, Tuple

import torch

_ENABLED = os.environ.get("ELFA_TRACE", "0") not in ("0", "")


def enable(on: bool = True) -> None:
    global _ENABLED
    _ENABLED = bool(on)


def enabled() -> bool:
    return _ENABLED


@contextlib.contextmanager
def nvtx_range(name: str):
    """``with nvtx_range("layer3.attn"):`` - pushes / pops an NVTX range when tracing is on and CUDA is present."""
    use = _ENABLED and torch.cuda.is_available()
    if use:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if use:
            torch.cuda.nvtx.range_pop()


class PhaseTimer:
    """Accumulates the time spent in named phases.

    ``with timer.phase("forward"): ...`` may be entered many times per step (once per micro-batch); the
    device time between the two events of every entry is added to the phase's total when
    :meth:`summary` runs. Phases may nest; a nested phase's time is also part of its parent's."""

    def __init__(self, device: Optional[torch.device] = None, active: Optional[bool] = None):
        self.device = device
        self.cuda = device is not None and device.type == "cuda"
        self.active = _ENABLED if active is None else active
        self._pending: List[Tuple[str, object, object]] = []       # (name, start event, end event)
        self._totals: Dict[str, float] = {}
        self._counts: Dict[str, int] = {}
        self._host: List[Tuple[str, float, float]] = []            # (name, t0, t1) seconds, host clock
        self._t_origin = time.perf_counter()

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.active:
            yield
            return
        h0 = time.perf_counter()
        if self.cuda:
            torch.cuda.nvtx.range_push(name)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        try:
            yield
        finally:
            h1 = time.perf_counter()
            self._host.append((name, h0 - self._t_origin, h1 - self._t_origin))
            if self.cuda:
                e1.record()
                torch.cuda.nvtx.range_pop()
                self._pending.append((name, e0, e1))
            else:
                self._totals[name] = self._totals.get(name, 0.0) + (h1 - h0) * 1e3
                self._counts[name] = self._counts.get(name, 0) + 1

    def _drain(self) -> None:
        if not self._pending:
            return
        torch.cuda.synchronize(self.device)
        for name, e0, e1 in self._pending:
            self._totals[name] = self._totals.get(name, 0.0) + e0.elapsed_time(e1)
            self._counts[name] = self._counts.get(name, 0) + 1
        self._pending.clear()

    def summary(self, reset: bool = False) -> Dict[str, Dict[str, float]]:
        """``{phase: {"ms": total, "calls": n}}`` (synchronises the device once)."""
        self._drain()
        out = {k: {"ms": v, "calls": self._counts[k]} for k, v in self._totals.items()}
        if reset:
            self._totals.clear()
            self._counts.clear()
        return out

    def write_chrome_trace(self, path: str, pid: int = 0) -> None:
        """Host-side ranges in the Chrome ``trace_event`` format (open in ``chrome://tracing`` or Perfetto)."""
        ev = [{"name": n, "ph": "X", "pid": pid, "tid": 0, "ts": t0 * 1e6, "dur": (t1 - t0) * 1e6} for n, t0, t1 in self._host]
        with open(path, "w") as f:
            json.dump({"traceEvents": ev, "displayTimeUnit": "ms"}, f)
