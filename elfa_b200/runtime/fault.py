"""Failure detection and host-side fault injection.

The reference has neither (only error-code tables, an unused ``ncclCommAbort`` binding and a
``HealthStatus`` record: ``src/runtime/cuda.zig:72-137``, ``src/nccl_bindings.zig:39-40``,
``src/telemetry/main.zig:159-226``). What this module adds:

* :class:`Heartbeat`: every rank writes ``<dir>/rank_<r>.hb`` (step, wall time) at each step
  boundary; :meth:`Heartbeat.wait_for_peers` is a soft barrier over those files with a timeout, so a
  rank that died between steps is noticed on the host *before* the survivors enter the next
  collective (which would otherwise block until the process-group timeout).
* :class:`FaultPlan`: faults requested through ``ELFA_FAULT`` and injected on the host only, e.g.
  ``ELFA_FAULT="nan_grad:rank=1,step=3;delay_ms:rank=0,step=2,ms=50;kill_rank:rank=2,step=4"``.
  ``nan_grad`` writes a NaN into the gradient buffer before the optimizer step (the step must be
  skipped and the dynamic loss scale halved), ``delay_ms`` sleeps before the step, ``kill_rank`` makes
  the rank leave between steps (no kernel or collective in flight), ``skip_signal`` makes a rank skip one
  fused collective so that its peers' bounded waits expire. Nothing here touches a GPU's state:
  device-side fault injection is deliberately absent.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional


class RankFailure(RuntimeError):
    """One or more peers stopped reporting."""

    def __init__(self, ranks: List[int], step: int, waited_s: float):
        super().__init__(f"rank(s) {ranks} did not reach step {step} within {waited_s:.1f} s")
        self.ranks, self.step = ranks, step


@dataclass
class Fault:
    kind: str
    args: Dict[str, float] = field(default_factory=dict)

    def matches(self, rank: int, step: int) -> bool:
        # ``attempt=k`` limits a fault to the k-th start of the job under the restarting launcher (0 = first start)
        attempt = int(os.environ.get("ELFA_RESTART_ATTEMPT", "0"))
        return (int(self.args.get("rank", rank)) == rank and int(self.args.get("step", step)) == step
                and int(self.args.get("attempt", attempt)) == attempt)


class FaultPlan:
    KINDS = ("nan_grad", "delay_ms", "kill_rank", "skip_signal")

    def __init__(self, faults: Optional[List[Fault]] = None):
        self.faults = faults or []

    @classmethod
    def parse(cls, text: str) -> "FaultPlan":
        faults = []
        for item in filter(None, (s.strip() for s in text.split(";"))):
            kind, _, rest = item.partition(":")
            kind = kind.strip()
            if kind not in cls.KINDS:
                raise ValueError(f"ELFA_FAULT: unknown fault '{kind}' (known: {', '.join(cls.KINDS)})")
            args = {}
            for kv in filter(None, (s.strip() for s in rest.split(","))):
                k, _, v = kv.partition("=")
                args[k.strip()] = float(v)
            faults.append(Fault(kind, args))
        return cls(faults)

    @classmethod
    def from_env(cls) -> "FaultPlan":
        return cls.parse(os.environ.get("ELFA_FAULT", ""))

    def active(self, kind: str, rank: int, step: int) -> Optional[Fault]:
        for f in self.faults:
            if f.kind == kind and f.matches(rank, step):
                return f
        return None

    def __bool__(self) -> bool:
        return bool(self.faults)


class Heartbeat:
    def __init__(self, directory: str, rank: int, world: int):
        self.dir, self.rank, self.world = directory, rank, world
        os.makedirs(directory, exist_ok=True)

    def _path(self, r: int) -> str:
        return os.path.join(self.dir, f"rank_{r}.hb")

    def beat(self, step: int) -> None:
        tmp = self._path(self.rank) + ".tmp"
        with open(tmp, "w") as f:
            f.write(f"{step} {time.time():.3f}\n")
        os.replace(tmp, self._path(self.rank))

    def read(self, r: int):
        try:
            with open(self._path(r)) as f:
                s, t = f.read().split()
            return int(s), float(t)
        except (OSError, ValueError):
            return -1, 0.0

    def stale_peers(self, max_age_s: float) -> List[int]:
        now = time.time()
        return [r for r in range(self.world) if r != self.rank and now - self.read(r)[1] > max_age_s]

    def wait_for_peers(self, step: int, timeout_s: float = 30.0, poll_s: float = 0.01) -> None:
        """Returns when every peer has reported ``step`` (or a later one); raises :class:`RankFailure` otherwise."""
        t0 = time.time()
        while True:
            behind = [r for r in range(self.world) if r != self.rank and self.read(r)[0] < step]
            if not behind:
                return
            if time.time() - t0 > timeout_s:
                raise RankFailure(behind, step, time.time() - t0)
            time.sleep(poll_s)
