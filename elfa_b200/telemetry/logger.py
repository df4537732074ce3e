"""Rank-0 text log, JSONL metrics, Prometheus exposition and health checks.

JSONL line (reference ``src/telemetry/main.zig:68-97``)::

    {"step":d,"tokens":d,"loss":%.6e,"lr":%.6e,"grad_norm":%.4e,"throughput":%.2f,
     "memory_used":d,"memory_total":d,"timestamp":d}

plus optional extra keys (``mfu``, ``step_ms``, ``loss_scale``, ``skipped``). The human line is
``[ts] step= loss= lr= tokens= throughput=`` (``:99-120``); the last 10 000 steps are kept in memory
(``:71-74``); the Prometheus text has the gauges ``efla_training_step``, ``efla_training_loss``,
``efla_training_throughput`` (``:133-156``) and, unlike the reference, can be served over HTTP when
``telemetry.enable_prometheus`` is set.
"""
from __future__ import annotations

import collections
import json
import math
import os
import sys
import threading
import time
from dataclasses import dataclass, field
from typing import Deque, Dict, Optional

import torch

LEVELS = {"debug": 0, "info": 1, "warn": 2, "err": 3}


@dataclass
class StepMetrics:
    step: int
    tokens: int
    loss: float
    lr: float
    grad_norm: float
    throughput: float
    memory_used: int = 0
    memory_total: int = 0
    timestamp: int = 0
    extra: Dict[str, float] = field(default_factory=dict)

    def to_json(self) -> str:
        base = ('{"step":%d,"tokens":%d,"loss":%.6e,"lr":%.6e,"grad_norm":%.4e,"throughput":%.2f,"memory_used":%d,'
                '"memory_total":%d,"timestamp":%d' % (self.step, self.tokens, self.loss, self.lr, self.grad_norm, self.throughput,
                                                      self.memory_used, self.memory_total, self.timestamp))
        for k, v in self.extra.items():
            base += ',"%s":%s' % (k, json.dumps(v))
        return base + "}"


@dataclass
class HealthStatus:
    gpu_healthy: bool = True
    memory_healthy: bool = True
    no_nan_inf: bool = True
    temperature_ok: bool = True

    def ok(self) -> bool:
        return self.gpu_healthy and self.memory_healthy and self.no_nan_inf and self.temperature_ok


@dataclass
class MemoryStats:
    allocated: int = 0
    freed: int = 0
    current: int = 0
    peak: int = 0

    def alloc(self, n: int) -> None:
        self.allocated += n
        self.current += n
        self.peak = max(self.peak, self.current)

    def free(self, n: int) -> None:
        self.freed += n
        self.current = max(0, self.current - n)


class TrainingStats:
    def __init__(self, window: int = 100):
        self.losses: Deque[float] = collections.deque(maxlen=window)
        self.tokens = 0
        self.t0 = time.time()

    def update(self, loss: float, tokens: int) -> None:
        self.losses.append(loss)
        self.tokens += tokens

    def average_loss(self) -> float:
        return sum(self.losses) / len(self.losses) if self.losses else 0.0

    def tokens_per_second(self) -> float:
        dt = time.time() - self.t0
        return self.tokens / dt if dt > 0 else 0.0


def check_nan_inf(values) -> bool:
    """True when every value is finite (tensor, list or scalar)."""
    if isinstance(values, torch.Tensor):
        return bool(torch.isfinite(values).all())
    try:
        return all(math.isfinite(float(v)) for v in values)
    except TypeError:
        return math.isfinite(float(values))


class Telemetry:
    def __init__(self, cfg=None, rank: int = 0, log_file: Optional[str] = None, log_level: str = "info",
                 enable_prometheus: bool = False, prometheus_port: int = 9090):
        if cfg is not None:
            log_file, log_level = cfg.log_file, cfg.log_level
            enable_prometheus, prometheus_port = cfg.enable_prometheus, cfg.prometheus_port
        self.rank = rank
        self.level = LEVELS.get(log_level, 1)
        self.ring: Deque[StepMetrics] = collections.deque(maxlen=10000)
        self._log = self._jsonl = None
        if rank == 0 and log_file:
            d = os.path.dirname(os.path.abspath(log_file))
            os.makedirs(d, exist_ok=True)
            self._log = open(log_file, "a", encoding="utf-8")
            self._jsonl = open(log_file + ".jsonl", "a", encoding="utf-8")
        self._server = None
        if rank == 0 and enable_prometheus:
            self._serve(prometheus_port)

    # ----------------------------------------------------------------- logging
    def log(self, level: str, scope: str, msg: str) -> None:
        if LEVELS.get(level, 1) < self.level:
            return
        line = "[%d] [%s] %s: %s" % (int(time.time()), level.upper(), scope, msg)
        print(line, file=sys.stderr)
        if self._log is not None:
            self._log.write(line + "\n")
            self._log.flush()

    def log_step(self, m: StepMetrics) -> None:
        if not m.timestamp:
            m.timestamp = int(time.time())
        self.ring.append(m)
        if self._jsonl is not None:
            self._jsonl.write(m.to_json() + "\n")
            self._jsonl.flush()

    def log_metrics(self, m: StepMetrics) -> None:
        self.log_step(m)
        if self.rank == 0:
            line = "[%d] step=%d loss=%.4f lr=%.3e tokens=%d throughput=%.1f" % (m.timestamp, m.step, m.loss, m.lr, m.tokens, m.throughput)
            if self._log is not None:
                self._log.write(line + "\n")
                self._log.flush()
            if self.level <= 1:
                print(line, file=sys.stderr)

    def log_health_check(self, h: HealthStatus) -> None:
        self.log("info" if h.ok() else "err", "health",
                 "gpu=%s memory=%s finite=%s temperature=%s" % (h.gpu_healthy, h.memory_healthy, h.no_nan_inf, h.temperature_ok))

    def health(self, loss: Optional[float] = None, device: Optional[torch.device] = None) -> HealthStatus:
        h = HealthStatus()
        if loss is not None:
            h.no_nan_inf = math.isfinite(loss)
        if device is not None and device.type == "cuda":
            try:
                free, total = torch.cuda.mem_get_info(device)
                h.memory_healthy = free > 0.02 * total
            except RuntimeError:
                h.gpu_healthy = False
            from .health import probe       # temperature, throttle reasons, ECC through NVML (read-only)
            try:
                uuid = "GPU-" + str(torch.cuda.get_device_properties(device).uuid).replace("GPU-", "")
            except (AttributeError, RuntimeError):
                uuid = None
            n, _ = probe(device.index or 0, uuid=uuid)
            h.gpu_healthy = h.gpu_healthy and n.gpu_healthy
            h.temperature_ok = n.temperature_ok
        return h

    # -------------------------------------------------------------- prometheus
    def export_prometheus(self) -> str:
        last = self.ring[-1] if self.ring else StepMetrics(0, 0, 0.0, 0.0, 0.0, 0.0)
        return ("# HELP efla_training_step Current training step\n# TYPE efla_training_step gauge\nefla_training_step %d\n"
                "# HELP efla_training_loss Current training loss\n# TYPE efla_training_loss gauge\nefla_training_loss %.6f\n"
                "# HELP efla_training_throughput Tokens per second\n# TYPE efla_training_throughput gauge\nefla_training_throughput %.2f\n"
                % (last.step, last.loss, last.throughput)) + self._extra_gauges(last)

    @staticmethod
    def _extra_gauges(m: StepMetrics) -> str:
        """Gauges beyond the reference's three: what a dashboard of a long run needs."""
        rows = [("efla_training_tokens", "Tokens consumed", float(m.tokens)), ("efla_training_lr", "Learning rate", m.lr),
                ("efla_training_grad_norm", "Global gradient norm", m.grad_norm),
                ("efla_memory_used_bytes", "Device memory in use", float(m.memory_used))]
        rows += [(f"efla_training_{k}", k.replace("_", " "), float(v)) for k, v in sorted(m.extra.items())]
        return "".join(f"# HELP {n} {h}\n# TYPE {n} gauge\n{n} {v:.6g}\n" for n, h, v in rows)

    def _serve(self, port: int) -> None:
        import http.server

        tel = self

        class H(http.server.BaseHTTPRequestHandler):
            def do_GET(self):       # noqa: N802
                body = tel.export_prometheus().encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/plain; version=0.0.4")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def log_message(self, *a):
                pass

        try:
            self._server = http.server.ThreadingHTTPServer(("127.0.0.1", port), H)
        except OSError as e:
            self.log("warn", "telemetry", f"prometheus endpoint not started: {e}")
            return
        threading.Thread(target=self._server.serve_forever, daemon=True).start()

    def close(self) -> None:
        for f in (self._log, self._jsonl):
            if f is not None:
                f.close()
        self._log = self._jsonl = None
        if self._server is not None:
            self._server.shutdown()
            self._server = None
