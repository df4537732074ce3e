"""Read-only GPU health probe through NVML: temperature, clock-throttle reasons, memory, uncorrected ECC errors.

Nothing here changes a setting of the GPU (no clocks, power limits, persistence or compute mode): it only reads.
``probe`` fills the ``gpu_healthy`` / ``memory_healthy`` / ``temperature_ok`` fields of a
:class:`~elfa_b200.telemetry.logger.HealthStatus` and returns the raw readings beside it; the NVML module is a
parameter so that the logic is tested on a CPU machine against a stand-in.

reference: ``src/telemetry/main.zig:122-131,159-197`` (``HealthStatus`` with ``gpu_healthy``, ``memory_healthy``,
``no_nan_inf``, ``temperature_ok`` and ``logHealthCheck``: the record exists, nothing fills it from the device).
"""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

from .logger import HealthStatus

# bits of nvmlDeviceGetCurrentClocksEventReasons that mean "the hardware is protecting itself"
HW_SLOWDOWN = 0x8
SW_THERMAL_SLOWDOWN = 0x20
HW_THERMAL_SLOWDOWN = 0x40
HW_POWER_BRAKE = 0x80
SW_POWER_CAP = 0x4           # normal under a dense GEMM on a power-capped part: reported, not a fault


def probe(index: int = 0, nvml: Any = None, max_temperature_c: int = 90, min_free_fraction: float = 0.02,
          uuid: Optional[str] = None) -> Tuple[HealthStatus, Dict[str, float]]:
    """Health of GPU ``index`` (NVML numbering) or, when ``uuid`` is given and NVML knows it, of that GPU - CUDA's
    device numbers follow ``CUDA_VISIBLE_DEVICES``, NVML's do not. ``nvml`` defaults to ``pynvml``; when it cannot be
    imported or initialised the status is returned with ``gpu_healthy`` left True and an ``"nvml": 0`` reading (no
    information is not a fault)."""
    h = HealthStatus()
    r: Dict[str, float] = {"nvml": 0}
    if nvml is None:
        try:
            import pynvml as nvml  # type: ignore
        except ImportError:
            return h, r
    try:
        nvml.nvmlInit()
    except Exception:
        return h, r
    try:
        dev = None
        if uuid is not None and hasattr(nvml, "nvmlDeviceGetHandleByUUID"):
            for form in (uuid, uuid.encode()):
                try:
                    dev = nvml.nvmlDeviceGetHandleByUUID(form)
                    break
                except Exception:
                    dev = None
        if dev is None:
            dev = nvml.nvmlDeviceGetHandleByIndex(index)
        r["nvml"] = 1
        try:
            r["temperature_c"] = float(nvml.nvmlDeviceGetTemperature(dev, 0))      # 0 = NVML_TEMPERATURE_GPU
        except Exception:
            r["temperature_c"] = 0.0                                                  # this driver has no such reading: no information
        mem = nvml.nvmlDeviceGetMemoryInfo(dev)
        r["memory_used"], r["memory_total"] = float(mem.used), float(mem.total)
        try:
            reasons = int(nvml.nvmlDeviceGetCurrentClocksEventReasons(dev))
        except Exception:
            reasons = int(nvml.nvmlDeviceGetCurrentClocksThrottleReasons(dev))
        r["clock_event_reasons"] = float(reasons)
        try:
            # 1 = uncorrected, 0 = volatile counter (since the last driver load)
            r["ecc_uncorrected"] = float(nvml.nvmlDeviceGetTotalEccErrors(dev, 1, 0))
        except Exception:
            r["ecc_uncorrected"] = 0.0                                                # ECC reporting not available
        h.temperature_ok = r["temperature_c"] <= max_temperature_c and not (reasons & (SW_THERMAL_SLOWDOWN | HW_THERMAL_SLOWDOWN))
        h.memory_healthy = (mem.total - mem.used) >= min_free_fraction * mem.total
        h.gpu_healthy = not (reasons & (HW_SLOWDOWN | HW_POWER_BRAKE)) and r["ecc_uncorrected"] == 0
    except Exception:
        h.gpu_healthy = False           # the device stopped answering NVML
    finally:
        try:
            nvml.nvmlShutdown()
        except Exception:
            pass
    return h, r


def describe(reasons: int) -> str:
    names = [(SW_POWER_CAP, "sw_power_cap"), (HW_SLOWDOWN, "hw_slowdown"), (SW_THERMAL_SLOWDOWN, "sw_thermal_slowdown"),
             (HW_THERMAL_SLOWDOWN, "hw_thermal_slowdown"), (HW_POWER_BRAKE, "hw_power_brake")]
    return ",".join(n for bit, n in names if reasons & bit) or "none"
