from .logger import Telemetry, StepMetrics, HealthStatus, MemoryStats, TrainingStats, check_nan_inf  # noqa: F401
