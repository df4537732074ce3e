"""Optimizers over flat parameter buffers, LR schedules, clipping and loss scaling."""
from .flat import FlatParams  # noqa: F401
from .optimizers import AdamW, Lion, LionMuon, Muon, build_optimizer  # noqa: F401
from .sched import LRScheduler  # noqa: F401
from .clip import GradientClipper, LossScaler  # noqa: F401
