"""Error taxonomy of the trainer, finite checks, and ``key=value`` override parsing.

Every failure the trainer reports is a :class:`TrainingError` with a stable ``code`` (the reference's error
names, so logs and scripts written against it still match) grouped by area. :func:`check_finite` is the
NaN / Inf test for scalars and tensors: it raises :class:`NotFiniteError` with code ``NaN`` or ``Inf`` and does
its reduction on the device the tensor lives on (one flag pair read back, not the data).
:func:`parse_key_value` splits ``"a=b, c.d=e"`` into a dict (pairs without ``=`` are skipped, whitespace
trimmed), which the CLI uses for ``--set section.key=value`` configuration overrides.

reference: ``src/util/error.zig:4-55`` (``TrainingError`` set), ``:89-117`` (``ErrorContext``), ``:119-129``
(``checkFinite`` / ``checkFiniteSlice``), ``src/util/cli.zig:74-87`` (``parseKeyValue``).
"""
from __future__ import annotations

import inspect
import math
from typing import Any, Dict, Union

import torch

CODES = {
    "config": ("InvalidConfig", "MissingConfig", "MissingConfigPath", "InvalidParameter"),
    "model": ("InvalidHiddenDim", "InvalidNumLayers", "InvalidNumHeads", "InvalidHeadDim", "HiddenDimNotDivisibleByHeads"),
    "training": ("InvalidBatchSize", "InvalidGradientAccumulation", "NaN", "Inf", "GradientOverflow", "LossOverflow"),
    "runtime": ("NoGpuAvailable", "NotEnoughGpus", "InvalidWorldSize", "InvalidRank"),
    "data": ("MissingDataPath", "MissingData", "InvalidData", "IndexOutOfRange"),
    "checkpoint": ("MissingCheckpoint", "MissingCheckpointPath", "InvalidCheckpoint", "InvalidCheckpointFile", "CheckpointCorrupted"),
    "tokenizer": ("MissingCorpus", "MissingTokenizer", "InvalidToken", "InvalidTokenizerFile"),
    "io": ("FileNotFound", "IoError"),
}
_AREA = {code: area for area, codes in CODES.items() for code in codes}


class TrainingError(Exception):
    """``TrainingError("CheckpointCorrupted", "sha256 mismatch in tensor 7")``; ``str()`` gives
    ``file:line: Code: message`` with the location of the ``raise``."""

    def __init__(self, code: str, message: str = ""):
        if code not in _AREA:
            raise ValueError(f"unknown error code {code!r}")
        self.code, self.area, self.message = code, _AREA[code], message
        frame = inspect.stack()[1]
        self.file, self.line = frame.filename, frame.lineno
        super().__init__(f"{self.file}:{self.line}: {code}: {message}")


class NotFiniteError(TrainingError):
    pass


def check_finite(value: Union[float, torch.Tensor], what: str = "value") -> None:
    """Raises ``NotFiniteError("NaN" | "Inf")`` when ``value`` (a number or a tensor of any shape) is not finite.
    NaN wins when both occur."""
    if isinstance(value, torch.Tensor):
        if value.numel() == 0:
            return
        v = value.detach()
        flags = torch.stack((torch.isnan(v).any(), torch.isinf(v).any())).tolist()      # one small read-back
        has_nan, has_inf = bool(flags[0]), bool(flags[1])
    else:
        has_nan, has_inf = math.isnan(value), math.isinf(value)
    if has_nan:
        raise NotFiniteError("NaN", f"{what} contains NaN")
    if has_inf:
        raise NotFiniteError("Inf", f"{what} contains Inf")


def parse_key_value(text: str) -> Dict[str, str]:
    out: Dict[str, str] = {}
    for pair in text.split(","):
        if "=" not in pair:
            continue
        key, value = pair.split("=", 1)
        out[key.strip(" \t")] = value.strip(" \t")
    return out


def _coerce(text: str, like: Any) -> Any:
    if isinstance(like, bool):
        if text.lower() in ("true", "yes", "1", "on"):
            return True
        if text.lower() in ("false", "no", "0", "off"):
            return False
        raise TrainingError("InvalidParameter", f"{text!r} is not a boolean")
    try:
        if isinstance(like, int):
            return int(text, 0)
        if isinstance(like, float):
            return float(text)
    except ValueError:
        raise TrainingError("InvalidParameter", f"{text!r} does not parse as {type(like).__name__}") from None
    return text


def apply_overrides(cfg: Any, overrides: Dict[str, str]) -> None:
    """Sets ``cfg.section[.sub].key`` for every ``"section.key": "text"`` pair, converting the text to the type of the
    field's current value; an unknown path raises ``TrainingError("InvalidParameter")``."""
    for path, text in overrides.items():
        obj = cfg
        parts = path.split(".")
        for name in parts[:-1]:
            if not hasattr(obj, name):
                raise TrainingError("InvalidParameter", f"no configuration section {name!r} in {path!r}")
            obj = getattr(obj, name)
        if not hasattr(obj, parts[-1]):
            raise TrainingError("InvalidParameter", f"no configuration key {path!r}")
        setattr(obj, parts[-1], _coerce(text, getattr(obj, parts[-1])))
