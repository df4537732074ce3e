"""YAML configuration schema.

Six required top-level maps (``model, training, runtime, data, checkpoint, telemetry``) with the
same keys, types and defaults as the reference trainer's schema
(reference: ``src/util/config.zig:62-123`` model, ``:254-337`` efla/prism, ``:356-463`` training,
``:481-538`` runtime, ``:541-568`` data, ``:590-631`` checkpoint, ``:634-662`` telemetry).

Differences, all deliberate:

* unknown keys and invalid enum strings produce a warning (the reference silently ignores them /
  silently falls back to the default);
* every knob is honoured by the trainer (the reference parses but ignores most of them);
* two optional extension maps, ``bench`` and ``quant``, carry what the reference schema cannot
  express (softmax-attention mixer options, MXFP8/NVFP4 formats, init std, synthetic data);
* ``runtime.rank`` / ``runtime.world_size`` are overridden by the ``RANK`` / ``WORLD_SIZE``
  environment variables when a launcher sets them (one process per GPU).
"""
from __future__ import annotations

import dataclasses
import hashlib
import os
import warnings
from dataclasses import dataclass, field, fields, is_dataclass
from typing import Any, Dict, Optional

import yaml

NORM_TYPES = ("layernorm", "rmsnorm")
ACTIVATIONS = ("relu", "gelu", "silu", "swiglu")
DTYPES = ("fp32", "fp16", "bf16", "fp8", "fp8_e4m3")
BETA_SCHEDULES = ("constant", "linear_warmup", "cosine_decay")
OPTIMIZERS = ("lion", "muon", "lion_muon", "adamw")
LR_SCHEDULES = ("constant", "linear_warmup", "cosine", "linear_warmup_cosine", "linear", "polynomial")
LOG_LEVELS = ("debug", "info", "warn", "err")
QUANT_FORMATS = ("none", "fp8_tensor", "mxfp8", "nvfp4", "int_affine")
SURROGATES = ("straight_through", "sigmoid_tempered", "piecewise_linear")


class ConfigError(ValueError):
    pass


def _enum(choices):
    return {"choices": choices}


@dataclass
class EflaConfig:
    enabled: bool = True
    num_heads: int = 128
    state_dim: int = 128
    chunk_size: int = 4096
    learned_beta: bool = True
    initial_beta: float = 1.0
    beta_schedule: str = field(default="constant", metadata=_enum(BETA_SCHEDULES))
    use_chunked_scan: bool = True


@dataclass
class PrismConfig:
    enabled: bool = True
    num_iterations: int = 3
    shortconv_window: int = 64
    use_proxy: bool = True
    forget_factor: float = 0.99


@dataclass
class ModelConfig:
    name: str = "efla-1t"
    vocab_size: int = 65536
    hidden_dim: int = 16384
    num_layers: int = 80
    num_heads: int = 128
    num_kv_heads: int = 16
    head_dim: int = 128
    intermediate_dim: int = 65536
    max_seq_len: int = 50_000_000
    norm_type: str = field(default="rmsnorm", metadata=_enum(NORM_TYPES))
    activation: str = field(default="gelu", metadata=_enum(ACTIVATIONS))
    tie_embeddings: bool = False
    dropout: float = 0.0
    dtype: str = field(default="bf16", metadata=_enum(DTYPES))
    target_params: int = 1_000_000_000_000
    efla: EflaConfig = field(default_factory=EflaConfig)
    prism: PrismConfig = field(default_factory=PrismConfig)

    def validate(self) -> None:
        for k in ("vocab_size", "hidden_dim", "num_layers", "num_heads", "head_dim", "intermediate_dim"):
            if getattr(self, k) <= 0:
                raise ConfigError(f"model.{k} must be positive")
        if self.hidden_dim % self.num_heads != 0:
            raise ConfigError("model.hidden_dim must be divisible by model.num_heads")
        if self.hidden_dim != self.num_heads * self.head_dim:
            raise ConfigError("model.hidden_dim must equal num_heads * head_dim")
        if self.num_heads % max(self.num_kv_heads, 1) != 0:
            raise ConfigError("model.num_heads must be divisible by model.num_kv_heads")
        if not (0.0 <= self.dropout < 1.0):
            raise ConfigError("model.dropout must be in [0, 1)")

    def estimate_parameters(self) -> int:
        """Closed-form estimate in the reference's shape (``config.zig:174-217``): it counts a Q
        projection and grouped K/V that the EFLA layer does not have, so it differs from the
        exact count of an instantiated model (use ``model.count_parameters()`` for that)."""
        V, D, L, I = self.vocab_size, self.hidden_dim, self.num_layers, self.intermediate_dim
        kv, hd = self.num_kv_heads, self.head_dim
        iters = self.prism.num_iterations if self.prism.enabled else 0
        per_layer = D * (D + 2 * kv * hd) + D * D + iters * 3 * D * hd + 2 * D * I + 2 * D
        emb = V * D + (0 if self.tie_embeddings else V * D)
        return emb + D + L * per_layer


@dataclass
class TrainingConfig:
    total_steps: int = 1_000_000
    warmup_steps: int = 2000
    micro_batch_size: int = 1
    global_batch_size: int = 512
    gradient_accumulation_steps: int = 64
    learning_rate: float = 1e-4
    min_learning_rate: float = 1e-5
    weight_decay: float = 0.1
    gradient_clip: float = 1.0
    label_smoothing: float = 0.0
    optimizer: str = field(default="lion_muon", metadata=_enum(OPTIMIZERS))
    lion_beta1: float = 0.95
    lion_beta2: float = 0.98
    muon_momentum: float = 0.95
    muon_iterations: int = 5
    lr_schedule: str = field(default="cosine", metadata=_enum(LR_SCHEDULES))
    mixed_precision: bool = True
    fp8_training: bool = True
    loss_scale: float = 65536.0
    dynamic_loss_scale: bool = True
    # AdamW extras (the reference hard-codes these inside its kernel call sites).
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95
    adam_eps: float = 1e-8

    def validate(self) -> None:
        if self.micro_batch_size <= 0 or self.global_batch_size <= 0:
            raise ConfigError("batch sizes must be positive")
        if self.global_batch_size % self.micro_batch_size != 0:
            raise ConfigError("training.global_batch_size must be a multiple of micro_batch_size")
        if self.gradient_accumulation_steps <= 0:
            raise ConfigError("training.gradient_accumulation_steps must be positive")
        if self.total_steps <= 0:
            raise ConfigError("training.total_steps must be positive")
        if not (0.0 <= self.label_smoothing < 1.0):
            raise ConfigError("training.label_smoothing must be in [0,1)")


@dataclass
class RuntimeConfig:
    world_size: int = 8
    rank: int = 0
    tensor_parallel_size: int = 8
    pipeline_parallel_size: int = 1
    zero_stage: int = 2
    cpu_offload: bool = False
    nvme_offload: bool = False
    nvme_path: str = "/tmp/offload"
    seed: int = 42
    deterministic: bool = True
    # extension: communication backend for the parallel layers ("fused" = in-kernel peer memory
    # collectives; "nccl" = the unfused library baseline).
    comm_backend: str = field(default="fused", metadata=_enum(("fused", "nccl")))
    sequence_parallel: bool = True
    # extension: ranks of one data-parallel replica that split the sequence dimension of a batch (ring attention)
    context_parallel_size: int = 1
    # "ring": key / value blocks travel round the group (contiguous sequence split); "zigzag": the ring with every rank
    # holding chunks r and 2N-1-r, which evens out the causal work; "ulysses": all-to-all to a head split and back
    context_parallel_mode: str = field(default="ring", metadata=_enum(("ring", "zigzag", "ulysses")))

    def validate(self) -> None:
        if self.world_size <= 0:
            raise ConfigError("runtime.world_size must be positive")
        if self.pipeline_parallel_size != 1:
            raise ConfigError("pipeline parallelism is not supported: runtime.pipeline_parallel_size must be 1")
        if self.tensor_parallel_size <= 0 or self.world_size % self.tensor_parallel_size != 0:
            raise ConfigError("runtime.world_size must be a multiple of tensor_parallel_size")
        if self.zero_stage not in (0, 1, 2, 3):
            raise ConfigError("runtime.zero_stage must be 0..3")
        if self.context_parallel_size <= 0 or self.data_parallel_size % self.context_parallel_size != 0:
            raise ConfigError("runtime.context_parallel_size must divide the data-parallel size")

    @property
    def data_parallel_size(self) -> int:
        return self.world_size // (self.tensor_parallel_size * self.pipeline_parallel_size)


@dataclass
class DataConfig:
    path: str = "data/train.bin"
    tokenizer_path: str = "tokenizer.bin"
    seq_len: int = 8192
    shuffle_buffer_size: int = 10000
    prefetch_factor: int = 2
    num_workers: int = 4
    pack_sequences: bool = True


@dataclass
class CheckpointConfig:
    dir: str = "checkpoints"
    save_interval: int = 1000
    keep_last_n: int = 5
    save_optimizer: bool = True
    compression: bool = True
    async_save: bool = True


@dataclass
class TelemetryConfig:
    log_level: str = field(default="info", metadata=_enum(LOG_LEVELS))
    log_file: str = "training.log"
    metrics_interval: int = 10
    enable_prometheus: bool = False
    prometheus_port: int = 9090
    track_memory: bool = True
    track_throughput: bool = True


@dataclass
class QuantConfig:
    """Extension map ``quant:`` — quantisation-aware-training formats per GEMM group."""
    attention: str = field(default="none", metadata=_enum(QUANT_FORMATS))
    mlp: str = field(default="none", metadata=_enum(QUANT_FORMATS))
    weight_bits: int = 8
    surrogate: str = field(default="straight_through", metadata=_enum(SURROGATES))
    optimizer_state_bits: int = 32
    amax_history: int = 16
    block_scaled_gemm: bool = True   # mxfp8 forward GEMMs on the block-scaled tensor-core path (same values as fake-quant + bf16 GEMM)
    # quantisation of the backward pass: "mxfp8" quantises the output gradient (1x32 blocks along its last dimension) and the
    # weight along the output dimension, so that the input-gradient GEMMs run block-scaled and tensor-parallel layers gather
    # e4m3 payloads of dy; the weight gradient multiplies the dequantised dy in bf16
    backward: str = field(default="none", metadata=_enum(("none", "mxfp8")))


@dataclass
class BenchConfig:
    """Extension map ``bench:`` — things the reference schema has no key for."""
    mixer: str = field(default="auto", metadata=_enum(("auto", "attention", "efla")))
    learned_positions: bool = True
    init_std: float = 0.0            # 0 → reference He-style defaults
    synthetic: str = field(default="none", metadata=_enum(("none", "uniform", "zipf")))
    zipf_s: float = 1.1
    data_seed: int = 0
    mlp_bias: bool = False
    activation_checkpointing: bool = False


@dataclass
class Config:
    model: ModelConfig = field(default_factory=ModelConfig)
    training: TrainingConfig = field(default_factory=TrainingConfig)
    runtime: RuntimeConfig = field(default_factory=RuntimeConfig)
    data: DataConfig = field(default_factory=DataConfig)
    checkpoint: CheckpointConfig = field(default_factory=CheckpointConfig)
    telemetry: TelemetryConfig = field(default_factory=TelemetryConfig)
    quant: QuantConfig = field(default_factory=QuantConfig)
    bench: BenchConfig = field(default_factory=BenchConfig)

    REQUIRED = ("model", "training", "runtime", "data", "checkpoint", "telemetry")

    # ------------------------------------------------------------------ loading
    @classmethod
    def from_dict(cls, raw: Dict[str, Any], *, env_override: bool = True) -> "Config":
        if not isinstance(raw, dict):
            raise ConfigError("top-level YAML node must be a map")
        for sec in cls.REQUIRED:
            if sec not in raw or raw[sec] is None:
                raise ConfigError(f"missing required section '{sec}'")
        known = {f.name for f in fields(cls)}
        for k in raw:
            if k not in known:
                warnings.warn(f"config: unknown top-level section '{k}' ignored")
        cfg = cls()
        for f in fields(cls):
            if f.name in raw and raw[f.name] is not None:
                setattr(cfg, f.name, _fill(getattr(cfg, f.name), raw[f.name], f.name))
        if env_override:
            if "WORLD_SIZE" in os.environ:
                cfg.runtime.world_size = int(os.environ["WORLD_SIZE"])
            if "RANK" in os.environ:
                cfg.runtime.rank = int(os.environ["RANK"])
        return cfg

    @classmethod
    def from_yaml(cls, text: str, **kw) -> "Config":
        return cls.from_dict(yaml.safe_load(text), **kw)

    @classmethod
    def from_file(cls, path: str, **kw) -> "Config":
        with open(path, "r", encoding="utf-8") as fh:
            return cls.from_yaml(fh.read(), **kw)

    # --------------------------------------------------------------- validation
    def validate(self) -> None:
        self.model.validate()
        self.training.validate()
        self.runtime.validate()
        dp = self.runtime.data_parallel_size
        per_step = self.training.micro_batch_size * dp * self.training.gradient_accumulation_steps
        if per_step != self.training.global_batch_size:
            warnings.warn(
                f"config: micro_batch({self.training.micro_batch_size}) x dp({dp}) x accumulation"
                f"({self.training.gradient_accumulation_steps}) = {per_step} != global_batch_size"
                f"({self.training.global_batch_size}); accumulation steps are derived from global_batch_size")
        if self.runtime.tensor_parallel_size > 1:
            tp = self.runtime.tensor_parallel_size
            if self.model.num_heads % tp or self.model.intermediate_dim % tp:
                raise ConfigError("num_heads and intermediate_dim must be divisible by tensor_parallel_size")

    def accumulation_steps(self) -> int:
        dp = self.runtime.data_parallel_size
        return max(1, self.training.global_batch_size // (self.training.micro_batch_size * dp))

    def mixer(self) -> str:
        if self.bench.mixer != "auto":
            return self.bench.mixer
        return "efla" if self.model.efla.enabled else "attention"

    # ----------------------------------------------------------------- analysis
    def estimate_memory_bytes(self, n_gpus: Optional[int] = None) -> int:
        """Per-GPU estimate with the reference's formula (``config.zig:220-230``) but dividing by
        the configured world size instead of a hard-coded 8."""
        n = n_gpus or self.runtime.world_size
        p = self.model.estimate_parameters()
        seq = min(self.data.seq_len, 100_000)
        act = seq * self.model.hidden_dim * self.model.num_layers * 4
        return (p * (2 + 2 + 4) + act) // max(n, 1)

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)

    def to_yaml(self) -> str:
        return yaml.safe_dump(self.to_dict(), sort_keys=False)

    def config_hash(self) -> str:
        """64 lowercase hex chars, stored in checkpoint metadata."""
        return hashlib.sha256(self.to_yaml().encode()).hexdigest()


def _coerce(value: Any, default: Any, path: str) -> Any:
    if isinstance(default, bool):
        if isinstance(value, bool):
            return value
        if isinstance(value, str) and value in ("true", "True", "yes"):
            return True
        if isinstance(value, str) and value in ("false", "False", "no"):
            return False
        raise ConfigError(f"{path}: expected bool, got {value!r}")
    if isinstance(default, int):
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"{path}: expected int, got {value!r}")
        if isinstance(value, float):
            if value != int(value):
                raise ConfigError(f"{path}: expected int, got {value!r}")
            return int(value)
        return value
    if isinstance(default, float):
        if isinstance(value, bool):
            raise ConfigError(f"{path}: expected float, got {value!r}")
        if isinstance(value, (int, float)):
            return float(value)
        if isinstance(value, str):       # PyYAML reads "1e-4" (no dot) as a string
            try:
                return float(value)
            except ValueError:
                pass
        raise ConfigError(f"{path}: expected float, got {value!r}")
    if isinstance(default, str):
        return str(value)
    return value


def _fill(obj: Any, raw: Dict[str, Any], path: str) -> Any:
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: expected a map")
    names = {f.name: f for f in fields(obj)}
    for k, v in raw.items():
        if k not in names:
            warnings.warn(f"config: unknown key '{path}.{k}' ignored")
            continue
        f = names[k]
        cur = getattr(obj, k)
        if is_dataclass(cur):
            if v is not None:
                _fill(cur, v, f"{path}.{k}")
            continue
        if v is None:
            continue
        val = _coerce(v, cur, f"{path}.{k}")
        choices = f.metadata.get("choices") if f.metadata else None
        if choices is not None and val not in choices:
            warnings.warn(f"config: {path}.{k}={val!r} is not one of {choices}; using default {cur!r}")
            continue
        if k == "dtype" and val == "fp8":
            val = "fp8_e4m3"
        setattr(obj, k, val)
    return obj


def default_1t() -> Config:
    """The reference's built-in 1T-parameter default (``config.zig`` ``default1T``)."""
    return Config()
