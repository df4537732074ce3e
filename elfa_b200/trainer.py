"""Training engine.

``Trainer`` owns model, flat buffers, optimizer, schedule, loss scaling, checkpoints and telemetry
and honours every knob of the YAML schema (the reference trainer parses but ignores most:
gradient accumulation, loss scale, label smoothing, optimizer / schedule choice, ZeRO / TP sizes;
reference ``src/runtime/trainer.zig:45-136`` init, ``:138-201`` run loop, ``:204-241`` train step,
``:243-270`` smoke test, ``:272-308`` resume, ``:371-403`` save).

One optimizer step = ``accumulation_steps`` micro-batches (forward + backward each, gradients
accumulated in the fp32 flat buffer by the backward kernels) followed by gradient reduction,
clipping and the update. Inputs are copied from pinned host memory on the compute stream; the loss
is read back once per step.
"""
from __future__ import annotations

import os
import time
from typing import Dict, List, Optional

import torch

from .checkpoint import CheckpointManager, CheckpointMetadata
from .config import Config
from .data import Batch, BinaryDataset, DataLoader, SyntheticDataset
from .optim import FlatParams, LossScaler, LRScheduler, build_optimizer
from .parallel import tp as tpl
from .parallel.mesh import ParallelContext, build_context, init_distributed
from .telemetry import StepMetrics, Telemetry


def build_model(cfg: Config, pc: ParallelContext, device):
    if cfg.mixer() == "efla":
        from .models.efla_model import EflaModel
        return EflaModel(cfg, pc, device)
    from .models.gpt import GPTModel
    return GPTModel(cfg, pc, device)


def peak_flops_per_gpu() -> float:
    """The bf16 rate the MFU figure is taken against: ``ELFA_PEAK_TFLOPS`` if set, else the sustained cuBLAS rate measured
    on this machine (``MEASURED_PEAKS.json`` next to the package, written by whoever benchmarked the box), else the
    1.4 PFLOP/s a power-capped B200 sustains. Not the datasheet number."""
    env = os.environ.get("ELFA_PEAK_TFLOPS")
    if env:
        return float(env) * 1e12
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        import json
        with open(path) as f:
            return float(json.load(f)["bf16_tflops_sustained"]) * 1e12
    except (OSError, KeyError, ValueError):
        return 1.4e15


def model_flops_per_token(cfg: Config) -> float:
    """Training FLOPs per token (forward + backward = 3x forward) for the GPT family: dense GEMMs
    (2 FLOPs per weight) plus causal attention (2 * 2 * S * D / 2 per layer)."""
    m = cfg.model
    D, F, L, V, S = m.hidden_dim, m.intermediate_dim, m.num_layers, m.vocab_size, cfg.data.seq_len
    up = 2 if m.activation == "swiglu" else 1
    per_layer = 2 * (4 * D * D + (up + 1) * D * F) + 2 * S * D
    return 3.0 * (L * per_layer + 2 * D * V)


class Trainer:
    def __init__(self, cfg: Config, device: Optional[torch.device] = None, pc: Optional[ParallelContext] = None,
                 telemetry: bool = True):
        cfg.validate()
        self.cfg = cfg
        if pc is None:
            world = init_distributed()
            tp = min(cfg.runtime.tensor_parallel_size, world)
            cp = cfg.runtime.context_parallel_size if world > 1 else 1
            pc = (build_context(tp, cfg.runtime.sequence_parallel, cfg.runtime.comm_backend, cp, cfg.runtime.context_parallel_mode)
                  if world > 1 else ParallelContext())
        self.pc = pc
        if pc.cp_size > 1 and cfg.mixer() != "attention" and pc.cp_mode == "zigzag":
            raise ValueError("the EFLA family splits a sequence into contiguous blocks (state hand-off from rank to rank): "
                             "use runtime.context_parallel_mode ring")
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = device
        torch.manual_seed(cfg.runtime.seed)
        if device.type == "cuda":
            from . import native
            native.set_deterministic(cfg.runtime.deterministic)
        if pc.comm_backend == "fused" and device.type == "cuda" and pc.tp_size > 1 and pc.symm is None:
            from .runtime.symm import SymmetricArena
            pc.symm = SymmetricArena.for_group(pc.tp_group, device)
        self.model = build_model(cfg, pc, device)
        self.model.train()
        if pc.cp_size > 1 and cfg.mixer() == "efla" and pc.comm_backend == "fused" and device.type == "cuda":
            # sequence-parallel EFLA: the ShortConv halo (and its gradient) goes from neighbour to neighbour through
            # peer-memory mailboxes (write-then-flag over NVLink)
            from .parallel import sp
            from .runtime.symm import SymmetricArena
            halo = cfg.training.micro_batch_size * max(cfg.model.prism.shortconv_window - 1, 1) * cfg.model.hidden_dim * 4
            arena_cp = SymmetricArena.for_group(pc.cp_group, device, 4 * halo + (8 << 20))
            sp.register_mailboxes(pc.cp_group, arena_cp, halo)
        dp_arena = None
        blockwise2 = (cfg.runtime.zero_stage == 2 and pc.tp_size == 1 and pc.cp_size == 1 and cfg.training.optimizer in ("adamw", "lion"))
        nvls0 = cfg.runtime.zero_stage == 0 and os.environ.get("ELFA_NVLS", "0") == "1"     # in-switch gradient all-reduce
        if (pc.dp_size > 1 and ((cfg.runtime.zero_stage in (1, 2) and not blockwise2) or nvls0) and pc.comm_backend == "fused"
                and device.type == "cuda" and cfg.model.dtype != "fp32"):
            from .runtime.symm import SymmetricArena
            n_est = sum(p.numel() + 64 for p in self.model.parameters()) + pc.dp_size * 1024
            dp_arena = SymmetricArena.for_group(pc.dp_group, device, n_est * 6 + (16 << 20))
        # stage 3 shards parameters, gradients and optimizer state per block; stage 2 shares its gradient path (reusable
        # per-block gradient slots, reduce-scatter per block next to backward) with resident parameters. Both need pure data
        # parallelism and an element-wise optimizer; otherwise stage 2 keeps the stage-1 mechanism (full gradient buffer)
        blockwise = cfg.runtime.zero_stage == 3 or (cfg.runtime.zero_stage == 2 and pc.tp_size == 1 and pc.cp_size == 1
                                                   and cfg.training.optimizer in ("adamw", "lion"))
        if blockwise and pc.dp_size > 1:
            from .parallel.zero3 import Zero3Shards
            arena3 = None
            if pc.comm_backend == "fused" and device.type == "cuda" and pc.tp_size == 1:
                from .runtime.symm import SymmetricArena
                n_est = sum(p.numel() + 64 for p in self.model.parameters())
                esz = 2 if cfg.model.dtype != "fp32" else 4
                per_block = n_est // max(cfg.model.num_layers, 1) + (1 << 20)
                arena3 = SymmetricArena.for_group(pc.dp_group, device, n_est * esz // pc.dp_size + 3 * per_block * 4 + n_est * 4 // 4 +
                                                     2 * per_block * 2 + n_est * 2 // 4 + (64 << 20))
            # ELFA_ZERO3_PREFETCH=0 (measurement aid): gathers and reduce-scatters run on the compute stream, nothing overlaps
            self.flat = Zero3Shards(self.model, pc, arena=arena3, shard_params=cfg.runtime.zero_stage == 3,
                                    prefetch=os.environ.get("ELFA_ZERO3_PREFETCH", "1") not in ("0", ""))
        else:
            self.flat = FlatParams(self.model.named_checkpoint_parameters(), dp_size=pc.dp_size, dp_rank=pc.dp_rank, allocator=dp_arena)
        self.zero3 = bool(getattr(self.flat, "presharded", False))
        self.optimizer = build_optimizer(cfg, self.flat, pc)
        # runtime.cpu_offload / nvme_offload: optimizer state lives on the host (and NVMe) between steps
        self.offload = None
        if cfg.runtime.cpu_offload or cfg.runtime.nvme_offload:
            from .runtime.offload import OptimizerStateOffload
            nvme = os.path.join(cfg.runtime.nvme_path, f"rank{pc.rank}") if cfg.runtime.nvme_offload else None
            self.offload = OptimizerStateOffload(self._optimizer_state_tensors(), self.device, nvme)
            self.offload.evict()
        t = cfg.training
        self.scheduler = LRScheduler(t.lr_schedule, t.learning_rate, t.min_learning_rate, t.warmup_steps, t.total_steps)
        self.scaler = LossScaler(t.loss_scale if t.mixed_precision else 1.0, t.dynamic_loss_scale and t.mixed_precision)
        self.ckpt = CheckpointManager(cfg.checkpoint.dir, cfg.checkpoint.keep_last_n, cfg.checkpoint.compression,
                                      cfg.checkpoint.async_save) if pc.rank == 0 and cfg.checkpoint.dir else None
        self.telemetry = Telemetry(cfg.telemetry, rank=pc.rank) if telemetry else None
        self.step = 0
        self.epoch = 0
        self.tokens_seen = 0
        self.best_loss = float("inf")
        self.accum = cfg.accumulation_steps()
        self.last_loss = float("nan")
        from .utils.history import LossHistory
        self.history = LossHistory()
        # host-side failure detection / fault injection (both off unless their environment variables are set)
        from .runtime.fault import FaultPlan, Heartbeat
        self.faults = FaultPlan.from_env()
        hb_dir = os.environ.get("ELFA_HEARTBEAT_DIR", "")
        self.heartbeat = Heartbeat(hb_dir, pc.rank, pc.world_size) if hb_dir and pc.world_size > 1 else None
        self.heartbeat_timeout = float(os.environ.get("ELFA_HEARTBEAT_TIMEOUT_S", "30"))
        # phase timer + NVTX ranges (ELFA_TRACE=1); inactive it costs one branch per phase
        from .utils.tracing import PhaseTimer
        self.tracer = PhaseTimer(self.device)
        self._peak = peak_flops_per_gpu()

    # ------------------------------------------------------------------ data
    def make_loader(self, data_path: Optional[str] = None) -> DataLoader:
        cfg, pc = self.cfg, self.pc
        path = data_path if data_path is not None else cfg.data.path
        S, mb = cfg.data.seq_len, cfg.training.micro_batch_size
        if cfg.bench.synthetic != "none" or not path:
            kind = cfg.bench.synthetic if cfg.bench.synthetic != "none" else "uniform"
            need = S * mb * self.accum * (pc.dp_size // pc.cp_size) * 4 + 1
            ds = SyntheticDataset(cfg.model.vocab_size, max(need, S * 64 + 1), kind, cfg.bench.data_seed, cfg.bench.zipf_s)
            shuffle = False
        else:
            ds = BinaryDataset.open(path)
            shuffle = True
        # the ranks of a context-parallel group read the same batch and keep their slice of the sequence
        # data.pack_sequences: rows hold documents back to back, each closed by the tokenizer's <eos>; attention and positions
        # then restart at every document (softmax-attention family without context parallelism; the EFLA family's state
        # runs through the row as in the reference)
        pack_eos = None
        if cfg.data.pack_sequences and cfg.mixer() == "attention" and pc.cp_size == 1:
            from .data.tokenizer import EOS as EOS_ID
            pack_eos = EOS_ID if EOS_ID < cfg.model.vocab_size else None
        loader = DataLoader(ds, mb, S, shuffle=shuffle, seed=cfg.runtime.seed, dp_rank=pc.dp_rank // pc.cp_size,
                            dp_size=pc.dp_size // pc.cp_size, pack_eos=pack_eos)
        depth = cfg.data.prefetch_factor * cfg.data.num_workers
        if depth > 0:       # data.prefetch_factor x data.num_workers batches are assembled ahead on a worker thread
            from .data.dataset import PrefetchLoader
            return PrefetchLoader(loader, depth)
        return loader

    # ------------------------------------------------------------------ step
    def train_step(self, batches: List[Batch]) -> torch.Tensor:
        """One optimizer step over ``batches`` (micro-batches). Returns the mean loss as a device
        scalar (no host synchronisation here)."""
        cfg = self.cfg
        if self.faults:
            f = self.faults.active("kill_rank", self.pc.rank, self.step)
            if f is not None:       # leaves between steps: nothing of this rank is in flight
                raise SystemExit(int(f.args.get("code", 17)))
            f = self.faults.active("delay_ms", self.pc.rank, self.step)
            if f is not None:
                time.sleep(f.args.get("ms", 10.0) / 1e3)
        if self.heartbeat is not None:
            # soft barrier on the host: a peer that died between steps is reported here instead of blocking the next collective
            self.heartbeat.beat(self.step)
            self.heartbeat.wait_for_peers(self.step, self.heartbeat_timeout)
        self.optimizer.zero_grad()
        n_micro = len(batches)
        total = None
        scale = self.scaler.scale
        self.optimizer.loss_scale = scale
        for b in batches:
            ids = b.input.to(self.device, non_blocking=True)
            tgt = b.target.to(self.device, non_blocking=True)
            doc = b.doc_start.to(self.device, non_blocking=True) if getattr(b, "doc_start", None) is not None else None
            pos0 = 0
            if self.pc.cp_size > 1 and self.pc.cp_mode == "zigzag":
                from .parallel.ring_attention import zigzag_slices
                (a0, a1), (b0, b1) = zigzag_slices(ids.shape[1], self.pc.cp_rank, self.pc.cp_size)
                pos0 = (a0, b0)
                ids = torch.cat((ids[:, a0:a1], ids[:, b0:b1]), 1).contiguous()
                tgt = torch.cat((tgt[:, a0:a1], tgt[:, b0:b1]), 1).contiguous()
            elif self.pc.cp_size > 1:
                sl = ids.shape[1] // self.pc.cp_size
                pos0 = self.pc.cp_rank * sl
                ids, tgt = ids[:, pos0:pos0 + sl].contiguous(), tgt[:, pos0:pos0 + sl].contiguous()
            # packed rows mask the targets that would cross a document boundary: average over the tokens that count
            denom = float((int((b.target >= 0).sum()) if doc is not None else tgt.numel()) * n_micro)
            if self.pc.cp_size > 1:
                denom = float(tgt.numel() * n_micro)
            if self.zero3:
                self.flat.before_forward()
            with self.tracer.phase("forward"):
                if self.pc.cp_size > 1 and cfg.mixer() == "efla":
                    # sequence-parallel EFLA: the state and the ShortConv halo cross the ranks inside the model
                    loss = self.model(ids, tgt, pos0=pos0, loss_denominator=denom, grad_scale=scale, sp_group=self.pc.cp_group)
                elif doc is not None:
                    loss = self.model(ids, tgt, pos0=pos0, loss_denominator=denom, grad_scale=scale, doc_start=doc)
                else:
                    loss = self.model(ids, tgt, pos0=pos0, loss_denominator=denom, grad_scale=scale)
            with self.tracer.phase("backward"):
                loss.backward()          # grad_scale is applied inside the loss op's backward
            if self.zero3:
                self.flat.after_backward()
            total = loss.detach() if total is None else total + loss.detach()
        if self.faults and self.faults.active("nan_grad", self.pc.rank, self.step) is not None:
            self.flat.grads[:1].fill_(float("nan"))     # the optimizer's non-finite guard must skip this step
        lr = self.scheduler.get_lr()
        with self.tracer.phase("optimizer"):
            if self.offload is not None:
                self.offload.fetch()
            self.optimizer.step(lr)
            if self.offload is not None:
                if self.device.type != "cuda" and self.ckpt is not None:
                    self.ckpt.wait()        # an asynchronous save may still be reading the state tensors themselves
                self.offload.evict()
        self.scheduler.step()
        self.step += 1
        self.tokens_seen += sum(b.num_tokens for b in batches) * (self.pc.dp_size // self.pc.cp_size)
        return total

    def finish_step(self, loss_dev: torch.Tensor) -> float:
        """Host side of a step: reads the loss, updates the loss scale and health state."""
        loss = float(loss_dev)
        if self.device.type == "cuda":
            # the loss read above has synchronised the stream, so the device status word is current: a bounded wait
            # that ran out (partly gathered / reduced data) or an id outside the vocabulary ends the run here, before the
            # loss scale, the history or a checkpoint see this step
            from .native import check_status
            check_status()
        if self.pc.dp_size > 1:
            import torch.distributed as dist
            t = torch.tensor([loss], device=self.device)
            dist.all_reduce(t, group=self.pc.dp_group)
            loss = float(t) / self.pc.dp_size
        skipped = self.optimizer.skipped() if self.scaler.dynamic else (loss != loss)
        self.scaler.update(bool(skipped))
        self.last_loss = loss
        if loss == loss:
            self.best_loss = min(self.best_loss, loss)
        return loss

    # ------------------------------------------------------------------- run
    def run(self, data_path: Optional[str] = None, max_steps: Optional[int] = None, early_stop_patience: int = 0,
            early_stop_min_delta: float = 0.0) -> List[float]:
        cfg = self.cfg
        loader = self.make_loader(data_path)
        if self.step > 0:
            loader.skip(self.step * self.accum)      # resumed run: continue where the data stream stopped
            self.epoch = loader.epoch
        losses: List[float] = []
        total = cfg.training.total_steps if max_steps is None else min(cfg.training.total_steps, self.step + max_steps)
        t_last, tok_last = time.time(), self.tokens_seen
        while self.step < total:
            batches = []
            for _ in range(self.accum):
                before = loader.epoch
                batches.append(loader.next_cycling())
                if loader.epoch != before:
                    self.epoch = loader.epoch
            loss = self.finish_step(self.train_step(batches))
            losses.append(loss)
            self.history.record(self.step, loss)
            if early_stop_patience > 0 and self.history.should_stop_early(early_stop_patience, early_stop_min_delta):
                break
            if self.telemetry is not None and self.step % max(cfg.telemetry.metrics_interval, 1) == 0:
                now = time.time()
                thr = (self.tokens_seen - tok_last) / max(now - t_last, 1e-9)
                t_last, tok_last = now, self.tokens_seen
                used = total_mem = 0
                if self.device.type == "cuda" and cfg.telemetry.track_memory:
                    free, total_mem = torch.cuda.mem_get_info(self.device)
                    used = total_mem - free
                extra: Dict[str, float] = {"loss_scale": self.scaler.scale}
                if self.device.type == "cuda":
                    extra["mfu"] = thr * model_flops_per_token(cfg) / (self._peak * self.pc.world_size)
                if self.step == 1 or self.step % (50 * max(cfg.telemetry.metrics_interval, 1)) == 0:
                    h = self.telemetry.health(loss, self.device)       # finite loss, free memory, NVML temperature / throttle / ECC
                    if self.step == 1 or not h.ok():
                        self.telemetry.log_health_check(h)
                self.telemetry.log_metrics(StepMetrics(self.step, self.tokens_seen, loss, self.scheduler.get_lr(),
                                                       self.optimizer.grad_norm(), thr if cfg.telemetry.track_throughput else 0.0,
                                                       used, total_mem, int(now), extra))
            si = cfg.checkpoint.save_interval
            if si > 0 and self.step % si == 0:
                self.save_checkpoint()
        if self.ckpt is not None:
            self.ckpt.wait()
        if hasattr(loader, "close"):
            loader.close()          # stops the prefetch thread
        return losses

    def smoke_test(self, steps: int = 3) -> List[float]:
        """A few steps on constant tokens (inputs all 1, targets all 2), like the reference's smoke
        test, but asserting that the loss is finite and decreases."""
        S = min(self.cfg.data.seq_len, 16)
        ids = torch.ones((1, S), dtype=torch.int64)
        tgt = torch.full((1, S), 2, dtype=torch.int64)
        out = []
        for _ in range(steps):
            out.append(self.finish_step(self.train_step([Batch(ids, tgt)])))
        if not all(x == x for x in out):
            raise RuntimeError(f"smoke test produced a non-finite loss: {out}")
        return out

    # ------------------------------------------------------------ checkpoints
    def _gather_logical(self) -> List:
        """(name, full tensor) list on every rank of the TP group (rank 0 writes)."""
        import torch.distributed as dist
        pc = self.pc
        if self.zero3:
            return self.flat.full_tensors()
        out = []
        for name, p in self.model.named_checkpoint_parameters():
            t = p.detach()
            shard = getattr(p, "tp_shard", None)
            if pc.tp_size > 1 and shard is not None:
                parts = [torch.empty_like(t) for _ in range(pc.tp_size)]
                dist.all_gather(parts, t.contiguous(), group=pc.tp_group)
                t = tpl.unshard_param(parts, "vocab" if shard[0] == "vocab" else shard[0])
            out.append((name, t))
        return out

    def _optimizer_state_tensors(self) -> dict:
        opt = self.optimizer
        if hasattr(opt, "muon"):            # Lion + Muon: two moment buffers, one shared master copy
            d = {"muon.m": opt.muon.m, "lion.m": opt.lion.m}
            if not opt.muon.master_is_param:
                d["master"] = opt.muon.master
            return d
        return dict(opt.state_tensors())

    def save_checkpoint(self) -> Optional[str]:
        cfg = self.cfg
        if self.offload is not None:
            self.offload.fetch()
        tensors = self._gather_logical()
        opt_state = None
        if cfg.checkpoint.save_optimizer:
            opt_state = {"optimizer": self.optimizer.state_dict(), "scheduler": self.scheduler.state_dict(),
                         "scaler": self.scaler.state_dict(), "world": (self.pc.dp_size, self.pc.tp_size)}
        if self.offload is not None and self.device.type == "cuda":
            self.offload.evict()            # state_dict made host copies; on a CPU device it returns the tensors themselves
        if self.ckpt is None:
            return None
        meta = CheckpointMetadata(step=self.step, epoch=self.epoch, tokens_seen=self.tokens_seen,
                                  loss=float(self.last_loss if self.last_loss == self.last_loss else 0.0),
                                  learning_rate=float(self.scheduler.get_lr()), timestamp=int(time.time()), git_revision="",
                                  config_hash=cfg.config_hash())
        rng = torch.get_rng_state().numpy().tobytes()
        return self.ckpt.save(self.step, tensors, meta, opt_state, rng, cfg.to_yaml())

    def resume(self, path: str) -> CheckpointMetadata:
        if self.offload is not None:
            self.offload.fetch()
        try:
            return self._resume(path)
        finally:
            if self.offload is not None:
                self.offload.evict()

    def _resume(self, path: str) -> CheckpointMetadata:
        mgr = self.ckpt or CheckpointManager(self.cfg.checkpoint.dir or os.path.dirname(path), 0)
        meta, tensors, opt, rng, _ = mgr.load_full(path)
        pc = self.pc
        if self.zero3:
            self.flat.load_full(tensors)
        with torch.no_grad():
            for name, p in ([] if self.zero3 else self.model.named_checkpoint_parameters()):
                if name not in tensors:
                    raise KeyError(f"checkpoint is missing tensor '{name}'")
                full = tensors[name]
                shard = getattr(p, "tp_shard", None)
                if pc.tp_size > 1 and shard is not None:
                    full = tpl.shard_param(full, shard[0], pc.tp_size, pc.tp_rank)
                if tuple(full.shape) != tuple(p.shape):
                    raise ValueError(f"tensor '{name}': checkpoint shape {tuple(full.shape)} != model shape {tuple(p.shape)}")
                p.copy_(full.to(p.device, p.dtype))
        self.step, self.epoch, self.tokens_seen = meta.step, meta.epoch, meta.tokens_seen
        def _logical(o) -> bool:
            inner = o.get("optimizer", {})
            return inner.get("format") == "logical" or ("muon" in inner and inner["muon"].get("format") == "logical")
        loadable = opt is not None and (_logical(opt) or (tuple(opt.get("world", (1, 1))) == (pc.dp_size, pc.tp_size) and pc.tp_size == 1))
        if loadable:
            # logical (per-parameter) state re-shards itself for this run's data- and tensor-parallel sizes
            self.optimizer.load_state_dict(opt["optimizer"])
            self.scheduler.load_state_dict(opt["scheduler"])
            self.scaler.load_state_dict(opt["scaler"])
        else:
            # no optimizer state (or flat shards of another layout): moments restart from zero, master weights
            # are rebuilt from the loaded parameters, the schedule is reconstructed from the step
            self.scheduler.step_count = meta.step
            opt_obj = getattr(self.optimizer, "muon", self.optimizer)
            if not opt_obj.master_is_param:
                opt_obj.master.copy_(self.flat.flat[opt_obj.lo:opt_obj.hi].float())
        if rng is not None and len(rng) == torch.get_rng_state().numel():
            import numpy as np
            torch.set_rng_state(torch.from_numpy(np.frombuffer(rng, dtype=np.uint8).copy()))
        return meta

    def close(self) -> None:
        if self.offload is not None:
            self.offload.close()
        if self.ckpt is not None:
            self.ckpt.wait()
        if self.telemetry is not None:
            self.telemetry.close()
