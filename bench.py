#!/usr/bin/env python
"""Headline benchmark: training throughput (tokens/s, whole job) of the 7B GPT decoder with
tensor + sequence parallelism over N GPUs and MXFP8 quantisation-aware training
(configs/bench/gpt7b_tp8_mxfp8.yaml: 32 layers, d_model 4096, 32 heads, ffn 11008, vocab 32000,
seq_len 4096, global batch 32 sequences, AdamW, random-init weights, synthetic Zipf(1.1) tokens).

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench.py --gpus 8 --steps 3 --warmup 3

One "step" is one full optimizer step over the global batch (32 x 4096 tokens at every N: strong
scaling). Two timed regions of K steps each, both bracketed by barrier + synchronize and timed with
CUDA events (max over ranks):
  * device-side (`value`): inputs already on the GPU, the loss stays on the GPU;
  * end to end (`e2e`): through Trainer.train_step / finish_step with the step's token ids copied
    from pinned host memory and the loss read back to the host every step.
The working set of a step (tens of GB) is far larger than L2, so no explicit L2 flush is needed.
Prints ONE JSON line on rank 0.

``--config configs/bench/gpt350m_zero1.yaml`` (or ``gpt1p3b_zero3.yaml``, ``gpt13b_tp4dp2_nvfp4.yaml``) runs the
other benchmark configurations with the parallelism their file names: tensor parallel size ``min(file, N)``,
the remaining ranks data parallel with the file's ZeRO stage; pure data-parallel files keep the micro-batch
per GPU fixed (weak scaling).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "tokens/sec/box (max over ranks) 7B TP8 FP8"


class ClockSampler:
    """Samples SM clocks and throttle reasons of this rank's GPU with nvidia-smi while running."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, uuid: str = ""):
        # nvidia-smi numbers GPUs by PCI order, not by CUDA_VISIBLE_DEVICES: address the device by its UUID when known
        self.index, self.uuid, self.rows, self.proc = index, uuid, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.uuid or self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 8:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "gpu_uuid": self.uuid or None}


def reference_arm(args) -> int:
    # The reference (kollarsandor/elfa) is a Zig program with no Python packaging: the offline install
    # the offline `pip install --no-index ... --target baseline/_ref <reference checkout>` stops with "Neither 'setup.py'
    # nor 'pyproject.toml' found", there is no zig toolchain, its build needs a missing tests/unit/main.zig,
    # and 5 of its 11 .cu files do not compile with nvcc 12.9.
    rank = int(os.environ.get("RANK", "0"))
    if rank == 0:
        print(json.dumps({"impl": "reference", "unavailable": "reference is a Zig binary that does not build offline: pip finds no "
                          "setup.py/pyproject.toml, no zig toolchain, build.zig needs a missing tests/unit/main.zig, 5 of 11 .cu "
                          "files fail nvcc 12.9"}))
    return 0


# Loss of the very first step (random-init weights, seeded data, no update yet) measured on one GPU; a run at any N must
# reproduce it: the initial weights and the data do not depend on the parallel layout.
FIRST_STEP_LOSS = {"gpt-7b-tp8-mxfp8": (10.8394, 0.02)}


def self_check(pc, cfg, mb: int, dev) -> dict:
    """Correctness of the fused compute + collective kernels on this job's own ranks and per-rank shapes, outside the timed
    region: each kernel against the library path (NCCL collective + the plain GEMM kernels) on the same inputs. The bound is
    relative: 2^-8 of the largest reference magnitude (one bf16 rounding of the output plus summation-order effects)."""
    import torch
    import torch.distributed as dist
    from elfa_b200.ops.gemm import gemm
    from elfa_b200.ops.gemm_mxfp8 import Mxfp8Operand, gemm_mxfp8, quantize_mxfp8, sf_numel
    from elfa_b200.parallel import fused
    from elfa_b200.parallel import tp as tpl
    world, rank = pc.tp_size, pc.tp_rank
    D, F = cfg.model.hidden_dim, cfg.model.intermediate_dim
    M = mb * cfg.data.seq_len
    Ml = M // world
    g = torch.Generator(device="cpu").manual_seed(4242 + rank)
    res = {}

    def rel(a, b):
        return float((a.float() - b.float()).abs().max()), float(b.float().abs().max()) * 2.0 ** -8

    # all-gather -> GEMM (bf16), MLP-up shape
    x = torch.randn(Ml, D, generator=g).to(torch.bfloat16).to(dev)
    w = (torch.randn(D, F // world, generator=g) * 0.02).to(torch.bfloat16).to(dev)
    saved = pc.comm_backend
    pc.comm_backend = "fused"
    y, xf, _ = tpl.ag_gemm(x, w, pc, b_mn=True)
    pc.comm_backend = "nccl"
    y0, xf0, _ = tpl.ag_gemm(x, w, pc, b_mn=True)
    e, b = rel(y, y0)
    res["ag_gemm"] = {"max_err": e, "bound": b, "gathered_equal": bool(torch.equal(xf, xf0)), "ok": e <= b and bool(torch.equal(xf, xf0))}
    # all-gather -> GEMM (MXFP8, one kernel) against quantise + NCCL all-gather + block-scaled GEMM
    if fused.supported_mxfp8(Ml, D, F // world):
        w_op, _ = quantize_mxfp8(w.t().contiguous(), right=True)
        pc.comm_backend = "fused"
        y, xq_full, _ = fused.ag_gemm_mxfp8(x, w_op, pc)
        fused.wait_pending_copies(pc)
        op, xq = quantize_mxfp8(x, dequantized=True)
        pay = torch.empty(M, D, device=dev, dtype=torch.uint8)
        sf = torch.empty(sf_numel(M, D), device=dev, dtype=torch.uint8)
        dist.all_gather_into_tensor(pay, op.payload, group=pc.tp_group)
        dist.all_gather_into_tensor(sf, op.scales, group=pc.tp_group)
        y0 = gemm_mxfp8(Mxfp8Operand(pay, sf, M, D, False), w_op)
        e, b = rel(y, y0)
        own = bool(torch.equal(xq_full[rank * Ml:(rank + 1) * Ml], xq))
        res["ag_gemm_mxfp8"] = {"max_err": e, "bound": b, "own_rows_equal": own, "ok": e <= b and own}
    # GEMM -> reduce-scatter, MLP-down shape, against an fp32 sum of the ranks' bf16-input products
    a = torch.randn(M, F // world, generator=g).to(torch.bfloat16).to(dev)
    w2 = (torch.randn(F // world, D, generator=g) * 0.02).to(torch.bfloat16).to(dev)
    pc.comm_backend = "fused"
    o = tpl.gemm_rs(a, w2, pc, b_mn=True)
    part = torch.empty(M, D, device=dev, dtype=torch.float32)
    gemm(a, w2, b_mn=True, out=part)
    dist.all_reduce(part, group=pc.tp_group)
    ref = part[rank * Ml:(rank + 1) * Ml]
    e, b = rel(o, ref)
    b *= 2.0      # the partial products travel as bf16: one more rounding per rank
    res["gemm_rs"] = {"max_err": e, "bound": b, "ok": e <= b}
    # the same with block-scaled MXFP8 operands, against the fp32 sum of the products of the dequantised operands
    if fused.supported_rs_mxfp8(M, F // world, D, world):
        from elfa_b200.ops.gemm_mxfp8 import dequantize_mxfp8
        a_op, _ = quantize_mxfp8(a)
        w_op, _ = quantize_mxfp8(w2.t().contiguous(), right=True)
        o = fused.gemm_rs_mxfp8(a_op, w_op, pc)
        gemm(dequantize_mxfp8(a_op), dequantize_mxfp8(w_op), out=part)
        dist.all_reduce(part, group=pc.tp_group)
        e, b = rel(o, part[rank * Ml:(rank + 1) * Ml])
        b *= 2.0
        res["gemm_rs_mxfp8"] = {"max_err": e, "bound": b, "ok": e <= b}
    pc.comm_backend = saved
    ok = torch.tensor([1.0 if all(v["ok"] for v in res.values()) else 0.0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    res["ok"] = bool(ok.item() > 0)
    res["what"] = "fused kernels vs library path on this job's per-rank shapes, every rank, bound = 2^-8 * max|reference|"
    torch.cuda.synchronize()
    return res


def roofline(cfg, tokens_per_s: float, world: int, bf16_peak: float, baseline: bool) -> dict:
    """Per-class roofline of the GPT family: the FLOPs of one token split by the precision they run at, each class against its
    own peak - bf16 against the measured sustained cuBLAS rate, block-scaled e4m3 against twice that (the nominal fp8 : bf16
    ratio; no fp8 peak is measured on the machine). ``fraction`` = time at peak / measured time."""
    m = cfg.model
    D, F, L, V, S = m.hidden_dim, m.intermediate_dim, m.num_layers, m.vocab_size, cfg.data.seq_len
    up = 2 if m.activation == "swiglu" else 1
    lin = 2.0 * L * ((1 + 2 * m.num_kv_heads / m.num_heads) * D * D + D * D + (up + 1) * D * F)   # one pass over the layers' weights
    head = 2.0 * D * V
    attn = 3.0 * L * 2 * S * D                                                      # causal attention, forward + backward
    q_fwd = not baseline and cfg.quant.attention in ("mxfp8", "nvfp4") and cfg.quant.mlp in ("mxfp8", "nvfp4")
    q_bwd = q_fwd and cfg.quant.backward == "mxfp8"
    fp8 = lin * ((1 if q_fwd else 0) + (1 if q_bwd else 0))                          # forward and input-gradient products
    bf16 = 3.0 * lin - fp8 + 3.0 * head + attn                                       # weight gradients, head, attention, the rest
    t_peak = fp8 / (2.0 * bf16_peak) + bf16 / bf16_peak          # seconds per token on one GPU with every class at its peak
    per_gpu = tokens_per_s / world
    return {"flops_per_token": {"block_scaled_e4m3": fp8, "bf16": bf16},
            "peaks_tflops": {"bf16_measured_sustained": bf16_peak / 1e12, "e4m3_nominal_2x": 2.0 * bf16_peak / 1e12},
            "fraction": t_peak * per_gpu}


def plan_run(cfg, yaml_tp: int, yaml_world: int, world: int, micro_batch: int = 0, keep_global_batch: bool = False):
    """Chooses the parallel layout for ``world`` GPUs from the sizes the configuration FILE names (``yaml_tp``,
    ``yaml_world``: read before any launcher variable touches them) and writes it into ``cfg``.
    Returns (micro_batch, scaling, metric)."""
    if yaml_tp == yaml_world:
        # the headline configuration: tensor + sequence parallel over all N GPUs, fixed global batch (strong scaling)
        cfg.runtime.tensor_parallel_size = world
        cfg.runtime.zero_stage = 0
        mb = micro_batch or 4      # 4 sequences of 4096 tokens per micro-batch: 160 GB peak on one GPU, less with tensor parallelism
        scaling = "strong"
        metric = METRIC if cfg.model.name.startswith("gpt-7b") else f"tokens/sec/box (max over ranks) {cfg.model.name}"
    else:
        # the data-parallel configurations (ZeRO stage from the file): tp = min(file's tp, N), the rest is data parallel
        tp = min(yaml_tp, world)
        dp = world // tp
        cfg.runtime.tensor_parallel_size = tp
        if dp == 1:
            cfg.runtime.zero_stage = 0
        mb = micro_batch or cfg.training.micro_batch_size
        if yaml_tp == 1 and not keep_global_batch:      # fixed micro-batch per GPU: weak scaling
            cfg.training.global_batch_size = mb * dp
        scaling = "weak" if yaml_tp == 1 else "strong"
        metric = f"tokens/sec/box (max over ranks) {cfg.model.name}"
    return mb, scaling, metric


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "baseline"],
                    help="ours: this framework; reference: the unmodified reference (unavailable: it does not build); baseline: the "
                         "same model in eager PyTorch with torch.matmul / SDPA / NCCL (baseline/torch_nccl.py), none of this framework's kernels")
    ap.add_argument("--config", default=os.path.join(ROOT, "configs", "bench", "gpt7b_tp8_mxfp8.yaml"))
    ap.add_argument("--micro-batch", type=int, default=0, help="sequences per micro-batch (0 = auto)")
    ap.add_argument("--comm", default=None, choices=[None, "fused", "nccl"])
    ap.add_argument("--twin", type=int, default=0, metavar="N",
                    help="measurement aid, one GPU: play rank 0 of an N-rank job with every collective replaced by a no-op "
                         "(torch's fake process group): the per-rank compute time without communication. Marks the result invalid")
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (marks the result invalid)")
    ap.add_argument("--global-batch", type=int, default=0, help="debug only: override the global batch (marks the result invalid)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import warnings
    warnings.simplefilter("ignore")
    import torch
    import torch.distributed as dist
    from elfa_b200 import native
    from elfa_b200.config import Config
    from elfa_b200.data import Batch
    from elfa_b200.trainer import Trainer, model_flops_per_token

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.twin and (world != 1 or args.gpus != 1):
        print("bench.py: --twin runs as a single process on one GPU", file=sys.stderr)
        return 2
    if world != args.gpus:
        print(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run for N > 1", file=sys.stderr)
        return 2
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    baseline = args.impl == "baseline"
    if not baseline:
        native.lib.load()

    # the file's own world / tensor-parallel sizes choose the branch; the launcher's WORLD_SIZE must not overwrite them first
    cfg = Config.from_file(args.config, env_override=False)
    yaml_tp, yaml_world = cfg.runtime.tensor_parallel_size, cfg.runtime.world_size
    cfg.runtime.rank = int(os.environ.get("RANK", "0"))
    real_world = world
    if args.twin:
        # the job's shapes and call sequence at N ranks, on this one GPU: collectives return at once and move nothing
        from torch.testing._internal.distributed.fake_pg import FakeStore
        dist.init_process_group(backend="fake", store=FakeStore(), rank=0, world_size=args.twin)
        world = args.twin
        args.comm = "nccl"          # the library call sites; the fused kernels need real peers
    cfg.runtime.world_size = world
    if args.comm:
        cfg.runtime.comm_backend = args.comm
    cfg.checkpoint.dir = ""
    cfg.checkpoint.save_interval = 0
    cfg.telemetry.log_file = ""
    if args.layers:
        cfg.model.num_layers = args.layers
    if args.global_batch:
        cfg.training.global_batch_size = args.global_batch
    mb, scaling, metric = plan_run(cfg, yaml_tp, yaml_world, world, args.micro_batch, bool(args.global_batch))
    cfg.training.micro_batch_size = mb
    dp_size = world // cfg.runtime.tensor_parallel_size
    cfg.training.gradient_accumulation_steps = max(1, cfg.training.global_batch_size // (mb * dp_size))
    pc = None
    if args.twin:
        from elfa_b200.parallel.mesh import build_context
        pc = build_context(cfg.runtime.tensor_parallel_size, cfg.runtime.sequence_parallel, "nccl")
    if baseline:
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        from torch_nccl import BaselineTrainer
        from elfa_b200.parallel.mesh import init_distributed
        init_distributed()
        cfg.validate()
        trainer = BaselineTrainer(cfg, torch.device("cuda", local))
        rank = trainer.rank
    else:
        trainer = Trainer(cfg, telemetry=False, pc=pc)
        rank = trainer.pc.rank
    S, G = cfg.data.seq_len, cfg.training.global_batch_size
    n_micro = cfg.training.gradient_accumulation_steps
    tokens_per_step = G * S

    # synthetic Zipf tokens, one global batch per step, staged in pinned host memory
    loader = trainer.make_loader() if baseline else trainer.make_loader("")
    total_steps = args.warmup + 2 * args.steps
    host_steps = []
    for _ in range(min(total_steps, 4)):
        host_steps.append([loader.next_cycling() for _ in range(n_micro)])
    if hasattr(loader, "close"):
        loader.close()              # the prefetch thread is not needed once the steps are staged
    dev = trainer.device
    dev_steps = [[Batch(b.input.to(dev), b.target.to(dev)) for b in st] for st in host_steps[:2]]

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    first_loss = None
    for i in range(args.warmup):
        l = trainer.finish_step(trainer.train_step(host_steps[i % len(host_steps)]))
        if first_loss is None:
            first_loss = l          # before any update: depends on the initial weights and the data only, not on N
    sync_all()
    check = None
    if not baseline and real_world > 1 and not args.twin and cfg.runtime.tensor_parallel_size > 1 and trainer.pc.comm_backend == "fused":
        check = self_check(trainer.pc, cfg, mb, dev)
    st = 0 if baseline else native.status()
    if args.twin:
        st &= ~0x8      # the twin's gathered / reduced buffers hold garbage: the optimizer's non-finite flag means nothing there
    if st:
        print(f"bench.py: device status 0x{st:x} after warm-up", file=sys.stderr)
        return 3

    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(local).uuid)
    except Exception:
        uuid = ""
    sampler = ClockSampler(local, uuid)
    sampler.start()
    # ---- device-side timing
    if not baseline:
        native.lib.raw("elfa_launch_count")(1)
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    last = None
    for i in range(args.steps):
        last = trainer.train_step(dev_steps[i % len(dev_steps)])
    e1.record()
    sync_all()
    launches = 0 if baseline else int(native.lib.raw("elfa_launch_count")(0))
    dev_ms = e0.elapsed_time(e1)
    # ---- end-to-end timing (pinned host inputs, loss read back every step)
    sync_all()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    loss = float("nan")
    for i in range(args.steps):
        loss = trainer.finish_step(trainer.train_step(host_steps[i % len(host_steps)]))
    e3.record()
    sync_all()
    e2e_ms = e2.elapsed_time(e3)
    clocks = sampler.stop()

    t = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = float(t[0]), float(t[1])
    st = 0 if baseline else native.status()
    if rank == 0:
        ms_step = dev_ms / args.steps
        value = tokens_per_step / (ms_step / 1e3)
        e2e_value = tokens_per_step / (e2e_ms / args.steps / 1e3)
        peaks = {}
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peaks = json.load(f)
        except OSError:
            pass
        flops = model_flops_per_token(cfg)
        tpn = cfg.runtime.tensor_parallel_size
        if cfg.quant.attention == "none" and cfg.quant.mlp == "none":
            dtype_note = "bf16 (fp32 master weights / moments / grad accumulation)"
        else:
            bwd = ("input-gradient GEMMs multiply MXFP8-quantised dy and weights (block-scaled on the tensor cores where the fused "
                   "kernels allow, gathered as e4m3 payloads under tensor parallelism), weight-gradient GEMMs bf16 on the dequantised dy"
                   if cfg.quant.backward == "mxfp8" else "backward GEMMs bf16")
            dtype_note = (f"bf16 ({cfg.quant.attention.upper()} / {cfg.quant.mlp.upper()} QAT on the attention / MLP GEMMs: forward GEMMs multiply block-scaled "
                          "payloads on the tensor cores at N = 1; at N > 1 the column-parallel layers all-gather quantised payloads and multiply them block-scaled, "
                          f"the row-parallel GEMM->reduce-scatter kernel multiplies block-scaled MXFP8 payloads too (NVFP4 layers: fake-quantised bf16 operands, the same product); {bwd}; "
                          "fp32 master weights / moments / grad accumulation)")
        parallelism = "single" if world == 1 else "+".join(
            ([f"tp{tpn}+sp"] if tpn > 1 else []) + ([f"dp{dp_size}-zero{cfg.runtime.zero_stage}"] if dp_size > 1 else []))
        peak = peaks.get("bf16_tflops_sustained", 1400.0) * 1e12
        out = {
            "metric": metric, "value": value, "unit": "tokens/s", "n_gpus": real_world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": dtype_note,
            "data": f"synthetic Zipf({cfg.bench.zipf_s}) token ids (seed {cfg.bench.data_seed}), random-init N(0,{cfg.bench.init_std}) weights",
            "config": {"model": cfg.model.name, "layers": cfg.model.num_layers, "d_model": cfg.model.hidden_dim,
                       "heads": cfg.model.num_heads, "ffn": cfg.model.intermediate_dim, "vocab": cfg.model.vocab_size,
                       "global_batch": G, "seq_len": S, "micro_batch": mb, "parallelism": parallelism,
                       "comm_backend": cfg.runtime.comm_backend, "quant": {"attention": cfg.quant.attention, "mlp": cfg.quant.mlp, "backward": cfg.quant.backward},
                       "l2": "per-step working set (tens of GB) exceeds the 126 MB L2; no explicit flush"},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": 2 * G * S * 8, "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": launches,
            "clocks": clocks,
            # the FLOP model covers the GPT family (dense GEMMs + softmax attention) only
            "mfu_of_measured_sustained_bf16": value * flops / (peak * world) if cfg.mixer() == "attention" else None,
            "model_tflops_per_gpu": value * flops / world / 1e12 if cfg.mixer() == "attention" else None,
            "roofline": roofline(cfg, value, world, peak, baseline) if cfg.mixer() == "attention" else None,
            "loss": loss, "loss_first_step": first_loss, "device_status": st,
            "peak_memory_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1),
        }
        if baseline:
            out["impl"] = "baseline"
            out["gpu_launches"] = 0
            out["baseline_note"] = ("eager PyTorch restatement (torch.matmul, scaled_dot_product_attention, torch.nn.functional, fused "
                                    "torch AdamW, NCCL collectives); none of this framework's kernels run")
            out["config"]["comm_backend"] = "nccl (library)"
        if check is not None:
            out["check"] = check
        if first_loss is not None and cfg.model.name in FIRST_STEP_LOSS:
            ref, tol = FIRST_STEP_LOSS[cfg.model.name]
            out["loss_first_step_reference"] = {"n1_value": ref, "tolerance": tol, "ok": abs(first_loss - ref) <= tol}
        if args.layers or args.global_batch:
            out["invalid"] = "layer count or global batch overridden for debugging"
        if args.twin:
            out["twin_of_n_gpus"] = args.twin
            out["invalid"] = (f"communication-free twin of rank 0 of a {args.twin}-GPU job on one GPU (collectives are no-ops, numbers are "
                              "garbage): ms_per_step is the per-rank compute time; exposed communication = measured ms_per_step at N - this")
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if check is not None and not check["ok"]:
        print(f"bench.py: the multi-GPU self-check failed: {check}", file=sys.stderr)
        return 5
    if st & 0x3 and not args.twin:
        print(f"bench.py: device status 0x{st:x}: a bounded device-side wait timed out inside the timed region", file=sys.stderr)
        return 4
    return 0


if __name__ == "__main__":
    sys.exit(main())
