"""Worker run by the multi-process tests (one process per rank, launched by torch.distributed.run).

modes:
  fused   - fused ag_gemm / gemm_rs against the library (NCCL) path, repeated calls (GPU)
  tp      - a small GPT trained with TP=world (+sequence parallel) against the same model on one rank
  hybrid  - tensor parallel x data parallel with ZeRO-2 and mixed NVFP4 / MXFP8 QAT against the single-rank result
  cp      - ring attention and a context-parallel GPT against the single-rank result
  timeout - a fused wait that nothing satisfies must return with the timeout status, not hang (GPU)
"""
import os
import sys
import warnings

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
warnings.simplefilter("ignore")

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from elfa_b200.config import Config  # noqa: E402
from elfa_b200.parallel import tp as tpl  # noqa: E402
from elfa_b200.parallel.mesh import build_context, init_distributed  # noqa: E402


def small_cfg(dtype, tp, backend, quant="none", quant_backward=None):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = Config.from_file(os.path.join(root, "configs", "bench", "smoke_cpu.yaml"))
    cfg.model.dtype = dtype
    # the model grows with the tensor-parallel size beyond 4 so that every rank keeps at least one head and 64 hidden columns
    heads = max(4, tp)
    cfg.model.hidden_dim, cfg.model.num_heads, cfg.model.head_dim = 64 * heads, heads, 64
    cfg.model.intermediate_dim = 256 * heads
    cfg.data.seq_len = 256
    cfg.model.max_seq_len = 256
    cfg.training.micro_batch_size, cfg.training.global_batch_size = 2, 2
    cfg.runtime.tensor_parallel_size = tp
    cfg.runtime.comm_backend = backend
    cfg.model.num_kv_heads = int(os.environ.get("ELFA_TEST_KV_HEADS", str(heads)))
    cfg.data.pack_sequences = os.environ.get("ELFA_TEST_PACK", "0") == "1"
    cfg.quant.attention = cfg.quant.mlp = quant
    cfg.quant.backward = quant_backward if quant_backward is not None else os.environ.get("ELFA_TEST_QUANT_BACKWARD", "none")
    cfg.checkpoint.dir = ""
    cfg.checkpoint.save_interval = 0
    cfg.telemetry.log_file = ""
    return cfg


def mode_fused(pc, dev):
    from elfa_b200 import native
    from elfa_b200.runtime.symm import SymmetricArena
    # every shape below keeps its own ring slots, and the gathered / received buffers grow with the number of ranks
    pc.symm = SymmetricArena.for_group(pc.tp_group, dev, (1 << 30) * max(1, pc.tp_size // 2))
    world, rank = pc.tp_size, pc.tp_rank
    torch.manual_seed(1234)
    worst = 0.0
    for it, (Ml, K, N) in enumerate([(128, 256, 512), (256, 512, 1376), (512, 1024, 1536), (256, 512, 1376), (128, 256, 512),
                                     (512, 4096, 1536), (2048, 1024, 2560), (1024, 512, 4096)]):   # the last two: CTA-pair tiles
        g = torch.Generator(device="cpu").manual_seed(100 + it)
        x_all = torch.randn(Ml * world, K, generator=g).to(torch.bfloat16).to(dev)
        w = (torch.randn(K, N, generator=g) * 0.05).to(torch.bfloat16).to(dev)
        x_local = x_all[rank * Ml:(rank + 1) * Ml].contiguous()
        pc.comm_backend = "fused"
        y, x_full, pre = tpl.ag_gemm(x_local, w, pc, b_mn=True, act="gelu", preact=True)
        pc.comm_backend = "nccl"
        y_ref, x_ref, pre_ref = tpl.ag_gemm(x_local, w, pc, b_mn=True, act="gelu", preact=True)
        torch.cuda.synchronize()
        assert torch.equal(x_full, x_ref), "gathered input differs"
        assert torch.equal(x_full, x_all)
        e1 = (y.float() - y_ref.float()).abs().max().item()
        e2 = (pre.float() - pre_ref.float()).abs().max().item()
        # reduce-scatter: every rank holds a K-slice
        a = torch.randn(Ml * world, K, generator=g).to(torch.bfloat16).to(dev)
        w2 = (torch.randn(K, N, generator=g) * 0.05).to(torch.bfloat16).to(dev)
        kl = K // world
        a_l = a[:, rank * kl:(rank + 1) * kl].contiguous()
        w_l = w2[rank * kl:(rank + 1) * kl].contiguous()
        pc.comm_backend = "fused"
        o = tpl.gemm_rs(a_l, w_l, pc, b_mn=True)
        torch.cuda.synchronize()
        ref = (a.double() @ w2.double())[rank * Ml:(rank + 1) * Ml].float()
        e3 = (o.float() - ref).abs().max().item()
        # every rank's partial product travels as bf16 (one rounding each, relative error at most 2^-8: eight significand bits;
        # summed in fp32) and the sum is rounded once more: 2^-8 * (sum over ranks of the largest partial magnitude + the
        # largest reference magnitude), plus a margin for the fp32 accumulation inside the products
        pmax = (a_l.double() @ w_l.double()).abs().max().reshape(1)
        dist.all_reduce(pmax, group=pc.tp_group)
        tol = 1.05 * 2.0 ** -8 * (pmax.item() + ref.abs().max().item())
        assert e1 == 0.0 and e2 == 0.0, f"ag_gemm differs from the library path: {e1} {e2}"
        assert e3 < tol, f"gemm_rs error {e3} > {tol}"
        worst = max(worst, e3)
    # quantise-before-send all-gather -> block-scaled GEMM: bit-identical to the one-GPU path on the whole input
    from elfa_b200.ops.gemm_mxfp8 import gemm_mxfp8, quantize_mxfp8
    from elfa_b200.parallel import fused
    pc.comm_backend = "fused"
    for it, (Ml, K, N) in enumerate([(128, 256, 512), (256, 512, 1376), (512, 4096, 1536), (128, 256, 512), (1024, 1024, 2048),
                                     (256, 512, 1376), (2048, 4096, 1536), (128, 128, 64)]):   # CTA pairs with several tiles each; one narrow tile
        g = torch.Generator(device="cpu").manual_seed(300 + it)
        x_all = torch.randn(Ml * world, K, generator=g).to(torch.bfloat16).to(dev)
        w = (torch.randn(K, N, generator=g) * 0.05).to(torch.bfloat16).to(dev)
        w_op, _ = quantize_mxfp8(w.t().contiguous(), right=True)
        x_local = x_all[rank * Ml:(rank + 1) * Ml].contiguous()
        assert fused.supported_mxfp8(Ml, K, N)
        y, x_full, pre = fused.ag_gemm_mxfp8(x_local, w_op, pc, act="gelu", preact=True)
        fused.wait_pending_copies(pc)
        xa_op, xq_all = quantize_mxfp8(x_all, dequantized=True)
        pre_ref = torch.empty_like(pre)
        y_ref = gemm_mxfp8(xa_op, w_op, gelu=True, preact=pre_ref)
        torch.cuda.synchronize()
        assert torch.equal(x_full, xq_all), f"gathered quantised rows differ ({Ml}, {K}, {N})"
        assert torch.equal(y, y_ref) and torch.equal(pre, pre_ref), f"quantised all-gather GEMM differs ({Ml}, {K}, {N})"
    # block-scaled GEMM -> reduce-scatter: every rank holds a K-slice of both operands, quantised along K
    from elfa_b200.ops.gemm_mxfp8 import dequantize_mxfp8
    for it, (Ml, Kl, N) in enumerate([(128, 128, 256), (256, 512, 4096), (1024, 1376, 4096), (128, 96, 192), (2048, 512, 4096)]):
        g = torch.Generator(device="cpu").manual_seed(500 + it * 8 + rank)
        a = torch.randn(Ml * world, Kl, generator=g).to(torch.bfloat16).to(dev)
        w = (torch.randn(N, Kl, generator=g) * 0.05).to(torch.bfloat16).to(dev)
        a_op, _ = quantize_mxfp8(a)
        w_op, _ = quantize_mxfp8(w, right=True)
        assert fused.supported_rs_mxfp8(Ml * world, Kl, N, world)
        o = fused.gemm_rs_mxfp8(a_op, w_op, pc)
        part = dequantize_mxfp8(a_op).double() @ dequantize_mxfp8(w_op).double().t()
        pmax = part.abs().max().reshape(1)
        dist.all_reduce(pmax, group=pc.tp_group)
        dist.all_reduce(part, group=pc.tp_group)
        ref = part[rank * Ml:(rank + 1) * Ml].float()
        torch.cuda.synchronize()
        e = (o.float() - ref).abs().max().item()
        bound = 1.05 * 2.0 ** -8 * (pmax.item() + ref.abs().max().item())      # one bf16 rounding per partial, one of the sum
        assert e <= bound, f"block-scaled gemm_rs ({Ml}, {Kl}, {N}): {e} vs bound {bound}"
    st = native.status()
    assert st == 0, f"device status 0x{st:x}"
    dist.barrier()
    bad = pc.symm.check_canaries()          # nobody (this rank or a peer) wrote past the end of a ring slot or a flag region
    assert not bad, f"guard words overwritten behind {bad}"
    dist.barrier()
    if rank == 0:
        print(f"FUSED_OK worst_rs_err={worst:.4f}")


def mode_tp(pc, dev, backend, dtype):
    from elfa_b200.parallel.mesh import ParallelContext
    from elfa_b200.trainer import Trainer
    world = pc.tp_size
    quant = os.environ.get("ELFA_TEST_QUANT", "none")      # "mxfp8": the quantised all-gather path of the fused backend
    cfg = small_cfg(dtype, world, backend, quant)
    tr = Trainer(cfg, device=dev, pc=pc, telemetry=False)
    losses = tr.run(max_steps=4)
    ref = None
    if pc.rank == 0:
        cfg1 = small_cfg(dtype, 1, "nccl", quant)
        cfg1.runtime.world_size = 1
        tr1 = Trainer(cfg1, device=dev, pc=ParallelContext(), telemetry=False)
        ref = tr1.run(max_steps=4)
        tol = 2e-4 if dtype == "fp32" else 0.05
        for a, b in zip(losses, ref):
            assert abs(a - b) < tol * max(1.0, abs(b)), f"TP losses {losses} differ from single-rank {ref}"
        print(f"TP_OK backend={backend} losses={[round(x, 4) for x in losses]} ref={[round(x, 4) for x in ref]}")
    dist.barrier()


def mode_cp(dev, dtype, tp, cp_mode="ring"):
    """Ring attention against attention over the whole sequence (forward and gradients), then a small GPT
    trained with the sequence split over a context-parallel group against the same model on one rank."""
    from elfa_b200.ops.attention import attention_ref
    from elfa_b200.parallel.mesh import ParallelContext
    from elfa_b200.parallel.ring_attention import ring_attention, zigzag_slices
    from elfa_b200.parallel.ulysses import ulysses_attention
    from elfa_b200.trainer import Trainer
    world, rank = dist.get_world_size(), dist.get_rank()
    cp = world // tp
    pc = build_context(tp, True, "nccl", cp_size=cp, cp_mode=cp_mode)
    assert pc.cp_size == cp and len(pc.cp_ranks) == cp
    tdt = torch.float32 if dtype == "fp32" else torch.bfloat16
    g = torch.Generator().manual_seed(5)
    S, B, H, hd = 256 * cp, 2, 2, 64
    full = torch.randn(S, B, 3, H, hd, generator=g).to(dev, tdt)
    dout = torch.randn(S, B, H * hd, generator=g).to(dev, tdt)
    sl, c = S // cp, pc.cp_rank
    for causal in (True, False):
        ref_in = full.float().clone().requires_grad_(True)
        ref = attention_ref(ref_in, causal=causal)
        ref.backward(dout.float())
        if cp_mode == "zigzag":
            if not causal:
                continue
            (a0, a1), (b0, b1) = zigzag_slices(S, c, cp)
            take = lambda t: torch.cat((t[a0:a1], t[b0:b1]), 0)
        else:
            take = lambda t: t[c * sl:(c + 1) * sl]
        loc = take(full).clone().requires_grad_(True)
        if cp_mode == "ulysses":
            out = ulysses_attention(loc, pc.cp_group, causal=causal)
        else:
            out = ring_attention(loc, pc.cp_group, causal=causal, zigzag=cp_mode == "zigzag")
        out.backward(take(dout).contiguous())
        tol = 1e-4 if dtype == "fp32" else 3e-2
        tol_g = tol * (1.0 + max(1.0, ref_in.grad.abs().max().item()))
        e_o = (out.float() - take(ref)).abs().max().item()
        e_g = (loc.grad.float() - take(ref_in.grad)).abs().max().item()
        assert e_o < tol and e_g < tol_g, f"ring attention causal={causal}: out err {e_o}, grad err {e_g}"
    seq = 256 * cp                   # every block product gets at least one full 128-row tile, also under the zig-zag split
    cfg = small_cfg(dtype, tp, "nccl")
    cfg.data.seq_len = cfg.model.max_seq_len = seq
    cfg.runtime.world_size = world
    cfg.runtime.context_parallel_size = cp
    cfg.runtime.context_parallel_mode = cp_mode
    cfg.runtime.zero_stage = 1
    tr = Trainer(cfg, device=dev, pc=pc, telemetry=False)
    losses = tr.run(max_steps=4)
    if rank == 0:
        cfg1 = small_cfg(dtype, 1, "nccl")
        cfg1.data.seq_len = cfg1.model.max_seq_len = seq
        cfg1.runtime.world_size = 1
        ref_l = Trainer(cfg1, device=dev, pc=ParallelContext(), telemetry=False).run(max_steps=4)
        tol = 2e-4 if dtype == "fp32" else 0.05
        for a, b in zip(losses, ref_l):
            assert abs(a - b) < tol * max(1.0, abs(b)), f"context-parallel losses {losses} differ from single-rank {ref_l}"
        print(f"CP_OK mode={cp_mode} cp={cp} tp={tp} losses={[round(x, 4) for x in losses]} ref={[round(x, 4) for x in ref_l]}")
    dist.barrier()


def mode_zero(dev, backend, dtype, stage):
    """Data parallel with ZeRO sharding (dp = world, tp = 1) against one rank on the global batch."""
    from elfa_b200 import native
    from elfa_b200.parallel.mesh import ParallelContext
    from elfa_b200.trainer import Trainer
    pc = build_context(1, False, backend)
    world = pc.dp_size
    cfg = small_cfg(dtype, 1, backend)
    cfg.runtime.zero_stage = stage
    accum = 2 if stage >= 2 else 1            # stages 2 and 3 also cover gradient accumulation over micro-batches
    cfg.training.micro_batch_size = 2
    cfg.training.global_batch_size = 2 * world * accum
    tr = Trainer(cfg, device=dev, pc=pc, telemetry=False)
    losses = tr.run(max_steps=4)
    if dev.type == "cuda":
        assert native.status() == 0
    if stage == 2:
        # real gradient sharding: no full-size fp32 gradient buffer, two reusable block slots + the shard instead; parameters whole
        rep = tr.flat.memory_report()
        nb = len(tr.flat.block_buckets)
        assert tr.zero3 and not tr.flat.shard_params and rep["param_bytes_at_rest"] >= rep["param_bytes_unsharded"], rep
        if nb >= 4:
            assert rep["grad_bytes"] < rep["grad_bytes_unsharded"], rep
        assert tr.flat.reduce_scatters == 4 * (accum * nb + 1), tr.flat.reduce_scatters
    if stage == 3:
        rep = tr.flat.memory_report()
        assert tr.zero3 and rep["param_bytes_at_rest"] * world <= rep["param_bytes_unsharded"] + 4096 * world, rep
        nb = len(tr.flat.block_buckets)
        if tr.flat.gather_in_gemm:
            # forward: the four products of a block fetch their matrices themselves; backward gathers whole blocks
            assert tr.flat.gemm_gathers == 4 * accum * nb * 4, (tr.flat.gemm_gathers, nb)
            assert tr.flat.gathers == 4 * (accum * nb + 1), (tr.flat.gathers, nb)
        else:
            # per micro-batch: every block gathered for forward and for backward; the rest once per step
            assert tr.flat.gathers == 4 * (accum * 2 * nb + 1), (tr.flat.gathers, nb)
        assert tr.flat.reduce_scatters == 4 * (accum * nb + 1), tr.flat.reduce_scatters
    if pc.rank == 0:
        cfg1 = small_cfg(dtype, 1, "nccl")
        cfg1.runtime.world_size = 1
        cfg1.runtime.zero_stage = 0
        cfg1.training.micro_batch_size = 2 * world * accum
        cfg1.training.global_batch_size = 2 * world * accum
        tr1 = Trainer(cfg1, device=dev, pc=ParallelContext(), telemetry=False)
        ref = tr1.run(max_steps=4)
        tol = 2e-4 if dtype == "fp32" else 0.05
        for a, b in zip(losses, ref):
            assert abs(a - b) < tol * max(1.0, abs(b)), f"ZeRO losses {losses} differ from single-rank {ref}"
        print(f"ZERO_OK stage={stage} backend={backend} fused={tr.optimizer.zero_fused is not None} "
              f"peer_kernels={getattr(tr.flat, 'arena', None) is not None} gather_in_gemm={getattr(tr.flat, 'gather_in_gemm', False)} nvls={getattr(tr.optimizer, 'nvls', None) is not None} "
              f"losses={[round(x, 4) for x in losses]} ref={[round(x, 4) for x in ref]}")
    dist.barrier()


def mode_hybrid(dev, backend, dtype, tp):
    """The layout of the 13B benchmark configuration in small: tensor parallel groups of ``tp`` ranks x data parallel
    with ZeRO-2, NVFP4 QAT on the MLP GEMMs and MXFP8 on the attention GEMMs, against one rank on the global batch."""
    from elfa_b200.parallel.mesh import ParallelContext
    from elfa_b200.trainer import Trainer
    pc = build_context(tp, True, backend)
    assert pc.tp_size == tp and pc.dp_size == dist.get_world_size() // tp
    assert pc.tp_ranks == [pc.dp_rank * tp + t for t in range(tp)]          # tensor-parallel ranks are neighbours
    cfg = small_cfg(dtype, tp, backend)
    cfg.runtime.world_size = dist.get_world_size()
    cfg.runtime.zero_stage = 2
    cfg.quant.attention, cfg.quant.mlp = "mxfp8", "nvfp4"
    cfg.training.micro_batch_size = 2
    cfg.training.global_batch_size = 2 * pc.dp_size
    tr = Trainer(cfg, device=dev, pc=pc, telemetry=False)
    losses = tr.run(max_steps=4)
    if pc.rank == 0:
        cfg1 = small_cfg(dtype, 1, "nccl")
        cfg1.runtime.world_size = 1
        cfg1.runtime.zero_stage = 0
        cfg1.quant.attention, cfg1.quant.mlp = "mxfp8", "nvfp4"
        cfg1.training.micro_batch_size = cfg1.training.global_batch_size = 2 * pc.dp_size
        ref = Trainer(cfg1, device=dev, pc=ParallelContext(), telemetry=False).run(max_steps=4)
        tol = 2e-3 if dtype == "fp32" else 0.05
        for a, b in zip(losses, ref):
            assert abs(a - b) < tol * max(1.0, abs(b)), f"hybrid losses {losses} differ from single-rank {ref}"
        print(f"HYBRID_OK tp={tp} dp={pc.dp_size} losses={[round(x, 4) for x in losses]} ref={[round(x, 4) for x in ref]}")
    dist.barrier()


def mode_ckpt(dev, stage, ckpt_dir, tp=1, dtype="fp32", resume_tp=None):
    """Sharded optimizer state survives a checkpoint: train 2 + save + 2 more == resume + 2, for data-parallel shards,
    tensor-parallel slices, and a resume under another (tp, dp) split of the same ranks."""
    from elfa_b200.trainer import Trainer
    world = dist.get_world_size()
    resume_tp = tp if resume_tp is None else resume_tp

    def make(tp_):
        pc = build_context(tp_, tp_ > 1, "nccl")
        cfg = small_cfg(dtype, tp_, "nccl")
        cfg.runtime.world_size = world
        cfg.runtime.zero_stage = stage if pc.dp_size > 1 else 0
        cfg.training.micro_batch_size = 2 if tp_ == tp else 2 * (world // tp) // pc.dp_size
        cfg.training.global_batch_size = 2 * (world // tp)
        cfg.checkpoint.dir = ckpt_dir
        cfg.checkpoint.save_optimizer = True
        cfg.checkpoint.async_save = False
        return Trainer(cfg, device=dev, pc=pc, telemetry=False), pc
    tr, pc = make(tp)
    tr.run(max_steps=2)
    path = tr.save_checkpoint()
    dist.barrier()
    paths = [path]
    dist.broadcast_object_list(paths, src=0)
    cont = tr.run(max_steps=2)
    tr2, pc2 = make(resume_tp)
    tr2.resume(paths[0])
    again = tr2.run(max_steps=2)
    tol = (1e-5 if resume_tp == tp else 2e-4) if dtype == "fp32" else 2e-2
    for a, b in zip(cont, again):
        assert abs(a - b) < tol * max(1.0, abs(a)), f"resume diverges: {cont} vs {again}"
    if resume_tp == tp:
        # the restored state itself: moments and master weights equal the saved ones on every rank
        sd1 = tr.optimizer.state_dict()
        sd2 = tr2.optimizer.state_dict()
        for k in sd1["tensors"]:
            for n in sd1["tensors"][k]:
                d = (sd1["tensors"][k][n].float() - sd2["tensors"][k][n].float()).abs().max().item()
                assert d < (1e-5 if dtype == "fp32" else 2e-2), f"optimizer state {k}/{n} differs by {d} after resume"
    if dist.get_rank() == 0:
        print(f"CKPT_OK stage={stage} tp={tp}->{resume_tp} {dtype} cont={[round(x, 5) for x in cont]} again={[round(x, 5) for x in again]}")
    dist.barrier()


def mode_baseline(dev, dtype, tp, stage):
    """The eager-PyTorch baseline arm under tensor x data parallelism against the product arm on one rank."""
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline"))
    from torch_nccl import BaselineTrainer
    from elfa_b200.parallel.mesh import ParallelContext
    from elfa_b200.trainer import Trainer
    world = dist.get_world_size()
    dp = world // tp
    cfg = small_cfg(dtype, tp, "nccl", "mxfp8", "mxfp8")
    cfg.runtime.world_size = world
    cfg.runtime.zero_stage = stage
    cfg.training.micro_batch_size, cfg.training.global_batch_size = 2, 2 * dp
    tr = BaselineTrainer(cfg, dev)
    loader = tr.make_loader()
    losses = [tr.finish_step(tr.train_step([loader.next_cycling() for _ in range(tr.accum)])) for _ in range(4)]
    if dist.get_rank() == 0:
        cfg1 = small_cfg(dtype, 1, "nccl", "mxfp8", "mxfp8")
        cfg1.runtime.world_size = 1
        cfg1.runtime.zero_stage = 0
        cfg1.training.micro_batch_size = cfg1.training.global_batch_size = 2 * dp
        ref = Trainer(cfg1, device=dev, pc=ParallelContext(), telemetry=False).run(max_steps=4)
        tol = 2e-3 if dtype == "fp32" else 0.05
        for a, b in zip(losses, ref):
            assert abs(a - b) < tol * max(1.0, abs(b)), f"baseline arm {losses} differs from the product arm {ref}"
        print(f"BASELINE_OK tp={tp} dp={dp} stage={stage} losses={[round(x, 4) for x in losses]} ref={[round(x, 4) for x in ref]}")
    dist.barrier()


def mode_efla_tp(dev, dtype, tp, cp=1):
    """The EFLA + PRISM family under tensor parallelism (heads, MLP columns and vocabulary sharded; norms, PRISM and the
    ShortConv replicated) x data parallelism against one rank on the global batch."""
    from elfa_b200.parallel.mesh import ParallelContext
    from elfa_b200.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    world = dist.get_world_size()
    pc = build_context(tp, True, "nccl", cp)
    replicas = world // tp // cp          # ranks of a context-parallel group share a batch and split its sequences

    def cfg_for(tp_, world_, opt):
        cfg = Config.from_file(os.path.join(root, "configs", "smoke.yaml"))
        cfg.model.dtype = dtype
        cfg.model.num_layers = 2
        cfg.runtime.tensor_parallel_size, cfg.runtime.world_size = tp_, world_
        cfg.runtime.context_parallel_size = cp if world_ > 1 else 1
        cfg.training.optimizer = opt
        cfg.training.learning_rate = 1e-3
        cfg.training.micro_batch_size = 2 if world_ > 1 else 2 * replicas
        cfg.training.global_batch_size = 2 * replicas
        cfg.data.path = ""
        cfg.checkpoint.dir = ""
        cfg.checkpoint.save_interval = 0
        cfg.telemetry.log_file = ""
        return cfg
    losses = Trainer(cfg_for(tp, world, "lion"), device=dev, pc=pc, telemetry=False).run(max_steps=4)
    muon = Trainer(cfg_for(tp, world, "lion_muon"), device=dev, pc=pc, telemetry=False).run(max_steps=2)   # shard-wise Newton-Schulz: runs, not compared
    assert all(x == x for x in muon)
    if dist.get_rank() == 0:
        ref = Trainer(cfg_for(1, 1, "lion"), device=dev, pc=ParallelContext(), telemetry=False).run(max_steps=4)
        tol = 2e-3 if dtype == "fp32" else 0.05
        for a, b in zip(losses, ref):
            assert abs(a - b) < tol * max(1.0, abs(b)), f"EFLA TP losses {losses} differ from single-rank {ref}"
        print(f"EFLA_TP_OK tp={tp} cp={cp} dp={world // tp} losses={[round(x, 4) for x in losses]} ref={[round(x, 4) for x in ref]}")
    dist.barrier()


def mode_multimem(pc, dev):
    """In-switch collectives (multimem.ld_reduce / multimem.st) against the library's, fp32 and bf16."""
    from elfa_b200 import native
    from elfa_b200.parallel.nvls import MultimemGroup
    from elfa_b200.runtime.symm import SymmetricArena
    arena = SymmetricArena.for_group(pc.tp_group, dev, 256 << 20)
    world, rank = arena.world, arena.rank
    if not arena.multicast_ptr:
        if rank == 0:
            print("MULTIMEM_SKIPPED no multicast mapping on this machine")
        dist.barrier()
        return
    mm = MultimemGroup(arena)
    n = world * 1024 * 257
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        esz = 4 if dtype == torch.float32 else 2
        reg = arena.alloc(n * esz, f"mm.test.{esz}")
        x = reg.view(dtype, (n,))
        g = torch.Generator(device="cpu").manual_seed(7 + rank)
        mine = torch.randn(n, generator=g).to(dtype).to(dev)
        ref = mine.float().clone()
        dist.all_reduce(ref, group=pc.tp_group)
        for _ in range(2):      # twice: the barrier words are counted, not reset
            x.copy_(mine)
            mm.all_reduce_(reg, n, dtype, 0.5)
            torch.cuda.synchronize()
            e = (x.float() - 0.5 * ref).abs().max().item()
            assert e <= tol * ref.abs().max().item(), f"multimem all-reduce {dtype}: {e}"
        x.copy_(mine)
        out = torch.empty(n // world, dtype=dtype, device=dev)
        mm.reduce_scatter(reg, n, out, dtype)
        torch.cuda.synchronize()
        per = n // world
        e = (out.float() - ref[rank * per:(rank + 1) * per]).abs().max().item()
        assert e <= tol * ref.abs().max().item(), f"multimem reduce-scatter {dtype}: {e}"
        x.copy_(mine)
        mm.all_gather_(reg, n, dtype)
        torch.cuda.synchronize()
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine, group=pc.tp_group)
        want = torch.cat([parts[r][r * per:(r + 1) * per] for r in range(world)])
        assert torch.equal(x, want), f"multimem all-gather {dtype}"
    assert native.status() == 0
    dist.barrier()
    assert not arena.check_canaries()
    dist.barrier()
    if rank == 0:
        print("MULTIMEM_OK")


def mode_mailbox(pc, dev):
    """Ring hand-off through peer mailboxes: several rounds, payload checked against the sender's rank."""
    from elfa_b200 import native
    from elfa_b200.parallel.sp import PeerMailbox, ring_exchange_peer
    from elfa_b200.runtime.symm import SymmetricArena
    arena = SymmetricArena.for_group(pc.tp_group, dev, 64 << 20)
    box = PeerMailbox(arena, 1 << 20)
    r, w = pc.rank, pc.tp_size
    for rnd in range(6):
        x = torch.full((4096,), float(r * 100 + rnd), device=dev, dtype=torch.float32)
        got = ring_exchange_peer(x, box)
        torch.cuda.synchronize()
        assert native.status() == 0
        want = float(((r - 1) % w) * 100 + rnd)
        assert bool((got == want).all()), (r, rnd, float(got[0]), want)
    # the registered route: ring_exchange in both directions (what the differentiable halo exchange uses)
    from elfa_b200.parallel import sp
    sp.register_mailboxes(pc.tp_group, arena, 1 << 20)
    for rnd in range(3):
        for step in (1, -1):
            x = torch.full((2, 15, 64), float(r * 10 + rnd), device=dev, dtype=torch.bfloat16)
            got = sp.ring_exchange(x, step, pc.tp_group)
            torch.cuda.synchronize()
            assert bool((got == float(((r - step) % w) * 10 + rnd)).all()), (r, rnd, step)
    assert native.status() == 0 and not arena.check_canaries()
    dist.barrier()
    if r == 0:
        print("MAILBOX_OK")


def mode_killrank(dev):
    """A rank leaves between steps; the survivors notice through the heartbeat files before their next collective."""
    from elfa_b200.runtime.fault import RankFailure
    from elfa_b200.trainer import Trainer
    pc = build_context(1, False, "nccl")
    cfg = small_cfg("fp32", 1, "nccl")
    cfg.runtime.zero_stage = 0
    cfg.training.micro_batch_size = 2
    cfg.training.global_batch_size = 2 * pc.dp_size
    tr = Trainer(cfg, device=dev, pc=pc, telemetry=False)
    try:
        tr.run(max_steps=6)
        print(f"rank {pc.rank}: NO_FAILURE_SEEN")
    except RankFailure as e:
        print(f"DETECTED rank={pc.rank} missing={e.ranks} step={e.step}", flush=True)
    os._exit(0)          # the group is broken: leave without the collective teardown


def mode_timeout(pc, dev):
    """Only rank 0 launches the fused all-gather GEMM; its peers never push, so the wait on their
    counters must give up after the limit and report it through the status word."""
    import time
    from elfa_b200 import native
    from elfa_b200.parallel import fused
    from elfa_b200.runtime.symm import SymmetricArena
    pc.symm = SymmetricArena.for_group(pc.tp_group, dev, 256 << 20)
    fused._WAIT_MS = 300
    x = torch.randn(128, 256, device=dev).to(torch.bfloat16)
    w = torch.randn(256, 256, device=dev).to(torch.bfloat16)
    pc.comm_backend = "fused"
    # every rank creates the slot (the creation barrier is collective) ...
    st = fused._state(pc)
    st.next_slot("ag", fused._round_class(128 * pc.tp_size * 256 * 2))
    st.counter["ag"] -= 1
    dist.barrier()
    if pc.rank == 0:
        t0 = time.time()
        tpl.ag_gemm(x, w, pc, b_mn=True)
        torch.cuda.synchronize()
        dt = time.time() - t0
        s = native.status()
        assert s & native.ST_FLAG_TIMEOUT, f"expected the flag-timeout status, got 0x{s:x}"
        assert dt < 5.0, f"bounded wait took {dt:.1f}s"
        # the context is still usable
        assert float((x.float() @ w.float()).abs().sum()) > 0
        print(f"TIMEOUT_OK waited={dt:.2f}s")
    dist.barrier()


def main():
    mode = sys.argv[1]
    backend = sys.argv[2] if len(sys.argv) > 2 else "nccl"
    dtype = sys.argv[3] if len(sys.argv) > 3 else "bf16"
    use_cuda = torch.cuda.is_available() and mode not in ("tp_cpu", "zero_cpu", "ckpt_cpu", "killrank_cpu", "cp_cpu", "hybrid_cpu", "baseline_cpu", "efla_tp_cpu")
    world = init_distributed("nccl" if use_cuda else "gloo")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if use_cuda else torch.device("cpu")
    if mode == "killrank_cpu":
        mode_killrank(dev)
        return
    if mode == "ckpt_cpu":
        mode_ckpt(dev, int(sys.argv[2]), sys.argv[3], int(sys.argv[4]) if len(sys.argv) > 4 else 1,
                  sys.argv[5] if len(sys.argv) > 5 else "fp32", int(sys.argv[6]) if len(sys.argv) > 6 else None)
        dist.destroy_process_group()
        return
    if mode in ("efla_tp", "efla_tp_cpu"):
        mode_efla_tp(dev, dtype, int(sys.argv[4]) if len(sys.argv) > 4 else 2, int(sys.argv[5]) if len(sys.argv) > 5 else 1)
        dist.destroy_process_group()
        return
    if mode in ("baseline", "baseline_cpu"):
        mode_baseline(dev, dtype, int(sys.argv[4]) if len(sys.argv) > 4 else 2, int(sys.argv[5]) if len(sys.argv) > 5 else 0)
        dist.destroy_process_group()
        return
    if mode in ("hybrid", "hybrid_cpu"):
        mode_hybrid(dev, backend, dtype, int(sys.argv[4]) if len(sys.argv) > 4 else 2)
        dist.destroy_process_group()
        return
    if mode in ("cp", "cp_cpu"):
        mode_cp(dev, dtype, int(sys.argv[4]) if len(sys.argv) > 4 else 1, sys.argv[5] if len(sys.argv) > 5 else "ring")
        dist.destroy_process_group()
        return
    if mode in ("zero", "zero_cpu"):
        mode_zero(dev, backend, dtype, int(sys.argv[4]) if len(sys.argv) > 4 else 1)
        dist.destroy_process_group()
        return
    pc = build_context(world, True, backend)
    if mode == "fused":
        mode_fused(pc, dev)
    elif mode in ("tp", "tp_cpu"):
        mode_tp(pc, dev, backend, dtype)
    elif mode == "timeout":
        mode_timeout(pc, dev)
    elif mode == "mailbox":
        mode_mailbox(pc, dev)
    elif mode == "multimem":
        mode_multimem(pc, dev)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
