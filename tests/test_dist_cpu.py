"""Multi-process CPU (gloo) tests of the tensor/sequence-parallel layer."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(nproc, args, port, timeout=600, extra_env=None, allow_fail=False):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "dist_worker.py"), *args]
    env = dict(os.environ, OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES="")
    env.update(extra_env or {})
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)


@pytest.mark.parametrize("world", [2, 4])
def test_tp_sp_matches_single_rank_on_cpu(world):
    r = _run(world, ["tp_cpu", "nccl", "fp32"], 29611 + world)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "TP_OK" in r.stdout


def test_tp_sp_with_quantised_backward_matches_single_rank_on_cpu():
    """MXFP8 forward and backward quantisation (dy blocks along its last dimension, weights along the same one): the
    tensor-parallel result equals the single-rank one because the shard boundaries are block boundaries."""
    r = _run(2, ["tp_cpu", "nccl", "fp32"], 29618, extra_env={"ELFA_TEST_QUANT": "mxfp8", "ELFA_TEST_QUANT_BACKWARD": "mxfp8"})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "TP_OK" in r.stdout


def test_tp_sp_with_grouped_query_attention_and_packed_rows_matches_single_rank_on_cpu():
    """model.num_kv_heads = 2 under 4 query heads, tensor parallel over 2 ranks (one key head each), data.pack_sequences on."""
    r = _run(2, ["tp_cpu", "nccl", "fp32"], 29619, extra_env={"ELFA_TEST_KV_HEADS": "2", "ELFA_TEST_PACK": "1"})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "TP_OK" in r.stdout


@pytest.mark.parametrize("world,tp,mode", [(2, 1, "ring"), (4, 2, "ring"), (2, 1, "ulysses"), (2, 1, "zigzag")])
def test_context_parallel_attention_and_training_on_cpu(world, tp, mode):
    r = _run(world, ["cp_cpu", "nccl", "fp32", str(tp), mode], 29660 + world + {"ring": 0, "ulysses": 10, "zigzag": 20}[mode])
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "CP_OK" in r.stdout


def test_tensor_parallel_times_data_parallel_zero2_mixed_quant_on_cpu():
    """The layout of the 13B benchmark configuration in small: TP 2 x DP 2, ZeRO-2, NVFP4 MLP + MXFP8 attention QAT."""
    r = _run(4, ["hybrid_cpu", "nccl", "fp32", "2"], 29691)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "HYBRID_OK tp=2 dp=2" in r.stdout


@pytest.mark.parametrize("stage", [0, 1, 2, 3])
def test_zero_data_parallel_matches_single_rank_on_cpu(stage):
    r = _run(2, ["zero_cpu", "nccl", "fp32", str(stage)], 29621 + stage)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "ZERO_OK" in r.stdout


def test_zero3_gather_in_gemm_bookkeeping_on_cpu():
    """Stage 3 with the forward products fetching their matrices themselves (on CPU ranks a library all-gather stands in for
    the kernel's copy warps): same losses as one rank, four fetches per block and micro-batch, whole-block gathers only in
    backward."""
    r = _run(2, ["zero_cpu", "nccl", "fp32", "3"], 29628, extra_env={"ELFA_ZERO3_GATHER_IN_GEMM": "1"})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "ZERO_OK stage=3" in r.stdout and "gather_in_gemm=True" in r.stdout


@pytest.mark.parametrize("stage", [1, 2, 3])
def test_sharded_optimizer_state_survives_checkpoint(stage, tmp_path):
    r = _run(2, ["ckpt_cpu", str(stage), str(tmp_path / "ck")], 29641 + stage)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "CKPT_OK" in r.stdout


@pytest.mark.parametrize("world,stage,tp,dtype,resume_tp", [(2, 0, 2, "fp32", 2), (2, 0, 2, "bf16", 2), (4, 1, 2, "bf16", 2),
                                                            (2, 1, 2, "fp32", 1), (2, 1, 1, "fp32", 2)])
def test_optimizer_state_is_layout_independent(world, stage, tp, dtype, resume_tp, tmp_path):
    """Tensor-parallel ranks get their own moments / master weights back, and a checkpoint written under one
    (tp, dp) split resumes under another with its moments intact."""
    r = _run(world, ["ckpt_cpu", str(stage), str(tmp_path / "ck"), str(tp), dtype, str(resume_tp)], 29700 + world + 3 * tp + resume_tp)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "CKPT_OK" in r.stdout


@pytest.mark.parametrize("world,tp,stage", [(2, 2, 0), (4, 2, 1)])
def test_baseline_arm_under_tensor_and_data_parallelism_matches_the_product_arm(world, tp, stage):
    r = _run(world, ["baseline_cpu", "nccl", "fp32", str(tp), str(stage)], 29730 + world + stage)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "BASELINE_OK" in r.stdout


@pytest.mark.parametrize("world,tp,cp", [(2, 2, 1), (4, 2, 1), (2, 1, 2), (4, 2, 2)])
def test_efla_family_tensor_and_sequence_parallel_training_matches_single_rank_on_cpu(world, tp, cp):
    """Heads sharded over tensor-parallel ranks; with cp > 1 the sequences are split over ranks too (state hand-off and
    ShortConv halo differentiated through), through the trainer."""
    r = _run(world, ["efla_tp_cpu", "nccl", "fp32", str(tp), str(cp)], 29740 + world + 10 * cp)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "EFLA_TP_OK" in r.stdout


def test_efla_family_tensor_parallel_in_bf16_on_cpu():
    """The same with a bf16 model: every weight stays bf16 although the fp32 learned scalar leads the flat buffer's order
    (tensor-parallel replicated class), and the losses follow the single-rank run."""
    r = _run(2, ["efla_tp_cpu", "nccl", "bf16", "2", "1"], 29759)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "EFLA_TP_OK tp=2" in r.stdout


def test_rank_that_leaves_between_steps_is_detected_on_the_host(tmp_path):
    """Host-side fault injection (kill_rank) + heartbeat soft barrier: survivors raise RankFailure, nobody hangs."""
    env = {"ELFA_FAULT": "kill_rank:rank=2,step=3,code=0", "ELFA_HEARTBEAT_DIR": str(tmp_path / "hb"), "ELFA_HEARTBEAT_TIMEOUT_S": "3"}
    r = _run(3, ["killrank_cpu"], 29651, extra_env=env, allow_fail=True)
    out = r.stdout + r.stderr
    assert "DETECTED rank=0 missing=[2] step=3" in out and "DETECTED rank=1 missing=[2] step=3" in out, out[-3000:]
    assert "NO_FAILURE_SEEN" not in out


def test_fault_plan_parsing_and_nan_gradient_skips_the_step():
    import torch
    from elfa_b200.config import Config
    from elfa_b200.runtime.fault import FaultPlan
    from elfa_b200.trainer import Trainer
    plan = FaultPlan.parse("nan_grad:rank=0,step=1; delay_ms:rank=1,step=2,ms=5")
    assert plan.active("nan_grad", 0, 1) and not plan.active("nan_grad", 0, 2) and plan.active("delay_ms", 1, 2).args["ms"] == 5
    with pytest.raises(ValueError):
        FaultPlan.parse("explode:rank=0")
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = Config.from_file(os.path.join(root, "configs", "bench", "smoke_cpu.yaml"), env_override=False)
    cfg.checkpoint.dir = ""
    cfg.telemetry.log_file = ""
    cfg.training.mixed_precision = True
    cfg.training.dynamic_loss_scale = True
    cfg.training.loss_scale = 1024.0
    tr = Trainer(cfg, device=torch.device("cpu"), telemetry=False)
    tr.faults = plan
    w0 = tr.flat.flat.clone()
    tr.run(max_steps=1)                       # step 0: normal
    w1 = tr.flat.flat.clone()
    assert not torch.equal(w0, w1) and tr.scaler.scale == 1024.0
    tr.run(max_steps=1)                       # step 1: NaN injected -> update skipped, loss scale halved
    assert torch.equal(tr.flat.flat, w1) and tr.scaler.scale == 512.0 and tr.scaler.skipped_steps == 1
