"""Multi-process CPU (gloo) tests of the tensor/sequence-parallel layer."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(nproc, args, port, timeout=600):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "dist_worker.py"), *args]
    env = dict(os.environ, OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES="")
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)


@pytest.mark.parametrize("world", [2, 4])
def test_tp_sp_matches_single_rank_on_cpu(world):
    r = _run(world, ["tp_cpu", "nccl", "fp32"], 29611 + world)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "TP_OK" in r.stdout


@pytest.mark.parametrize("stage", [0, 1, 3])
def test_zero_data_parallel_matches_single_rank_on_cpu(stage):
    r = _run(2, ["zero_cpu", "nccl", "fp32", str(stage)], 29621 + stage)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "ZERO_OK" in r.stdout


@pytest.mark.parametrize("stage", [1, 3])
def test_sharded_optimizer_state_survives_checkpoint(stage, tmp_path):
    r = _run(2, ["ckpt_cpu", str(stage), str(tmp_path / "ck")], 29641 + stage)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "CKPT_OK" in r.stdout
