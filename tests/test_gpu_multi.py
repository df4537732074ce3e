"""Multi-GPU tests: fused all-gather→GEMM / GEMM→reduce-scatter kernels, TP training, bounded waits.

Each test launches one process per GPU (2 by default, ELFA_TEST_GPUS to change) with NVLS disabled
in NCCL; the kernels under test use plain peer loads / stores."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _ngpus():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    want = int(os.environ.get("ELFA_TEST_GPUS", "2"))
    return min(n, want)


def _run(args, port, timeout=600, extra_env=None, nproc=None):
    n = _ngpus()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    if nproc is not None:
        if n < nproc:
            pytest.skip(f"needs at least {nproc} GPUs (ELFA_TEST_GPUS={nproc})")
        n = nproc
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "dist_worker.py"), *args]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **(extra_env or {}))
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)


def _why(r):
    """The workers' own error lines first (the launcher's per-rank summary is long at 8 ranks), then the tails."""
    own = [ln for ln in r.stderr.splitlines() if ("Error" in ln or "assert" in ln) and "ChildFailedError" not in ln and "elastic" not in ln]
    return "\n".join(own[:12]) + "\n" + r.stdout[-2000:] + r.stderr[-3000:]


def test_fused_ag_gemm_and_gemm_rs(cuda_device):
    r = _run(["fused"], 29701)
    assert r.returncode == 0, _why(r)
    assert "FUSED_OK" in r.stdout


@pytest.mark.parametrize("mode", ["ring", "zigzag", "ulysses"])
def test_context_parallel_attention_and_training(cuda_device, mode):
    r = _run(["cp", "nccl", "bf16", "1", mode], {"ring": 29710, "zigzag": 29712, "ulysses": 29711}[mode])
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "CP_OK" in r.stdout


@pytest.mark.parametrize("backend", ["nccl", "fused"])
def test_tp_training_matches_single_gpu(cuda_device, backend):
    r = _run(["tp", backend, "bf16"], 29702 if backend == "nccl" else 29703)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "TP_OK" in r.stdout


def test_tp_mxfp8_quantised_all_gather_matches_single_gpu(cuda_device):
    """MXFP8 QAT with the fused backend: column-parallel layers all-gather e4m3 payloads + scales."""
    r = _run(["tp", "fused", "bf16"], 29708, extra_env={"ELFA_TEST_QUANT": "mxfp8"})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "TP_OK" in r.stdout


def test_tp_mxfp8_quantised_backward_matches_single_gpu(cuda_device):
    """quant.backward = mxfp8 under tensor parallelism: row-parallel layers all-gather e4m3 payloads of dy, the
    reduce-scatter kernel multiplies the dequantised dy; the losses follow the single-GPU run with the same setting."""
    r = _run(["tp", "fused", "bf16"], 29713, extra_env={"ELFA_TEST_QUANT": "mxfp8", "ELFA_TEST_QUANT_BACKWARD": "mxfp8"})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "TP_OK" in r.stdout


def test_missing_peer_signal_times_out_cleanly(cuda_device):
    r = _run(["timeout"], 29704)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "TIMEOUT_OK" in r.stdout


@pytest.mark.parametrize("backend", ["nccl", "fused"])
def test_zero1_data_parallel_matches_single_gpu(cuda_device, backend):
    r = _run(["zero", backend, "bf16", "1"], 29705 if backend == "nccl" else 29706)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "ZERO_OK" in r.stdout
    if backend == "fused":
        assert "fused=True" in r.stdout


@pytest.mark.parametrize("backend", ["nccl", "fused"])
def test_zero3_parameter_sharding_matches_single_gpu(cuda_device, backend):
    """Stage 3: blocks gathered on demand (prefetch on a side stream), gradients reduce-scattered per block;
    `fused` = peer-load gather / reduce kernels on a symmetric arena instead of the library collectives."""
    r = _run(["zero", backend, "bf16", "3"], 29707 if backend == "nccl" else 29708)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "ZERO_OK stage=3" in r.stdout
    if backend == "fused":
        assert "peer_kernels=True" in r.stdout


def test_zero3_parameter_gather_inside_the_gemm(cuda_device):
    """Stage 3 with the forward products fetching their matrices from the owners' shards themselves (bulk loads from peer
    memory into the local slot, K blocks multiplied as they arrive); same losses as one GPU on the global batch."""
    r = _run(["zero", "fused", "bf16", "3"], 29718, extra_env={"ELFA_ZERO3_GATHER_IN_GEMM": "1"})
    assert r.returncode == 0, _why(r)
    assert "ZERO_OK stage=3" in r.stdout and "gather_in_gemm=True" in r.stdout


@pytest.mark.parametrize("backend", ["nccl", "fused"])
def test_zero2_gradient_sharding_matches_single_gpu(cuda_device, backend):
    """Stage 2: whole parameters, per-block gradient slots reduce-scattered (bf16 on the wire, side stream) into fp32 shards,
    parameter shards all-gathered after the update; two micro-batches per step."""
    r = _run(["zero", backend, "bf16", "2"], 29714 if backend == "nccl" else 29715)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "ZERO_OK stage=2" in r.stdout
    if backend == "fused":
        assert "peer_kernels=True" in r.stdout


def test_multimem_collectives_through_the_switch(cuda_device):
    """ELFA_NVLS=1: all-reduce / reduce-scatter / all-gather with multimem instructions against the library's results; then a
    data-parallel run whose gradient all-reduce goes through the switch. Every rank exits normally."""
    r = _run(["multimem"], 29716, extra_env={"ELFA_NVLS": "1"})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "MULTIMEM_OK" in r.stdout or "MULTIMEM_SKIPPED" in r.stdout
    if "MULTIMEM_OK" in r.stdout:
        r = _run(["zero", "fused", "bf16", "0"], 29717, extra_env={"ELFA_NVLS": "1"})
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
        assert "ZERO_OK stage=0" in r.stdout and "nvls=True" in r.stdout


def test_tensor_parallel_times_data_parallel_zero2_mixed_quant(cuda_device):
    """The layout of the 13B benchmark configuration in small (TP 2 x DP 2, ZeRO-2, NVFP4 MLP + MXFP8 attention QAT, fused
    backend) against one GPU on the global batch. Needs four GPUs (``ELFA_TEST_GPUS=4``); the same worker runs as four gloo
    ranks in the CPU suite."""
    r = _run(["hybrid", "fused", "bf16", "2"], 29719, nproc=4)
    assert r.returncode == 0, _why(r)
    assert "HYBRID_OK tp=2 dp=2" in r.stdout


def test_efla_family_tensor_parallel_training(cuda_device):
    """The EFLA + PRISM family with heads, MLP columns and vocabulary sharded over two GPUs (bf16, Lion; Lion + Muon runs too)
    against one GPU on the global batch."""
    r = _run(["efla_tp", "nccl", "bf16", "2"], 29720, nproc=2)
    assert r.returncode == 0, _why(r)
    assert "EFLA_TP_OK tp=2" in r.stdout


def test_ring_handoff_through_peer_mailboxes(cuda_device):
    r = _run(["mailbox"], 29709)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "MAILBOX_OK" in r.stdout
