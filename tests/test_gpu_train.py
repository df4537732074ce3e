"""End-to-end: the small GPT trained on the GPU (bf16, native kernels) follows the CPU fp32 run."""
import os
import warnings

import pytest
import torch

from elfa_b200 import native

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(device, dtype, quant="none", steps=8, backward="none"):
    warnings.simplefilter("ignore")
    from elfa_b200.config import Config
    from elfa_b200.trainer import Trainer
    cfg = Config.from_file(os.path.join(ROOT, "configs", "bench", "smoke_cpu.yaml"), env_override=False)
    cfg.model.dtype = dtype
    cfg.checkpoint.dir = ""
    cfg.telemetry.log_file = ""
    cfg.quant.attention = cfg.quant.mlp = quant
    cfg.quant.backward = backward
    cfg.training.learning_rate = 3e-3          # large enough for the loss to move in a few steps
    tr = Trainer(cfg, device=device, telemetry=False)
    return tr, tr.run(max_steps=steps)


def test_loss_curve_matches_cpu_fp32(cuda_device):
    _, cpu = _run(torch.device("cpu"), "fp32")
    tr, gpu = _run(cuda_device, "bf16")
    assert native.status() == 0
    for a, b in zip(gpu, cpu):
        assert abs(a - b) < 0.03 * abs(b), (gpu, cpu)
    assert native.lib.raw("elfa_launch_count")(0) > 0


@pytest.mark.parametrize("quant", ["mxfp8", "nvfp4"])
def test_qat_loss_curve_close_to_cpu_oracle(cuda_device, quant):
    _, cpu = _run(torch.device("cpu"), "fp32", quant, steps=4)
    _, gpu = _run(cuda_device, "bf16", quant, steps=4)
    assert native.status() == 0
    for a, b in zip(gpu, cpu):
        assert abs(a - b) < 0.05 * abs(b), (gpu, cpu)


def test_mxfp8_quantised_backward_close_to_cpu_oracle(cuda_device):
    """quant.backward = mxfp8: dy and the weights' output axis are quantised, the input-gradient GEMMs run block-scaled;
    the CPU oracle applies the same quantisation to fp32 operands."""
    _, cpu = _run(torch.device("cpu"), "fp32", "mxfp8", steps=4, backward="mxfp8")
    _, plain = _run(torch.device("cpu"), "fp32", "mxfp8", steps=4)
    _, gpu = _run(cuda_device, "bf16", "mxfp8", steps=4, backward="mxfp8")
    assert native.status() == 0
    assert cpu != plain                       # the backward quantisation changes the updates
    for a, b in zip(gpu, cpu):
        assert abs(a - b) < 0.05 * abs(b), (gpu, cpu)


def test_checkpoint_resume_continues_identically(cuda_device, tmp_path):
    warnings.simplefilter("ignore")
    from elfa_b200.config import Config
    from elfa_b200.trainer import Trainer
    cfg = Config.from_file(os.path.join(ROOT, "configs", "bench", "smoke_cpu.yaml"), env_override=False)
    cfg.model.dtype = "bf16"
    cfg.checkpoint.dir = str(tmp_path / "ck")
    cfg.checkpoint.save_interval = 3
    cfg.telemetry.log_file = ""
    a = Trainer(cfg, device=cuda_device, telemetry=False)
    la = a.run(max_steps=6)
    a.close()
    b = Trainer(cfg, device=cuda_device, telemetry=False)
    meta = b.resume(os.path.join(cfg.checkpoint.dir, "step_00000003"))
    assert meta.step == 3
    cfg.checkpoint.save_interval = 0
    lb = b.run(max_steps=3)
    for x, y in zip(la[3:], lb):
        assert abs(x - y) < 2e-3 * abs(x), (la, lb)


def test_deterministic_mode_repeats_bit_for_bit(cuda_device):
    """runtime.deterministic: no split-K atomics, embedding gradient reduced over sorted ids - two runs give identical bits."""
    warnings.simplefilter("ignore")
    from elfa_b200.config import Config
    from elfa_b200.trainer import Trainer

    def run():
        cfg = Config.from_file(os.path.join(ROOT, "configs", "bench", "smoke_cpu.yaml"), env_override=False)
        cfg.model.dtype = "bf16"
        cfg.checkpoint.dir = ""
        cfg.telemetry.log_file = ""
        cfg.runtime.deterministic = True
        cfg.training.learning_rate = 3e-3
        tr = Trainer(cfg, device=cuda_device, telemetry=False)
        losses = tr.run(max_steps=3)
        return losses, tr.flat.flat.clone()
    la, wa = run()
    lb, wb = run()
    assert la == lb and torch.equal(wa, wb)
    assert native.deterministic()
