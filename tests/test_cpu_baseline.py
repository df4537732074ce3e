"""The library baseline arm (eager PyTorch, baseline/torch_nccl.py) trains the same model as the product arm: same initial
weights, same data, same losses on CPU in fp32."""
import os
import sys
import warnings

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))


def _cfg(quant="none", backward="none"):
    from elfa_b200.config import Config
    cfg = Config.from_file(os.path.join(ROOT, "configs", "bench", "smoke_cpu.yaml"), env_override=False)
    cfg.model.dtype = "fp32"
    cfg.checkpoint.dir = ""
    cfg.telemetry.log_file = ""
    cfg.quant.attention = cfg.quant.mlp = quant
    cfg.quant.backward = backward
    cfg.training.learning_rate = 3e-3
    return cfg


def _losses(trainer, loader, steps):
    out = []
    for _ in range(steps):
        out.append(trainer.finish_step(trainer.train_step([loader.next_cycling() for _ in range(trainer.accum)])))
    return out


def test_baseline_arm_follows_the_product_arm_on_cpu():
    warnings.simplefilter("ignore")
    from torch_nccl import BaselineTrainer
    from elfa_b200.trainer import Trainer
    for quant, bwd in (("none", "none"), ("mxfp8", "mxfp8")):
        a = Trainer(_cfg(quant, bwd), device=torch.device("cpu"), telemetry=False)
        la = a.run(max_steps=4)
        b = BaselineTrainer(_cfg(quant, bwd), torch.device("cpu"))
        lb = _losses(b, b.make_loader(), 4)
        assert abs(la[0] - lb[0]) < 1e-4 * abs(la[0]), (la, lb)          # same initial weights and data
        for x, y in zip(la, lb):
            assert abs(x - y) < 2e-3 * abs(x), (quant, la, lb)
