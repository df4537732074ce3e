"""Single-node multi-GPU launcher: one process per GPU through ``torch.distributed.run``.

    python -m elfa_b200.launch --gpus 8 train --config configs/bench/gpt7b_tp8_mxfp8.yaml [--resume latest]
    python -m elfa_b200.launch --gpus 1 smoke-test

Plays the role of the reference's cloud launcher (reference: ``cloud/modal/train.py:198-339`` - an
8-GPU job that shells out to the trainer binary with ``NCCL_DEBUG=INFO``,
``NCCL_ASYNC_ERROR_HANDLING=1`` and resolves ``latest`` / the highest ``step_N`` checkpoint,
``:84-124``) for a plain machine: it checks the GPU count, sets the environment, resolves
``--resume latest`` against the configured checkpoint directory and starts the ranks on 127.0.0.1.
With ``--max-restarts N`` it is also the recovery loop: a job that ends with an error (a rank that left, a
``RankFailure`` from the heartbeat, a ``CommTimeout`` from a bounded device wait) is started again from its newest
checkpoint; ``ELFA_RESTART_ATTEMPT`` tells the job which start it is.
"""
from __future__ import annotations

import argparse
import os
import socket
import subprocess
import sys
from typing import List


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def resolve_resume(argv: List[str]) -> List[str]:
    """Replaces ``--resume latest`` by the newest checkpoint of the config's checkpoint directory."""
    if "--resume" not in argv:
        return argv
    i = argv.index("--resume")
    if i + 1 >= len(argv) or argv[i + 1] != "latest":
        return argv
    from .checkpoint.manager import resolve_checkpoint
    from .config import Config
    ckdir = None
    if "--checkpoint-dir" in argv:
        ckdir = argv[argv.index("--checkpoint-dir") + 1]
    elif "--config" in argv:
        ckdir = Config.from_file(argv[argv.index("--config") + 1], env_override=False).checkpoint.dir
    if not ckdir:
        raise SystemExit("--resume latest needs --config or --checkpoint-dir")
    out = list(argv)
    out[i + 1] = resolve_checkpoint(ckdir)
    return out


def restart_args(argv: List[str]) -> List[str]:
    """The command line of a restart: ``train`` resumes from the newest checkpoint when there is one, anything
    else (and a run that has not saved yet) starts over."""
    if not argv or argv[0] != "train":
        return list(argv)
    out = list(argv)
    if "--resume" in out:
        i = out.index("--resume")
        del out[i:i + 2]
    try:
        return resolve_resume(out + ["--resume", "latest"])
    except (FileNotFoundError, ValueError, SystemExit, OSError):
        return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--gpus", type=int, default=0, help="processes to start (0 = all visible GPUs)")
    ap.add_argument("--port", type=int, default=0)
    ap.add_argument("--nccl-debug", default="WARN")
    ap.add_argument("--max-restarts", type=int, default=0,
                    help="start the job again (train: from the newest checkpoint) when it exits with an error, at most this many times")
    ap.add_argument("rest", nargs=argparse.REMAINDER, help="elfa_b200 command line (train --config ...)")
    a = ap.parse_args(argv)
    if not a.rest:
        ap.error("missing command, e.g. train --config configs/train.yaml")
    import torch
    n_visible = torch.cuda.device_count() if torch.cuda.is_available() else 0
    n = a.gpus or max(n_visible, 1)
    if n_visible and n > n_visible:
        raise SystemExit(f"--gpus {n} requested but only {n_visible} GPUs are visible")
    env = dict(os.environ)
    env.setdefault("NCCL_DEBUG", a.nccl_debug)
    env.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "1")
    env.setdefault("CUDA_DEVICE_ORDER", "PCI_BUS_ID")
    env.setdefault("OMP_NUM_THREADS", "4")
    if a.max_restarts > 0 or env.get("ELFA_FAULT") or env.get("ELFA_HEARTBEAT_DIR"):
        # a job in which ranks may leave: no NVLink multicast bindings anywhere (NCCL's NVLS, the symmetric arena's)
        env.setdefault("NCCL_NVLS_ENABLE", "0")
        env.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        env["ELFA_NVLS"] = "0"
    attempt = 0
    rest = resolve_resume(a.rest)
    while True:
        env["ELFA_RESTART_ATTEMPT"] = str(attempt)
        if n == 1:
            cmd = [sys.executable, "-m", "elfa_b200", *rest]
        else:
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
                   "--master-port", str(a.port or _free_port()), "-m", "elfa_b200", *rest]
        rc = subprocess.call(cmd, env=env)
        if rc == 0 or attempt >= a.max_restarts:
            return rc
        # a rank left or reported a failure: start the job again from the newest checkpoint (the checkpoints are
        # world-size agnostic, so --gpus may differ between the original command line and a manual restart as well)
        attempt += 1
        rest = restart_args(a.rest)
        print(f"[launch] exit code {rc}: restart {attempt} of {a.max_restarts}: {' '.join(rest)}", file=sys.stderr, flush=True)


if __name__ == "__main__":
    sys.exit(main())
