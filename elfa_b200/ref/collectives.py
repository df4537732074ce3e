"""Oracles for the fused compute + collective kernels: N ranks simulated in one process.

Every function takes per-rank inputs as a list (index = rank) and returns per-rank outputs the same way, doing in
plain fp32 / fp64 tensor code exactly what the fused kernels promise, including the order of the sums (rank
0, 1, ..., N-1: the kernels reduce slots in that fixed order, which is what makes them deterministic). The
multi-GPU tests compare the kernels with NCCL; these functions pin down the semantics without any process
group, and are themselves checked against the unsharded computation in the CPU tests.

* :func:`ag_gemm`     - all-gather of row shards, then GEMM with the rank's weight shard (column parallel);
* :func:`gemm_rs`     - GEMM on the rank's slice of the contraction dimension, then reduce-scatter of rows;
* :func:`rs_adamw_ag` - ZeRO-1/2 step: gradient reduce-scatter with 1/N (and loss-scale, clip) scaling, AdamW on the
  rank's shard of fp32 master weights, all-gather of the updated low-precision parameters;
* :func:`zero3_gather_gemm` - parameter shards gathered in front of the GEMM that consumes them.

reference: ``src/distributed/tensor_parallel.zig:77-170``, ``src/distributed/sequence_parallel.zig:79-200``,
``src/distributed/zero_sharding.zig:115-181`` (the unfused NCCL sequences these replace); AdamW as in
``src/kernels/optim_kernels.zig:129-167``.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch


def _ordered_sum(parts: List[torch.Tensor]) -> torch.Tensor:
    acc = parts[0].clone()
    for p in parts[1:]:
        acc = acc + p           # rank order, left to right
    return acc


def ag_gemm(x_shards: List[torch.Tensor], w_shards: List[torch.Tensor]) -> List[torch.Tensor]:
    """``x_shards[r] [M/N, K]``, ``w_shards[r] [K, n_r]`` -> rank r gets ``cat(x_shards) @ w_shards[r]`` ``[M, n_r]``."""
    x_full = torch.cat(x_shards, 0)
    return [x_full @ w for w in w_shards]


def gemm_rs(a_shards: List[torch.Tensor], w_shards: List[torch.Tensor]) -> List[torch.Tensor]:
    """``a_shards[r] [M, k_r]``, ``w_shards[r] [k_r, D]`` -> rank r gets rows ``[r M/N, (r+1) M/N)`` of the sum over ranks of
    ``a_shards[q] @ w_shards[q]`` (partials added in rank order)."""
    n = len(a_shards)
    partial = [a @ w for a, w in zip(a_shards, w_shards)]
    rows = partial[0].shape[0] // n
    return [_ordered_sum([p[r * rows:(r + 1) * rows] for p in partial]) for r in range(n)]


def adamw_update(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, step: int, lr: float, beta1: float, beta2: float,
                 eps: float, wd: float, decay_mask: Optional[torch.Tensor] = None) -> None:
    """In-place decoupled AdamW with bias correction on fp32 tensors."""
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    mh = m / (1 - beta1 ** step)
    vh = v / (1 - beta2 ** step)
    decay = wd if decay_mask is None else wd * decay_mask
    p.mul_(1 - lr * decay).sub_(lr * mh / (vh.sqrt() + eps))


def rs_adamw_ag(grads: List[torch.Tensor], master: List[torch.Tensor], m: List[torch.Tensor], v: List[torch.Tensor], step: int, lr: float,
                beta1: float = 0.9, beta2: float = 0.95, eps: float = 1e-8, wd: float = 0.1, loss_scale: float = 1.0,
                max_norm: float = 0.0, param_dtype: torch.dtype = torch.bfloat16) -> Tuple[List[torch.Tensor], float]:
    """One ZeRO-1/2 optimizer step over flat buffers. ``grads[r] [P]`` is rank r's full local gradient; ``master[r]``,
    ``m[r]``, ``v[r]`` are its fp32 shard ``[P/N]`` (updated in place). Returns every rank's gathered parameter buffer
    ``[P]`` in ``param_dtype`` and the global gradient norm. Phase A: the shard of the summed gradient, scaled by
    ``1 / (N loss_scale)``, and its sum of squares; the norm needs all shards before any update (phase B)."""
    n = len(grads)
    shard = grads[0].numel() // n
    red = [_ordered_sum([g[r * shard:(r + 1) * shard].float() for g in grads]) / (n * loss_scale) for r in range(n)]
    norm = float(torch.sqrt(_ordered_sum([(x.double() ** 2).sum() for x in red])))
    coef = 1.0 if max_norm <= 0 or norm <= max_norm else max_norm / (norm + 1e-6)
    for r in range(n):
        adamw_update(master[r], red[r] * coef, m[r], v[r], step, lr, beta1, beta2, eps, wd)
    gathered = torch.cat([p.to(param_dtype) for p in master], 0)
    return [gathered.clone() for _ in range(n)], norm


def zero3_gather_gemm(x: List[torch.Tensor], w_shards: List[torch.Tensor], shape: Tuple[int, int]) -> List[torch.Tensor]:
    """``w_shards[r]``: rank r's flat 1/N of a ``shape = [K, N_out]`` weight; every rank multiplies its own activations
    ``x[r] [M, K]`` with the gathered weight."""
    w = torch.cat(w_shards, 0)[: shape[0] * shape[1]].view(shape)
    return [xr @ w for xr in x]
