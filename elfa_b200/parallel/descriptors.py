"""Parallelism descriptors: pure arithmetic, no communication.

reference: ``src/tensor/sharding.zig:121-175`` (``ShardSpec``: remainder-aware split - shard ``i`` of a
dimension of size ``n`` over ``s`` shards has ``n//s + 1`` elements if ``i < n % s`` else ``n//s``),
``:183-222`` (``TensorParallelConfig`` with per-layer shard dimensions), ``:224-287``
(``SequenceParallelConfig``), ``:289-355`` (``ZeroConfig``: stages 0-3 and the 1 MiB round-robin
ownership rule), ``:357-422`` (``ParallelConfig``: dp/tp/pp/sp ranks → global rank).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple

ZERO_CHUNK = 1 << 20


@dataclass
class ShardSpec:
    dim: int
    num_shards: int
    shard_id: int

    def local_size(self, n: int) -> int:
        base, rem = divmod(n, self.num_shards)
        return base + 1 if self.shard_id < rem else base

    def offset(self, n: int) -> int:
        base, rem = divmod(n, self.num_shards)
        i = self.shard_id
        return i * (base + 1) if i < rem else rem * (base + 1) + (i - rem) * base

    def local_shape(self, shape: Tuple[int, ...]) -> Tuple[int, ...]:
        s = list(shape)
        s[self.dim] = self.local_size(shape[self.dim])
        return tuple(s)


@dataclass
class TensorParallelConfig:
    size: int = 1
    rank: int = 0
    embed_shard_dim: int = 0        # vocabulary
    qkv_shard_dim: int = 1          # column parallel
    attn_out_shard_dim: int = 0     # row parallel
    mlp_up_shard_dim: int = 1
    mlp_down_shard_dim: int = 0

    def spec(self, dim: int) -> ShardSpec:
        return ShardSpec(dim, self.size, self.rank)


@dataclass
class SequenceParallelConfig:
    size: int = 1
    rank: int = 0
    use_ring_attention: bool = False

    def local_range(self, seq_len: int) -> Tuple[int, int]:
        """(offset, length) of this rank's contiguous token block."""
        s = ShardSpec(0, self.size, self.rank)
        return s.offset(seq_len), s.local_size(seq_len)


@dataclass
class ZeroConfig:
    stage: int = 0
    partitions: int = 1
    rank: int = 0

    def should_shard_optimizer(self) -> bool:
        return self.stage >= 1

    def should_shard_gradients(self) -> bool:
        return self.stage >= 2

    def should_shard_params(self) -> bool:
        return self.stage >= 3

    def owner_of(self, offset: int) -> int:
        """Owner of a byte/element offset under the reference's rule: 1 MiB chunks dealt round-robin."""
        return (offset // ZERO_CHUNK) % self.partitions

    def owns(self, offset: int) -> bool:
        return self.owner_of(offset) == self.rank

    def flat_range(self, numel: int) -> Tuple[int, int]:
        """The contiguous range this framework gives rank ``rank`` of a flat buffer of ``numel``
        elements (``numel`` is padded to a multiple of ``partitions`` by the caller)."""
        n = numel // self.partitions
        return self.rank * n, (self.rank + 1) * n


@dataclass
class ParallelConfig:
    dp_size: int = 1
    tp_size: int = 1
    pp_size: int = 1
    sp_size: int = 1
    dp_rank: int = 0
    tp_rank: int = 0
    pp_rank: int = 0
    sp_rank: int = 0

    def world_size(self) -> int:
        return self.dp_size * self.tp_size * self.pp_size * self.sp_size

    def global_rank(self) -> int:
        r = (self.pp_rank * self.dp_size + self.dp_rank) * self.tp_size + self.tp_rank
        if self.sp_size > 1:
            r = r * self.sp_size + self.sp_rank
        return r

    @classmethod
    def from_global_rank(cls, rank: int, dp: int, tp: int, pp: int = 1, sp: int = 1) -> "ParallelConfig":
        sp_rank = rank % sp if sp > 1 else 0
        r = rank // sp if sp > 1 else rank
        tp_rank = r % tp
        r //= tp
        dp_rank = r % dp
        pp_rank = r // dp
        return cls(dp, tp, pp, sp, dp_rank, tp_rank, pp_rank, sp_rank)


def split_sizes(n: int, parts: int) -> List[int]:
    return [ShardSpec(0, parts, i).local_size(n) for i in range(parts)]
