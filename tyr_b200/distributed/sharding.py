"""Type-level sharding (Tyr/Sharding.lean): shard sizes/offsets with the remainder spread over the
first shards, ``ShardedTensor`` with a gather cache, ``MaybeSharded``, ``ShardedEmbedding`` and
``ShardedAdamState``.  An out-of-range shard axis means "replicated"."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple, Union

import torch


@dataclass(frozen=True)
class ShardDim:
    kind: str = "first"   # "first" | "last" | "dim"
    n: int = 0

    first = None
    last = None

    @staticmethod
    def dim(n: int) -> "ShardDim":
        return ShardDim("dim", n)

    def resolve(self, rank: int) -> Optional[int]:
        d = 0 if self.kind == "first" else (rank - 1 if self.kind == "last" else self.n)
        return d if 0 <= d < rank else None


ShardDim.first = ShardDim("first")
ShardDim.last = ShardDim("last")


@dataclass(frozen=True)
class ShardSpec:
    num_shards: int
    shard_idx: int
    shard_dim: ShardDim = ShardDim.first


def shard_size(full: int, num_shards: int, idx: int) -> int:
    base, rem = full // num_shards, full % num_shards
    return base + 1 if idx < rem else base


def shard_offset(full: int, num_shards: int, idx: int) -> int:
    base, rem = full // num_shards, full % num_shards
    return idx * (base + 1) if idx < rem else rem * (base + 1) + (idx - rem) * base


def sharded_shape(shape: Tuple[int, ...], spec: ShardSpec) -> Tuple[int, ...]:
    d = spec.shard_dim.resolve(len(shape))
    if d is None:
        return tuple(shape)
    return tuple(shape[:d]) + (shard_size(shape[d], spec.num_shards, spec.shard_idx),) + tuple(shape[d + 1:])


class ShardedTensor:
    def __init__(self, full_shape, rank: int, world_size: int, shard: torch.Tensor, shard_dim: ShardDim = ShardDim.first):
        if not 0 <= rank < world_size:
            raise ValueError("ShardedTensor: rank must be < world size")
        self.full_shape = tuple(full_shape)
        self.rank, self.world_size, self.shard_dim = rank, world_size, shard_dim
        want = sharded_shape(self.full_shape, ShardSpec(world_size, rank, shard_dim))
        if tuple(shard.shape) != want:
            raise ValueError(f"ShardedTensor: shard shape {list(shard.shape)} != expected {list(want)}")
        self.shard = shard
        self.cached_full: Optional[torch.Tensor] = None
        self.cache_is_stale = True

    @staticmethod
    def from_full(full: torch.Tensor, rank: int, world_size: int, shard_dim: ShardDim = ShardDim.first) -> "ShardedTensor":
        d = shard_dim.resolve(full.dim())
        if d is None:
            piece = full
        else:
            off = shard_offset(full.shape[d], world_size, rank)
            piece = full.narrow(d, off, shard_size(full.shape[d], world_size, rank)).clone()
        return ShardedTensor(full.shape, rank, world_size, piece, shard_dim)

    def gather(self) -> torch.Tensor:
        """Full tensor (cached until the shard changes).  Uneven shards are padded for transport."""
        if self.cached_full is not None and not self.cache_is_stale:
            return self.cached_full
        from . import all_gather_list, is_initialized
        d = self.shard_dim.resolve(len(self.full_shape))
        if d is None or not is_initialized() or self.world_size == 1:
            full = self.shard if d is None else self.shard
        else:
            n = self.full_shape[d]
            mx = shard_size(n, self.world_size, 0)
            pad = self.shard
            if self.shard.shape[d] < mx:
                padshape = list(self.shard.shape)
                padshape[d] = mx - self.shard.shape[d]
                pad = torch.cat([self.shard, self.shard.new_zeros(padshape)], dim=d)
            parts = all_gather_list(pad)
            parts = [p.narrow(d, 0, shard_size(n, self.world_size, r)) for r, p in enumerate(parts)]
            full = torch.cat(parts, dim=d)
        self.cached_full, self.cache_is_stale = full, False
        return full

    def scatter_grad(self, full_grad: torch.Tensor) -> torch.Tensor:
        """reduce_scatter(sum) of a full gradient: this rank's slice of the summed gradient."""
        from . import ReduceOp, all_reduce, is_initialized
        d = self.shard_dim.resolve(len(self.full_shape))
        g = all_reduce(full_grad, ReduceOp.sum) if (is_initialized() and self.world_size > 1) else full_grad
        if d is None:
            return g
        return g.narrow(d, shard_offset(self.full_shape[d], self.world_size, self.rank),
                        shard_size(self.full_shape[d], self.world_size, self.rank)).clone()

    def update_shard(self, new_shard: torch.Tensor) -> "ShardedTensor":
        if new_shard.shape != self.shard.shape:
            raise ValueError("updateShard: shape mismatch")
        self.shard = new_shard
        self.cache_is_stale = True
        return self


class MaybeSharded:
    """Either a replicated tensor or a ShardedTensor."""

    def __init__(self, value: Union[torch.Tensor, ShardedTensor]):
        self.value = value

    @property
    def is_sharded(self) -> bool:
        return isinstance(self.value, ShardedTensor)

    def full(self) -> torch.Tensor:
        return self.value.gather() if self.is_sharded else self.value


class ShardedEmbedding:
    """Embedding table sharded by rows; lookups gather the table first."""

    def __init__(self, table: ShardedTensor):
        self.table = table

    def forward(self, idx: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.embedding(idx, self.table.gather())


@dataclass
class ShardedAdamState:
    exp_avg: ShardedTensor
    exp_avg_sq: ShardedTensor
    step: int = 0
