"""DistributedSampler: the same LCG Fisher-Yates shuffle on every rank, different slices
(Tyr/Distributed.lean:246-351)."""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import List, Optional

_MASK = (1 << 64) - 1


def _lcg_next(state: int) -> int:
    return (state * 6364136223846793005 + 1442695040888963407) & _MASK


def _shuffle(arr: List[int], seed: int) -> List[int]:
    if len(arr) <= 1:
        return arr
    res = list(arr)
    state = seed & _MASK
    n = len(res)
    for i in range(n - 1):
        state = _lcg_next(state)
        j = i + state % (n - i)
        res[i], res[j] = res[j], res[i]
    return res


@dataclass
class DistributedSamplerConfig:
    dataset_size: int
    rank: int
    world_size: int
    seed: int = 42
    shuffle: bool = True
    drop_last: bool = False


@dataclass
class DistributedSampler:
    config: DistributedSamplerConfig
    indices: List[int]
    epoch: int = 0

    @staticmethod
    def create(cfg: DistributedSamplerConfig) -> "DistributedSampler":
        total, world, rank = cfg.dataset_size, cfg.world_size, cfg.rank
        per, rem = total // world, total % world
        start = rank * (per + 1) if rank < rem else rem * (per + 1) + (rank - rem) * per
        n = per + 1 if rank < rem else per
        if cfg.drop_last:
            n = per
            start = rank * per
        idx = list(range(total))
        if cfg.shuffle:
            idx = _shuffle(idx, cfg.seed)
        return DistributedSampler(cfg, idx[start:start + n], 0)

    def next_epoch(self) -> "DistributedSampler":
        e = self.epoch + 1
        s = DistributedSampler.create(replace(self.config, seed=(self.config.seed + e) & _MASK))
        s.epoch = e
        return s

    def size(self) -> int:
        return len(self.indices)

    def get_index(self, pos: int) -> Optional[int]:
        return self.indices[pos] if 0 <= pos < len(self.indices) else None
