"""DistAdam (Tyr/Optim/DistAdam.lean): bias-corrected AdamW with decoupled weight decay, and its
ZeRO-style distributed step (reduce_scatter(avg) of row shards -> local update -> all_gather of the
parameter and both moments, :185-267; falls back to all-reduce when dim 0 does not divide by the
world size, :201-204).  ``step_sharded`` / ``ShardedEmbeddingAdam`` keep the state sharded and gather
the parameter lazily (:328-453).  The fused single-kernel form is :mod:`tyr_b200.parallel.dp`."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from ..ops import optim_kernels as ok


@dataclass
class Config:
    lr: float = 0.008
    beta1: float = 0.65
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.005
    distributed: bool = False


@dataclass
class ParamState:
    exp_avg: torch.Tensor
    exp_avg_sq: torch.Tensor
    step: int = 0


def init_param_state(param: torch.Tensor) -> ParamState:
    return ParamState(torch.zeros_like(param), torch.zeros_like(param), 0)


def step_single(param: torch.Tensor, grad: torch.Tensor, state: ParamState, cfg: Config, lr_mul: float = 1.0,
                wd_mul: float = 1.0) -> Tuple[torch.Tensor, ParamState]:
    step = state.step + 1
    lr, wd = cfg.lr * lr_mul, cfg.weight_decay * wd_mul
    p = param.detach().clone()
    m, v = state.exp_avg.clone(), state.exp_avg_sq.clone()
    if p.is_cuda and p.dtype == torch.float32 and p.is_contiguous():
        ok.adamw_step_(p, grad.detach().contiguous(), m, v, lr=lr, beta1=cfg.beta1, beta2=cfg.beta2, eps=cfg.eps,
                       weight_decay=wd, step=step)
    else:
        g = grad.detach()
        m = m * cfg.beta1 + g * (1.0 - cfg.beta1)
        v = v * cfg.beta2 + g * g * (1.0 - cfg.beta2)
        bc1, bc2 = 1.0 - cfg.beta1 ** step, 1.0 - cfg.beta2 ** step
        upd = (m / bc1) / ((v / bc2).sqrt() + cfg.eps)
        p = (p - p * (lr * wd) if wd > 0 else p) - upd * lr
    return p.requires_grad_(True), ParamState(m, v, step)


def _dist():
    from .. import distributed as dist
    return dist


def step_distributed(param, grad, state: ParamState, cfg: Config, lr_mul: float = 1.0, wd_mul: float = 1.0):
    """Reduce-scatter the gradient, AdamW on the owned rows, all-gather parameter and moments
    (Tyr/Optim/DistAdam.lean:185-267).  The collectives are those of ``tyr_b200.distributed``: after
    ``distributed.enable_peer_collectives()`` they run on the peer-memory kernels instead of NCCL."""
    dist = _dist()
    if not cfg.distributed or not dist.is_initialized() or dist.get_world_size() <= 1:
        return step_single(param, grad, state, cfg, lr_mul, wd_mul)
    W, rank = dist.get_world_size(), dist.get_rank()
    if param.dim() == 0 or param.shape[0] % W != 0:
        g = dist.all_reduce(grad.detach(), dist.ReduceOp.avg)
        return step_single(param, g, state, cfg, lr_mul, wd_mul)
    rows = param.shape[0] // W
    sl = slice(rank * rows, (rank + 1) * rows)
    g_shard = dist.reduce_scatter(grad.detach(), dist.ReduceOp.avg)
    local = ParamState(state.exp_avg[sl].clone(), state.exp_avg_sq[sl].clone(), state.step)
    p_shard, s_shard = step_single(param.detach()[sl].clone(), g_shard, local, cfg, lr_mul, wd_mul)
    p_full = dist.all_gather(p_shard.detach())
    m_full = dist.all_gather(s_shard.exp_avg)
    v_full = dist.all_gather(s_shard.exp_avg_sq)
    return p_full.requires_grad_(True), ParamState(m_full, v_full, s_shard.step)


@dataclass
class ShardedState:
    """Moments exist only for this rank's row shard."""
    exp_avg: torch.Tensor
    exp_avg_sq: torch.Tensor
    step: int = 0


def step_sharded(param_shard: torch.Tensor, grad_full: torch.Tensor, state: ShardedState, cfg: Config):
    """``param_shard`` holds rows [rank*rows, (rank+1)*rows); returns the updated shard and state."""
    dist = _dist()
    if dist.is_initialized() and dist.get_world_size() > 1:
        g = dist.reduce_scatter(grad_full.detach(), dist.ReduceOp.avg)
    else:
        g = grad_full.detach()
    p, s = step_single(param_shard, g, ParamState(state.exp_avg, state.exp_avg_sq, state.step), cfg)
    return p, ShardedState(s.exp_avg, s.exp_avg_sq, s.step)


class ShardedEmbeddingAdam:
    """Row-sharded embedding table with sharded Adam state; ``gather()`` rebuilds the full table."""

    def __init__(self, full_table: torch.Tensor, cfg: Config):
        dist = _dist()
        self.cfg = cfg
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        if full_table.shape[0] % self.world != 0:
            raise ValueError("embedding rows must divide by the world size")
        rows = full_table.shape[0] // self.world
        self.shard = full_table.detach()[self.rank * rows:(self.rank + 1) * rows].clone()
        self.state = ShardedState(torch.zeros_like(self.shard), torch.zeros_like(self.shard), 0)
        self._cache: Optional[torch.Tensor] = None

    def gather(self) -> torch.Tensor:
        if self._cache is None:
            dist = _dist()
            self._cache = dist.all_gather(self.shard) if self.world > 1 else self.shard
        return self._cache

    def step(self, grad_full: torch.Tensor):
        p, self.state = step_sharded(self.shard, grad_full, self.state, self.cfg)
        self.shard = p.detach()
        self._cache = None
