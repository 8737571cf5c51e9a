"""NorMuon / Muon (Tyr/Optim/NorMuon.lean).

``step_single`` keeps the reference's order: momentum EMA on raw gradients -> Nesterov blend ->
(zero-gradient guard) -> decoupled weight decay -> ``muon_orthogonalize`` in bf16 -> scale in bf16
-> cast back -> subtract.  ``step_distributed_owner`` (all-reduce, owner updates, two broadcasts)
and ``step_distributed_group`` (block-cyclic ownership with reduce_scatter / all_gather lists,
:346-425) run over :mod:`tyr_b200.distributed`; the fused NVLink form of the group step lives in
:mod:`tyr_b200.parallel.dp`.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

from ..ops import polar


class ParamLabel(enum.Enum):
    smear_gate = "smearGate"
    attn_gate = "attnGate"
    attn = "attn"
    mlp = "mlp"
    embed = "embed"
    lm_head = "lmHead"
    scalars = "scalars"
    value_embed = "valueEmbed"


@dataclass
class LabeledParam:
    tensor: torch.Tensor
    label: ParamLabel
    lr_mul: float = 1.0
    wd_mul: float = 1.0


@dataclass
class Config:
    lr: float = 0.023
    weight_decay: float = 1.2
    momentum: float = 0.95
    beta2: float = 0.95
    num_iters: int = 5
    distributed: bool = False
    world_size: int = 1


@dataclass
class ParamState:
    momentum_buffer: Optional[torch.Tensor] = None
    second_moment: Optional[torch.Tensor] = None
    step: int = 0


def init_param_state(_param=None) -> ParamState:
    return ParamState()


def update_momentum(g: torch.Tensor, buf: Optional[torch.Tensor], momentum: float) -> torch.Tensor:
    """buf_t = momentum * buf_{t-1} + (1 - momentum) * g."""
    if buf is None:
        return g * (1.0 - momentum)
    return buf * momentum + g * (1.0 - momentum)


def aspect_ratio_scale(shape: Sequence[int]) -> float:
    if len(shape) >= 2 and shape[-2] > shape[-1]:
        return math.sqrt(shape[-2] / shape[-1])
    return 1.0


def step_single(param: torch.Tensor, grad: torch.Tensor, state: ParamState, cfg: Config,
                lr_mul: float = 1.0, wd_mul: float = 1.0) -> Tuple[torch.Tensor, ParamState]:
    g = grad.detach()
    new_mom = update_momentum(g, state.momentum_buffer, cfg.momentum)
    nesterov = g * (1.0 - cfg.momentum) + new_mom * cfg.momentum
    eff_lr = cfg.lr * lr_mul * aspect_ratio_scale(param.shape)
    wd = cfg.weight_decay * wd_mul
    p = param.detach()
    decayed = p - p * (eff_lr * wd) if wd > 0.0 else p
    if nesterov.numel() == 0 or float(nesterov.abs().max()) == 0.0:
        update = nesterov
    else:
        orth = polar.muon_orthogonalize(nesterov, cfg.num_iters)
        update = (orth.detach() * eff_lr).to(param.dtype)
    new_param = (decayed - update).detach().requires_grad_(True)
    return new_param, ParamState(new_mom, None, state.step + 1)


def _dist():
    from .. import distributed as dist
    return dist


def step_distributed_owner(param, grad, state: ParamState, cfg: Config, lr_mul: float, wd_mul: float,
                           owner_rank: int):
    dist = _dist()
    if not cfg.distributed or not dist.is_initialized() or dist.get_world_size() <= 1:
        return step_single(param, grad, state, cfg, lr_mul, wd_mul)
    rank = dist.get_rank()
    g = dist.all_reduce(grad.detach(), dist.ReduceOp.avg)
    if rank == owner_rank:
        new_p, new_s = step_single(param, g, state, cfg, lr_mul, wd_mul)
    else:
        new_p, new_s = param, state
    synced = dist.broadcast(new_p.detach() if rank == owner_rank else param.detach(), owner_rank)
    mom = new_s.momentum_buffer if (rank == owner_rank and new_s.momentum_buffer is not None) else torch.zeros_like(synced)
    mom = dist.broadcast(mom, owner_rank)
    return synced.detach().requires_grad_(True), ParamState(mom, new_s.second_moment, state.step + 1)


def step_group_local(params, grads, states, cfg: Config, lr_mul: float = 1.0, wd_mul: float = 1.0):
    out_p, out_s = [], []
    for i, p in enumerate(params):
        g = grads[i] if i < len(grads) and grads[i] is not None else torch.zeros_like(p)
        s = states[i] if i < len(states) else init_param_state(p)
        np_, ns = step_single(p, g, s, cfg, lr_mul, wd_mul)
        out_p.append(np_)
        out_s.append(ns)
    return out_p, out_s


def step_distributed_group(params: List[torch.Tensor], grads: List[torch.Tensor], states: List[ParamState],
                           cfg: Config, lr_mul: float = 1.0, wd_mul: float = 1.0):
    """Parameters are processed in blocks of ``world``; rank r owns parameter ``base + r``.
    Gradients are averaged with reduce_scatter over per-rank lists (zero-padded tail blocks), the
    owner steps, parameters AND momentum are replicated with all_gather (Tyr/Optim/NorMuon.lean:346-425).  The collectives
    are those of ``tyr_b200.distributed``: after ``distributed.enable_peer_collectives()`` they run on the peer-memory
    kernels instead of NCCL."""
    dist = _dist()
    if not params:
        return params, states
    if not cfg.distributed or not dist.is_initialized() or dist.get_world_size() <= 1:
        return step_group_local(params, grads, states, cfg, lr_mul, wd_mul)
    W, rank = dist.get_world_size(), dist.get_rank()
    out_p: List[torch.Tensor] = [None] * len(params)
    out_s: List[ParamState] = [None] * len(params)
    proto = params[0]
    for base in range(0, len(params), W):
        g_list = []
        for r in range(W):
            i = base + r
            g_list.append(grads[i].detach() if i < len(params) and grads[i] is not None else torch.zeros_like(proto))
        g_own = dist.reduce_scatter_list(g_list, dist.ReduceOp.avg)
        mine = base + rank
        if mine < len(params):
            st = states[mine] if mine < len(states) else init_param_state(params[mine])
            new_p, new_s = step_single(params[mine], g_own, st, cfg, lr_mul, wd_mul)
            p_send = new_p.detach()
            m_send = new_s.momentum_buffer
        else:
            p_send, m_send = torch.zeros_like(proto), torch.zeros_like(proto)
        p_all = dist.all_gather_list(p_send)
        m_all = dist.all_gather_list(m_send)
        for r in range(W):
            i = base + r
            if i < len(params):
                out_p[i] = p_all[r].detach().requires_grad_(True)
                prev = states[i] if i < len(states) else init_param_state(params[i])
                out_s[i] = ParamState(m_all[r], None, prev.step + 1)
    return out_p, out_s


def step_adam_like(param, grad, exp_avg, exp_avg_sq, step: int, lr: float, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.0):
    """Adam fallback for labels that do not take the Muon path (NorMuon.lean:439)."""
    g = grad.detach()
    exp_avg = exp_avg * beta1 + g * (1 - beta1)
    exp_avg_sq = exp_avg_sq * beta2 + g * g * (1 - beta2)
    bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
    upd = (exp_avg / bc1) / ((exp_avg_sq / bc2).sqrt() + eps)
    p = param.detach()
    p = p - p * (lr * wd) if wd > 0 else p
    return (p - lr * upd).requires_grad_(True), exp_avg, exp_avg_sq


LABEL_LR_MUL = {ParamLabel.smear_gate: 1.0, ParamLabel.attn_gate: 1.0, ParamLabel.attn: 1.0, ParamLabel.mlp: 1.0,
                ParamLabel.embed: 1.0, ParamLabel.lm_head: 1.0, ParamLabel.scalars: 1.0, ParamLabel.value_embed: 1.0}
LABEL_WD_MUL = {ParamLabel.smear_gate: 0.0, ParamLabel.attn_gate: 0.0, ParamLabel.attn: 1.0, ParamLabel.mlp: 1.0,
                ParamLabel.embed: 0.0, ParamLabel.lm_head: 0.0, ParamLabel.scalars: 0.0, ParamLabel.value_embed: 0.0}


def label_lr_mul(label: ParamLabel) -> float:
    return LABEL_LR_MUL[label]


def label_wd_mul(label: ParamLabel) -> float:
    return LABEL_WD_MUL[label]


def get_momentum(step: int, total_steps: int = 0, base_momentum: float = 0.95, warmup_steps: int = 300,
                 cooldown_steps: int = 50) -> float:
    """0.85 -> base over ``warmup_steps``, then constant (NorMuon.lean:513-523)."""
    if step < warmup_steps:
        return 0.85 + (step / warmup_steps) * (base_momentum - 0.85)
    return base_momentum
