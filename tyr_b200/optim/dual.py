"""DualOptimizer: matrices vs everything else (Tyr/Optim/DualOptimizer.lean).

Matrix parameters take a norm-constrained update - NorMuon, or a manifold variant (Stiefel via
ManifoldMuon, Orthogonal / Grassmann through the generic dual-map step :412) - while embeddings,
heads and scalars take DistAdam.  ``dim_lr_scale`` is (d / ref)^-0.5 (:105); labels map to groups
(:129-206); a matrix state whose kind does not match the configured optimizer is an error (:442).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field, replace
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import manifolds as mf
from . import distadam, manifold_muon, normuon
from .normuon import ParamLabel


class MatrixOptimizerKind(enum.Enum):
    nor_muon = "norMuon"
    manifold_muon = "manifoldMuon"


class MatrixManifoldFamily(enum.Enum):
    stiefel = "stiefel"
    orthogonal = "orthogonal"
    grassmann = "grassmann"


class ParamGroup(enum.Enum):
    matrix = "matrix"
    embedding = "embedding"
    unembedding = "unembedding"
    scalar = "scalar"


@dataclass
class Config:
    matrix_lr: float = 0.02
    embedding_lr: float = 0.3
    unembedding_lr: float = 0.004
    scalar_lr: float = 0.004
    matrix_weight_decay: float = 0.0
    adam_beta1: float = 0.8
    adam_beta2: float = 0.95
    adam_eps: float = 1e-10
    adam_weight_decay: float = 0.0
    momentum: float = 0.95
    num_iters: int = 5
    model_dim: int = 768
    reference_dim: int = 768
    matrix_optimizer: MatrixOptimizerKind = MatrixOptimizerKind.nor_muon
    manifold_family: MatrixManifoldFamily = MatrixManifoldFamily.stiefel
    distributed: bool = False
    world_size: int = 1


def dim_lr_scale(cfg: Config) -> float:
    return (cfg.model_dim / cfg.reference_dim) ** -0.5


def to_muon_config(cfg: Config) -> normuon.Config:
    return normuon.Config(lr=cfg.matrix_lr, weight_decay=cfg.matrix_weight_decay, momentum=cfg.momentum,
                          num_iters=cfg.num_iters, distributed=cfg.distributed, world_size=cfg.world_size)


def to_adam_config(cfg: Config) -> distadam.Config:
    return distadam.Config(lr=1.0, beta1=cfg.adam_beta1, beta2=cfg.adam_beta2, eps=cfg.adam_eps,
                           weight_decay=cfg.adam_weight_decay, distributed=cfg.distributed)


def label_to_group(label: ParamLabel) -> ParamGroup:
    if label in (ParamLabel.attn, ParamLabel.mlp, ParamLabel.smear_gate, ParamLabel.attn_gate):
        return ParamGroup.matrix
    if label in (ParamLabel.embed, ParamLabel.value_embed):
        return ParamGroup.embedding
    if label is ParamLabel.lm_head:
        return ParamGroup.unembedding
    return ParamGroup.scalar


def group_lr(cfg: Config, group: ParamGroup) -> float:
    if group is ParamGroup.matrix:
        return cfg.matrix_lr
    s = dim_lr_scale(cfg)
    return {ParamGroup.embedding: cfg.embedding_lr, ParamGroup.unembedding: cfg.unembedding_lr,
            ParamGroup.scalar: cfg.scalar_lr}[group] * s


def group_wd_mul(cfg: Config, group: ParamGroup) -> float:
    return 1.0 if group is ParamGroup.matrix else 0.0


@dataclass
class MatrixParamState:
    """Tagged state: which optimizer produced it."""
    kind: MatrixOptimizerKind
    family: Optional[MatrixManifoldFamily] = None
    muon: Optional[normuon.ParamState] = None
    manifold: Optional[manifold_muon.ParamState] = None
    momentum_buffer: Optional[torch.Tensor] = None
    step: int = 0


def init_matrix_state(cfg: Config) -> MatrixParamState:
    if cfg.matrix_optimizer is MatrixOptimizerKind.nor_muon:
        return MatrixParamState(cfg.matrix_optimizer, None, normuon.init_param_state())
    if cfg.manifold_family is MatrixManifoldFamily.stiefel:
        return MatrixParamState(cfg.matrix_optimizer, cfg.manifold_family, None, manifold_muon.init_param_state())
    return MatrixParamState(cfg.matrix_optimizer, cfg.manifold_family)


def _family_manifold(f: MatrixManifoldFamily) -> mf.Manifold:
    return {MatrixManifoldFamily.stiefel: mf.Stiefel(), MatrixManifoldFamily.orthogonal: mf.Orthogonal(),
            MatrixManifoldFamily.grassmann: mf.Grassmann()}[f]


def step_generic_manifold_single(param, grad, state: MatrixParamState, cfg: Config, lr_mul: float = 1.0):
    """Nesterov momentum + ``DualMapGeometry.dualMapStep`` under the spectral norm (:412)."""
    man = _family_manifold(state.family)
    geo = mf.SpectralDualMap(man, cfg.num_iters)
    g = grad.detach()
    mom = normuon.update_momentum(g, state.momentum_buffer, cfg.momentum)
    nesterov = g * (1.0 - cfg.momentum) + mom * cfg.momentum
    lr = cfg.matrix_lr * lr_mul * normuon.aspect_ratio_scale(param.shape)
    new = geo.dual_map_step(param.detach(), nesterov, lr)
    return new.detach().requires_grad_(True), replace(state, momentum_buffer=mom, step=state.step + 1)


def step_matrix_single(param, grad, state: MatrixParamState, cfg: Config, lr_mul: float = 1.0, wd_mul: float = 1.0):
    if state.kind is not cfg.matrix_optimizer or (state.kind is MatrixOptimizerKind.manifold_muon
                                                  and state.family is not cfg.manifold_family):
        raise RuntimeError(f"DualOptimizer: parameter state was produced by {state.kind.value}"
                           f"/{state.family.value if state.family else '-'} but the configuration selects "
                           f"{cfg.matrix_optimizer.value}/{cfg.manifold_family.value}")
    if state.kind is MatrixOptimizerKind.nor_muon:
        p, s = normuon.step_single(param, grad, state.muon, to_muon_config(cfg), lr_mul, wd_mul)
        return p, replace(state, muon=s, step=state.step + 1)
    if state.family is MatrixManifoldFamily.stiefel:
        mcfg = manifold_muon.Config(lr=cfg.matrix_lr, momentum=cfg.momentum, num_iters=cfg.num_iters)
        p, s = manifold_muon.step_single(param, grad, state.manifold, mcfg, lr_mul)
        return p, replace(state, manifold=s, step=state.step + 1)
    return step_generic_manifold_single(param, grad, state, cfg, lr_mul)


def step_matrix_group_local(params, grads, states, cfg: Config, lr_mul: float = 1.0, wd_mul: float = 1.0):
    out = [step_matrix_single(p, g, s, cfg, lr_mul, wd_mul) for p, g, s in zip(params, grads, states)]
    return [o[0] for o in out], [o[1] for o in out]


def step_matrix_group_distributed(params, grads, states, cfg: Config, lr_mul: float = 1.0, wd_mul: float = 1.0):
    from .. import distributed as dist
    if cfg.distributed and dist.is_initialized() and dist.get_world_size() > 1:
        grads = [dist.all_reduce(g.detach(), dist.ReduceOp.avg) for g in grads]
    return step_matrix_group_local(params, grads, states, cfg, lr_mul, wd_mul)


@dataclass
class MatrixBackendOps:
    """Closures a trainer uses without knowing which matrix optimizer is active (:577-609)."""
    init_state: callable
    step_group: callable

    @staticmethod
    def for_config(cfg: Config) -> "MatrixBackendOps":
        return MatrixBackendOps(lambda _p=None: init_matrix_state(cfg),
                                lambda ps, gs, ss, lr_mul=1.0, wd_mul=1.0:
                                step_matrix_group_distributed(ps, gs, ss, cfg, lr_mul, wd_mul))


class DualOptimizer:
    """Convenience driver over labelled parameters."""

    def __init__(self, params: Dict[str, Tuple[torch.Tensor, ParamLabel]], cfg: Config):
        self.cfg = cfg
        self.labels = {k: lab for k, (_, lab) in params.items()}
        self.matrix_states = {k: init_matrix_state(cfg) for k, (_, lab) in params.items()
                              if label_to_group(lab) is ParamGroup.matrix}
        self.adam_states = {k: distadam.init_param_state(p) for k, (p, lab) in params.items()
                            if label_to_group(lab) is not ParamGroup.matrix}

    def step(self, params: Dict[str, torch.Tensor], grads: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        out = {}
        acfg = to_adam_config(self.cfg)
        for k, p in params.items():
            group = label_to_group(self.labels[k])
            g = grads.get(k)
            if g is None:
                out[k] = p
                continue
            if group is ParamGroup.matrix:
                out[k], self.matrix_states[k] = step_matrix_single(p, g, self.matrix_states[k], self.cfg, 1.0,
                                                                   group_wd_mul(self.cfg, group))
            else:
                out[k], self.adam_states[k] = distadam.step_distributed(
                    p, g, self.adam_states[k], replace(acfg, lr=group_lr(self.cfg, group)))
        return out
