"""Stiefel-constrained Muon (Tyr/Optim/ManifoldMuon.lean).

Per step: momentum EMA + Nesterov blend on the ambient gradient, an inner solve for a dual
variable Lambda so that the matrix-sign direction of ``G + 2 W (Lambda + Lambda^T)`` is (nearly)
tangent at W (dual ascent :158 or damped fixed point :193; each iteration costs one Polar Express
msign and one residual ``W^T A + A^T W``), tangent projection (:132), normalisation, step with
Muon's aspect-ratio scaling and QR retraction (:241, tall column-wise / wide row-wise)."""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch

from ..manifolds import Stiefel, sym
from . import normuon
from . import polar_express as pe


class SolverKind(enum.Enum):
    dual_ascent = "dualAscent"
    fixed_point = "fixedPoint"


@dataclass
class Config:
    lr: float = 0.02
    momentum: float = 0.95
    num_iters: int = 5
    dual_ascent_steps: int = 2
    dual_ascent_lr: float = 0.1
    solver: SolverKind = SolverKind.dual_ascent
    min_solve_steps: int = 1
    solve_residual_tol: float = 1e-4
    solve_dual_delta_tol: float = 1e-5
    fixed_point_damping: float = 0.5
    distributed: bool = False


@dataclass
class SolveDiagnostics:
    iterations: int = 0
    residual: float = 0.0
    dual_delta: float = 0.0
    dual_objective: float = 0.0
    converged: bool = False
    solver: SolverKind = SolverKind.dual_ascent


@dataclass
class ParamState:
    momentum_buffer: Optional[torch.Tensor] = None
    dual_var: Optional[torch.Tensor] = None
    step: int = 0


def init_param_state(_param=None) -> ParamState:
    return ParamState()


def tangent_project(W, G):
    return G - W @ sym(W.transpose(-1, -2) @ G)


def tangent_residual(W, A):
    return W.transpose(-1, -2) @ A + A.transpose(-1, -2) @ W


def _dual_objective(W, G, lam) -> float:
    adj = G + 2.0 * (W @ (lam + lam.transpose(-1, -2)))
    return -float(torch.linalg.matrix_norm(adj.float(), "nuc"))


def solve_direction(W, G, dual0, cfg: Config):
    lam = dual0
    signed = G
    residual = dual_delta = 1e30
    iters, converged = 0, False
    damp = min(1.0, max(0.0, cfg.fixed_point_damping))
    for i in range(cfg.dual_ascent_steps):
        if converged:
            break
        prev = lam
        adj = G + 2.0 * (W @ (lam + lam.transpose(-1, -2)))
        signed = pe.apply(adj, pe.Config(cfg.num_iters))
        h = tangent_residual(W, signed)
        if cfg.solver is SolverKind.dual_ascent:
            lam = lam + h * cfg.dual_ascent_lr
        else:
            cand = lam - h * cfg.dual_ascent_lr
            lam = lam * (1.0 - damp) + cand * damp
        residual = float(h.norm())
        dual_delta = float((lam - prev).norm())
        iters = i + 1
        converged = (iters >= cfg.min_solve_steps and residual <= cfg.solve_residual_tol
                     and dual_delta <= cfg.solve_dual_delta_tol)
    diag = SolveDiagnostics(iters, residual, dual_delta, _dual_objective(W, G, lam), converged, cfg.solver)
    return signed, lam, diag


def retract_stiefel(W):
    return Stiefel().project(W)


def step_single_with_diagnostics(param, grad, state: ParamState, cfg: Config, lr_mul: float = 1.0):
    g = grad.detach()
    W = param.detach()
    m, n = W.shape
    new_mom = normuon.update_momentum(g, state.momentum_buffer, cfg.momentum)
    nesterov = g * (1.0 - cfg.momentum) + new_mom * cfg.momentum
    dual0 = state.dual_var if state.dual_var is not None else torch.zeros(n, n, dtype=W.dtype, device=W.device)
    if cfg.dual_ascent_steps == 0:
        signed = pe.apply(nesterov, pe.Config(cfg.num_iters))
        diag = SolveDiagnostics(0, float(tangent_residual(W, signed).norm()), 0.0,
                                _dual_objective(W, nesterov, dual0), True, cfg.solver)
        dual = dual0
    else:
        signed, dual, diag = solve_direction(W, nesterov, dual0, cfg)
    tdir = tangent_project(W, signed)
    fn = float(tdir.norm())
    unit = tdir if fn == 0.0 else tdir / fn
    eff_lr = cfg.lr * lr_mul * normuon.aspect_ratio_scale((m, n))
    new_param = retract_stiefel(W - unit * eff_lr).detach().requires_grad_(True)
    return new_param, ParamState(new_mom, dual, state.step + 1), diag


def step_single(param, grad, state: ParamState, cfg: Config, lr_mul: float = 1.0):
    p, s, _ = step_single_with_diagnostics(param, grad, state, cfg, lr_mul)
    return p, s


def step_group_local(params, grads, states, cfg: Config, lr_mul: float = 1.0):
    out_p, out_s = [], []
    for i, p in enumerate(params):
        g = grads[i] if i < len(grads) and grads[i] is not None else torch.zeros_like(p)
        s = states[i] if i < len(states) else init_param_state(p)
        np_, ns = step_single(p, g, s, cfg, lr_mul)
        out_p.append(np_)
        out_s.append(ns)
    return out_p, out_s


def step_distributed_group(params, grads, states, cfg: Config, lr_mul: float = 1.0):
    """All-reduce(avg) the gradients, then the local manifold step (ManifoldMuon.lean:342-367)."""
    from .. import distributed as dist
    if not params:
        return params, states
    if not cfg.distributed or not dist.is_initialized() or dist.get_world_size() <= 1:
        return step_group_local(params, grads, states, cfg, lr_mul)
    reduced = [dist.all_reduce((grads[i] if i < len(grads) and grads[i] is not None else torch.zeros_like(p)).detach(),
                               dist.ReduceOp.avg) for i, p in enumerate(params)]
    return step_group_local(params, reduced, states, cfg, lr_mul)


def benchmark_local_step(m: int, n: int, iters: int = 3, device="cpu") -> float:
    """Mean step latency in ms for an m x n Stiefel parameter (ManifoldMuon.lean:370)."""
    W = retract_stiefel(torch.randn(m, n, device=device))
    st = init_param_state()
    cfg = Config()
    t0 = time.perf_counter()
    for _ in range(iters):
        W, st = step_single(W, torch.randn(m, n, device=device), st, cfg)
    if torch.device(device).type == "cuda":
        torch.cuda.synchronize()
    return (time.perf_counter() - t0) * 1e3 / iters
