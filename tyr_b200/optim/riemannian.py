"""RiemannianSGD and RiemannianTreeSGD (Tyr/Optim/RiemannianSGD.lean, RiemannianTreeSGD.lean).

Natural-gradient-like steps where the metric is a low-rank factor plus a diagonal mass and the
linear system is solved with the Woodbury identity.

* ``step_mse`` / ``step_sequential_mse`` operate on :class:`tyr_b200.modular.RiemannianLinear`
  stacks (identity output metric, half squared error).
* ``TreeMetricFactor`` holds ``rank`` parameter-tree rows; ``step_cross_entropy`` builds the exact
  Fisher factor from one VJP per (position, class) output row (rank = batch*seq*vocab: tiny shapes
  only), ``step_cross_entropy_sampled_fisher`` samples labels from the model instead.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch

from .. import modular as md
from ..struct import tree as ts


@dataclass
class StepResult:
    params: object
    prediction: torch.Tensor
    input_factor: Optional[md.MetricFactor] = None
    input_cotangent: Optional[torch.Tensor] = None
    diagnostics: Optional[list] = None
    loss: float = 0.0


def step_mse(layer: md.RiemannianLinear, x, target, lr: float) -> StepResult:
    pred, tape = layer.forward_with_tape(x)
    residual = pred - target
    loss = 0.5 * float((residual * residual).sum())
    new, f, c, d = layer.backward_leaf_step(tape, md.MetricFactor.identity(layer.out_dim), residual, lr)
    return StepResult(new, pred, f, c, [d], loss)


def step_sequential_with_factor(layers, x, output_factor: md.MetricFactor, output_cotangent, lr: float) -> StepResult:
    pred, tapes = md.sequential_forward_with_tape(layers, x)
    new, f, c, d = md.sequential_backward_metric_step(layers, tapes, output_factor, output_cotangent, lr)
    return StepResult(new, pred, f, c, d)


def step_sequential_mse(layers, x, target, lr: float) -> StepResult:
    pred, tapes = md.sequential_forward_with_tape(layers, x)
    residual = pred - target
    r = step_sequential_with_factor(layers, x, md.MetricFactor.identity(pred.shape[0]), residual, lr)
    r.loss = 0.5 * float((residual * residual).sum())
    return r


# ---- tree version ---------------------------------------------------------------------------------------------------
def _dot(a, b) -> float:
    return float(sum((ts._raw(x).float() * ts._raw(y).float()).sum() for x, y in zip(ts.leaves(a), ts.leaves(b))))


def _axpy(a, x, y):
    """a*x + y over trees."""
    return ts.zip_with(lambda u, v: ts._like(u, ts._raw(u) * a + ts._raw(v)), x, y)


@dataclass
class StepDiagnostics:
    grad_norm: float = 0.0
    natural_norm: float = 0.0
    clipped: bool = False


@dataclass
class TreeMetricFactor:
    """``rank`` rows, each a parameter-shaped tree: K v = [<row_i, v>]_i."""
    rows: List[object]

    @property
    def rank(self) -> int:
        return len(self.rows)

    def apply(self, v) -> torch.Tensor:
        return torch.tensor([_dot(r, v) for r in self.rows], dtype=torch.float64)

    def apply_transpose(self, y: torch.Tensor, like):
        out = ts.tree_map(lambda t: ts._like(t, torch.zeros_like(ts._raw(t))), like)
        for yi, r in zip(y.tolist(), self.rows):
            out = _axpy(yi, r, out)
        return out

    def woodbury_inner(self, inv_mass: float) -> torch.Tensor:
        r = self.rank
        inner = torch.eye(r, dtype=torch.float64)
        for i in range(r):
            for j in range(i, r):
                v = inv_mass * _dot(self.rows[i], self.rows[j])
                inner[i, j] += v
                if i != j:
                    inner[j, i] += v
        return inner

    def apply_regularized(self, mass: float, v):
        return _axpy(1.0, self.apply_transpose(self.apply(v), v), ts.scale(v, mass))

    def solve_woodbury(self, mass: float, b):
        """(mass I + K^T K)^-1 b."""
        inv = 1.0 / mass
        y = torch.linalg.solve(self.woodbury_inner(inv), self.apply(b) * inv)
        corr = self.apply_transpose(y, b)
        return ts.zip_with(lambda u, c: ts._like(u, ts._raw(u) * inv - ts._raw(c) * inv), b, corr)


def _clip(tree, max_norm: Optional[float]):
    if not max_norm:
        return tree, False
    n = _dot(tree, tree) ** 0.5
    if n <= max_norm:
        return tree, False
    return ts.scale(tree, max_norm / n), True


def step_with_factor_and_mass(params, grad, factor: TreeMetricFactor, mass: float, lr: float,
                              max_step_norm: Optional[float] = None):
    nat = factor.solve_woodbury(mass, grad)
    nat, clipped = _clip(nat, max_step_norm)
    new = ts.zip_with(lambda p, d: ts._like(p, (ts._raw(p) - lr * ts._raw(d)).detach()), params, nat)
    return new, StepDiagnostics(_dot(grad, grad) ** 0.5, _dot(nat, nat) ** 0.5, clipped)


def step_with_factor(params, grad, factor: TreeMetricFactor, lr: float):
    return step_with_factor_and_mass(params, grad, factor, 1.0, lr)


def _vjp_rows(logits_fn: Callable, params, weights: torch.Tensor):
    """One VJP per row of ``weights`` ([rank, *logits.shape])."""
    leaves = ts.leaves(params, include_frozen=False)
    fresh = [ts._like(t, ts._raw(t).detach().clone().requires_grad_(True)) for t in leaves]
    p2 = ts.with_leaves(params, fresh, include_frozen=False)
    logits = logits_fn(p2)
    rows = []
    for w in weights:
        gs = torch.autograd.grad(logits, [ts._raw(t) for t in fresh], w.to(logits.dtype), retain_graph=True, allow_unused=True)
        rows.append(ts.with_leaves(params, [ts._like(t, g if g is not None else torch.zeros_like(ts._raw(t)))
                                            for t, g in zip(fresh, gs)], include_frozen=False))
    return logits.detach(), rows, p2


def step_cross_entropy(logits_fn: Callable, params, targets: torch.Tensor, lr: float, mass: float = 1e-3,
                       max_step_norm: Optional[float] = None):
    """Exact Fisher: rows sqrt(p_c) (e_c - p) per position and class, scaled by 1/sqrt(N)."""
    with torch.no_grad():
        base = logits_fn(params)
    N, V = base.shape
    p = torch.softmax(base.float(), -1)
    weights = []
    for n in range(N):
        for c in range(V):
            w = torch.zeros(N, V)
            w[n] = -p[n] * p[n, c].sqrt()
            w[n, c] += p[n, c].sqrt()
            weights.append(w / N ** 0.5)
    _, rows, _ = _vjp_rows(logits_fn, params, torch.stack(weights))
    g_w = (p - torch.nn.functional.one_hot(targets, V).float()) / N
    _, grad_rows, _ = _vjp_rows(logits_fn, params, g_w.unsqueeze(0))
    loss = float(torch.nn.functional.cross_entropy(base.float(), targets))
    new, diag = step_with_factor_and_mass(params, grad_rows[0], TreeMetricFactor(rows), mass, lr, max_step_norm)
    return new, loss, diag


def step_cross_entropy_sampled_fisher(logits_fn: Callable, params, targets: torch.Tensor, lr: float,
                                      samples: int = 4, mass: float = 1e-3, generator=None,
                                      max_step_norm: Optional[float] = None):
    with torch.no_grad():
        base = logits_fn(params)
    N, V = base.shape
    p = torch.softmax(base.float(), -1)
    weights = []
    for _ in range(samples):
        y = torch.multinomial(p, 1, generator=generator).squeeze(-1)
        weights.append((p - torch.nn.functional.one_hot(y, V).float()) / (N * samples) ** 0.5)
    _, rows, _ = _vjp_rows(logits_fn, params, torch.stack(weights))
    g_w = (p - torch.nn.functional.one_hot(targets, V).float()) / N
    _, grad_rows, _ = _vjp_rows(logits_fn, params, g_w.unsqueeze(0))
    loss = float(torch.nn.functional.cross_entropy(base.float(), targets))
    new, diag = step_with_factor_and_mass(params, grad_rows[0], TreeMetricFactor(rows), mass, lr, max_step_norm)
    return new, loss, diag
