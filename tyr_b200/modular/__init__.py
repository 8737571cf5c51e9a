"""Modular norms and Riemannian modules (Tyr/Modular/*.lean).

* ``NormedModule`` protocol (Norm.lean:47): ``norm``, ``dual_norm``, input sensitivity ``nu``,
  weight sensitivity ``mu``, ``normalize`` / ``normalize_dual``; ``normalized_update`` is the core
  modular optimisation step  dw = -lr * normalize_dual(grad).
* Atoms (Atomic.lean): ``Linear`` under the RMS->RMS operator norm (spectral norm scaled by
  sqrt(in/out), dual = nuclear), ``Embedding`` (max row RMS norm).
* ``Sequential`` composition (Compose.lean:32): nu multiplies, norms combine by max of
  downstream-scaled norms.
* LR budget allocation from sensitivities (Budget.lean:6-76).
* ``MetricFactor`` / ``DiagonalMass`` with Woodbury solves (MetricFactor.lean:8-124).
* ``ManifoldLinear`` (Stiefel / Grassmann / Orthogonal) and ``HyperbolicVector`` parameters with
  dual-map updates (Manifold.lean:34-375), ``RiemannianModule`` local linearisation and the
  tape-based forward/backward metric step for linear layers (RiemannianModule.lean:15-292).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

import torch

from .. import manifolds as mf


# ---- normed modules -------------------------------------------------------------------------------------
class NormedModule:
    def norm(self) -> float: raise NotImplementedError
    def dual_norm(self, grad) -> float: raise NotImplementedError
    def nu(self) -> float: return 1.0
    def mu(self) -> float: return 1.0
    def normalize(self): raise NotImplementedError
    def normalize_dual(self, grad): raise NotImplementedError

    def is_well_normed(self) -> bool:
        return self.norm() <= 1.0 + 1e-6

    def lipschitz_constant(self) -> float:
        return self.nu() * self.mu()

    def normalized_update(self, lr: float, grad):
        return self.scale_grad(self.normalize_dual(grad), -lr)

    @staticmethod
    def scale_grad(g, s: float):
        return g * s if isinstance(g, torch.Tensor) else type(g)(x * s for x in g)


class Linear(NormedModule):
    """y = x W^T with the RMS->RMS operator norm  ||W|| = sqrt(in/out) * sigma_max(W)."""

    def __init__(self, weight: torch.Tensor):
        self.weight = weight

    @staticmethod
    def init(in_dim: int, out_dim: int, generator=None) -> "Linear":
        w = torch.randn(out_dim, in_dim, generator=generator)
        return Linear(w).normalize()

    @property
    def _scale(self) -> float:
        out_dim, in_dim = self.weight.shape
        return math.sqrt(in_dim / out_dim)

    def forward(self, x):
        return x @ self.weight.T

    def norm(self) -> float:
        return self._scale * float(torch.linalg.matrix_norm(self.weight.float(), 2))

    def dual_norm(self, grad) -> float:
        return float(torch.linalg.matrix_norm(grad.float(), "nuc")) / self._scale

    def nu(self) -> float:
        return self.norm()

    def normalize(self) -> "Linear":
        n = self.norm()
        return Linear(self.weight / n if n > 0 else self.weight)

    def normalize_dual(self, grad):
        """Steepest direction under the spectral norm: msign(grad), scaled to unit modular norm."""
        u, _, vh = torch.linalg.svd(grad.float(), full_matrices=False)
        return ((u @ vh) / self._scale).to(grad.dtype)


class Embedding(NormedModule):
    """Rows live on the RMS unit ball: norm = max row RMS norm."""

    def __init__(self, table: torch.Tensor):
        self.table = table

    @staticmethod
    def init(vocab: int, dim: int, generator=None) -> "Embedding":
        return Embedding(torch.randn(vocab, dim, generator=generator)).normalize()

    def forward(self, idx):
        return torch.nn.functional.embedding(idx, self.table)

    def _rms(self, t):
        return t.float().pow(2).mean(-1).sqrt()

    def norm(self) -> float:
        return float(self._rms(self.table).max())

    def dual_norm(self, grad) -> float:
        return float(self._rms(grad).sum())

    def nu(self) -> float:
        return 1.0

    def normalize(self) -> "Embedding":
        return Embedding(self.table / self._rms(self.table).clamp_min(1e-12).unsqueeze(-1))

    def normalize_dual(self, grad):
        return grad / self._rms(grad).clamp_min(1e-12).unsqueeze(-1)


class Sequential(NormedModule):
    """m2 after m1."""

    def __init__(self, m1: NormedModule, m2: NormedModule):
        self.m1, self.m2 = m1, m2

    def forward(self, x):
        return self.m2.forward(self.m1.forward(x))

    def norm(self) -> float:
        return max(self.m1.norm() * self.m2.nu(), self.m2.norm())

    def dual_norm(self, grad) -> float:
        g1, g2 = grad
        return self.m1.dual_norm(g1) / max(self.m2.nu(), 1e-12) + self.m2.dual_norm(g2)

    def nu(self) -> float:
        return self.m1.nu() * self.m2.nu()

    def mu(self) -> float:
        return self.m1.mu() * self.m2.nu() + self.m2.mu()

    def normalize(self) -> "Sequential":
        return Sequential(self.m1.normalize(), self.m2.normalize())

    def normalize_dual(self, grad):
        g1, g2 = grad
        return (self.m1.normalize_dual(g1), self.m2.normalize_dual(g2))


def compose(m1, m2) -> Sequential:
    return Sequential(m1, m2)


# ---- LR budget ------------------------------------------------------------------------------------------------
@dataclass
class BudgetConfig:
    min_sensitivity: float = 1e-3
    max_sensitivity: float = 1e3
    min_multiplier: float = 0.1
    max_multiplier: float = 10.0


def sanitize_sensitivity(cfg: BudgetConfig, x: float) -> float:
    if not math.isfinite(x) or x <= 0:
        return 1.0
    return min(cfg.max_sensitivity, max(cfg.min_sensitivity, x))


def multiplier_from_sensitivity(cfg: BudgetConfig, sensitivity: float) -> float:
    m = 1.0 / sanitize_sensitivity(cfg, sensitivity)
    return min(cfg.max_multiplier, max(cfg.min_multiplier, m))


def sequential_downstream_scales(modules: Sequence[NormedModule]) -> List[float]:
    """For layer i: product of nu of every later layer (how much an update is amplified)."""
    out, acc = [], 1.0
    for m in reversed(modules):
        out.append(acc)
        acc *= m.nu()
    return list(reversed(out))


def budgeted_sequential_lrs(base_lr: float, modules: Sequence[NormedModule], cfg: BudgetConfig = BudgetConfig()) -> List[float]:
    return [base_lr * multiplier_from_sensitivity(cfg, s) for s in sequential_downstream_scales(modules)]


@dataclass
class GroupBudget:
    matrix: float = 1.0
    embedding: float = 1.0
    unembedding: float = 1.0
    scalar: float = 1.0

    def apply_to_base_lr(self, base_lr: float) -> "GroupBudget":
        return GroupBudget(self.matrix * base_lr, self.embedding * base_lr, self.unembedding * base_lr, self.scalar * base_lr)

    @staticmethod
    def of_sensitivities(cfg: BudgetConfig, matrix: float, embedding: float, unembedding: float, scalar: float):
        f = lambda s: multiplier_from_sensitivity(cfg, s)
        return GroupBudget(f(matrix), f(embedding), f(unembedding), f(scalar))


# ---- metric factors -------------------------------------------------------------------------------------------
@dataclass
class DiagonalMass:
    diag: torch.Tensor

    @staticmethod
    def ones(dim: int, device="cpu"): return DiagonalMass(torch.ones(dim, device=device))
    @staticmethod
    def of_scalar(dim: int, v: float, device="cpu"): return DiagonalMass(torch.full((dim,), v, device=device))
    def to_matrix(self): return torch.diagflat(self.diag)
    def inv_diag(self): return 1.0 / self.diag
    def inv_matrix(self): return torch.diagflat(self.inv_diag())
    def apply(self, x): return self.diag * x
    def apply_inv(self, x): return x / self.diag


@dataclass
class MetricFactor:
    """K in R^{rank x dim}; the metric is K^T K (optionally + a diagonal mass)."""
    matrix: torch.Tensor

    @staticmethod
    def identity(dim: int, device="cpu"): return MetricFactor(torch.eye(dim, device=device))
    @staticmethod
    def of_matrix(m): return MetricFactor(m)
    def pullback(self, A): return MetricFactor(self.matrix @ A)
    def gram(self): return self.matrix.T @ self.matrix
    def dense_metric(self, D: DiagonalMass): return D.to_matrix() + self.gram()
    def apply(self, x): return self.matrix @ x
    def apply_transpose(self, y): return self.matrix.T @ y
    def apply_regularized(self, D: DiagonalMass, x): return D.apply(x) + self.apply_transpose(self.apply(x))

    def woodbury_inner(self, D: DiagonalMass):
        r = self.matrix.shape[0]
        return torch.eye(r, dtype=self.matrix.dtype, device=self.matrix.device) + (self.matrix * D.inv_diag()) @ self.matrix.T

    def solve_woodbury(self, D: DiagonalMass, b):
        """(D + K^T K)^-1 b = D^-1 b - D^-1 K^T (I + K D^-1 K^T)^-1 K D^-1 b."""
        dinv_b = D.apply_inv(b)
        inner = self.woodbury_inner(D)
        y = torch.linalg.solve(inner, self.matrix @ dinv_b)
        return dinv_b - D.apply_inv(self.matrix.T @ y)


# ---- manifold-constrained parameters ------------------------------------------------------------------------------
class ManifoldLinear:
    """Linear layer whose weight [out, in] lives on a matrix manifold; updates are dual-map steps."""

    FAMILIES = {"stiefel": mf.Stiefel, "grassmann": mf.Grassmann, "orthogonal": mf.Orthogonal}

    def __init__(self, weight: torch.Tensor, family: str = "stiefel", num_iters: int = 5):
        if family not in self.FAMILIES:
            raise ValueError(f"unknown matrix manifold family {family}")
        if family == "orthogonal" and weight.shape[0] != weight.shape[1]:
            raise ValueError("OrthogonalLinear needs a square weight")
        self.family = family
        self.manifold = self.FAMILIES[family]()
        self.geometry = mf.SpectralDualMap(self.manifold, num_iters)
        self.weight = weight

    @staticmethod
    def init(in_dim: int, out_dim: int, family: str = "stiefel", generator=None) -> "ManifoldLinear":
        w = torch.randn(out_dim, in_dim, generator=generator)
        m = ManifoldLinear.FAMILIES[family]()
        return ManifoldLinear(m.project(w), family)

    def forward2d(self, x):
        return x @ self.weight.T

    def apply_dual_map_update(self, grad: torch.Tensor, lr: float) -> "ManifoldLinear":
        g = self.manifold.tangent_project(self.weight, grad) if self.family == "orthogonal" else grad
        if self.family == "orthogonal":
            new = self.manifold.exp(self.weight, -lr * g / g.norm().clamp_min(1e-12))
        else:
            new = self.geometry.dual_map_step(self.weight, g, lr)
        return ManifoldLinear(new, self.family)

    def on_manifold(self, atol: float = 1e-4) -> bool:
        return self.manifold.check(self.weight, atol)


def StiefelLinear(in_dim, out_dim, **kw): return ManifoldLinear.init(in_dim, out_dim, "stiefel", **kw)
def GrassmannLinear(in_dim, out_dim, **kw): return ManifoldLinear.init(in_dim, out_dim, "grassmann", **kw)
def OrthogonalLinear(dim, **kw): return ManifoldLinear.init(dim, dim, "orthogonal", **kw)


class HyperbolicVector:
    """A point of the hyperboloid as a trainable vector parameter."""

    def __init__(self, value: torch.Tensor):
        self.manifold = mf.Hyperbolic()
        self.value = value

    @staticmethod
    def init(n: int, generator=None) -> "HyperbolicVector":
        return HyperbolicVector(mf.Hyperbolic().project(torch.randn(n + 1, generator=generator) * 0.1))

    def apply_dual_map_update(self, grad: torch.Tensor, lr: float) -> "HyperbolicVector":
        t = self.manifold.sharp(self.value, grad)
        return HyperbolicVector(self.manifold.exp(self.value, -lr * t))


def manifold_step(params, grads, lr: float):
    """``ManifoldUpdatable.step`` over a (nested) tuple/list of manifold parameters."""
    if isinstance(params, (tuple, list)):
        return type(params)(manifold_step(p, g, lr) for p, g in zip(params, grads))
    return params.apply_dual_map_update(grads, lr)


# ---- Riemannian modules (local linearisation + metric pullback) -----------------------------------------------------
@dataclass
class LocalLinearization:
    """Jacobians of one layer at a point: A = d out / d in, B = d out / d params (flattened)."""
    A: torch.Tensor   # [out, in]
    B: torch.Tensor   # [out, param_dim]


@dataclass
class LayerStepDiagnostics:
    grad_norm: float = 0.0
    natural_norm: float = 0.0
    step_norm: float = 0.0


class RiemannianLinear:
    """y = W x with the pulled-back metric step of RiemannianModule.lean:144-200."""

    def __init__(self, weight: torch.Tensor, mass: float = 1.0):
        self.weight, self.mass = weight, mass

    @property
    def in_dim(self): return self.weight.shape[1]
    @property
    def out_dim(self): return self.weight.shape[0]

    def forward_with_tape(self, x):
        return self.weight @ x, x

    def linearize(self, x) -> LocalLinearization:
        out_dim, in_dim = self.weight.shape
        B = torch.zeros(out_dim, out_dim * in_dim, dtype=self.weight.dtype)
        for o in range(out_dim):
            B[o, o * in_dim:(o + 1) * in_dim] = x
        return LocalLinearization(self.weight, B)

    def backward_leaf_step(self, tape, output_factor: MetricFactor, output_cotangent, lr: float):
        """Natural-gradient-like step: solve (mass I + (L B)^T (L B)) d = B^T g by Woodbury, apply
        w <- w - lr d, and hand the pulled-back factor / cotangent to the layer below."""
        x = tape
        lin = self.linearize(x)
        K = output_factor.pullback(lin.B)                     # [rank, param_dim]
        g = lin.B.T @ output_cotangent                        # parameter cotangent
        D = DiagonalMass.of_scalar(g.shape[0], self.mass)
        d = K.solve_woodbury(D, g)
        new = RiemannianLinear(self.weight - lr * d.reshape(self.weight.shape), self.mass)
        diag = LayerStepDiagnostics(float(g.norm()), float(d.norm()), float(lr * d.norm()))
        return new, output_factor.pullback(lin.A), lin.A.T @ output_cotangent, diag


def sequential_forward_with_tape(layers: Sequence[RiemannianLinear], x):
    tapes = []
    for l in layers:
        x, t = l.forward_with_tape(x)
        tapes.append(t)
    return x, tapes


def sequential_backward_metric_step(layers, tapes, output_factor: MetricFactor, output_cotangent, lr: float):
    new_layers, diags = [], []
    f, c = output_factor, output_cotangent
    for l, t in zip(reversed(list(layers)), reversed(tapes)):
        nl, f, c, d = l.backward_leaf_step(t, f, c, lr)
        new_layers.append(nl)
        diags.append(d)
    return list(reversed(new_layers)), f, c, list(reversed(diags))
