"""Differentiable manifolds (Tyr/Manifolds/*.lean).

``Manifold`` is the Python form of the ``DifferentiableManifold`` class (Basic.lean:36): tangent /
cotangent handling, the musical isomorphisms ``sharp`` / ``flat``, ``exp`` and ``retract``;
``gradient_step`` is Basic.lean:134.  ``DualMapGeometry`` (Optimizer.lean:48-77) adds a
steepest-descent dual map that may differ from the Riemannian sharp (norm-constrained optimizers
such as Muon).  Families: Euclidean, Stiefel (QR retraction), Orthogonal (skew tangents, matrix
exponential), Grassmann (principal angles, log), Sphere, Oblique, Positive, SPD (log-Euclidean),
PSD fixed rank / Elliptope, fixed-rank embedded, Poincare ball, Hyperbolic (Minkowski metric).
Points and tangents are plain tensors; every family exposes ``project`` (onto the manifold),
``tangent_project``, ``retract``, ``exp`` where closed forms exist, ``inner`` and ``check``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch


def sym(a: torch.Tensor) -> torch.Tensor:
    return 0.5 * (a + a.transpose(-1, -2))


def skew(a: torch.Tensor) -> torch.Tensor:
    return 0.5 * (a - a.transpose(-1, -2))


class Manifold:
    """Base: a flat (Euclidean) space where T = T* = M and exp(x, v) = x + v."""
    name = "euclidean"

    def project(self, x):
        return x

    def tangent_project(self, x, g):
        return g

    def zero_tangent(self, x):
        return torch.zeros_like(x)

    def add_tangent(self, x, u, v):
        return u + v

    def scale_tangent(self, x, s: float, v):
        return v * s

    def inner(self, x, u, v) -> torch.Tensor:
        return (u * v).sum()

    def norm(self, x, v) -> torch.Tensor:
        return self.inner(x, v, v).clamp_min(0).sqrt()

    def sharp(self, x, cot):
        """Cotangent -> tangent (Riemannian gradient of an ambient gradient)."""
        return self.tangent_project(x, cot)

    def flat(self, x, v):
        return v

    def exp(self, x, v):
        return x + v

    def retract(self, x, v):
        return self.exp(x, v)

    def check(self, x, atol: float = 1e-4) -> bool:
        return True

    def distance(self, x, y) -> torch.Tensor:
        return (x - y).norm()


EuclideanSpace = Manifold


def gradient_step(m: Manifold, x, grad, lr: float):
    """x' = retract(x, -lr * sharp(grad))."""
    return m.retract(x, m.scale_tangent(x, -lr, m.sharp(x, grad)))


class EmbeddedManifold(Manifold):
    """A manifold given by a projection of the ambient space (Embedded.lean:18): the retraction is
    ``project(x + v)`` and tangents are ambient vectors projected at x."""

    def retract(self, x, v):
        return self.project(x + v)

    def exp(self, x, v):
        return self.retract(x, v)


class Stiefel(EmbeddedManifold):
    """{W in R^{m x n}, n <= m : W^T W = I} (Stiefel.lean:32-76); retraction by reduced QR with
    the sign fixed so that R has a positive diagonal."""
    name = "stiefel"

    def project(self, x):
        m, n = x.shape[-2:]
        if n > m:
            return self.project(x.transpose(-1, -2)).transpose(-1, -2)
        q, r = torch.linalg.qr(x.float(), mode="reduced")
        d = torch.sign(torch.diagonal(r, dim1=-2, dim2=-1))
        d = torch.where(d == 0, torch.ones_like(d), d)
        return (q * d.unsqueeze(-2)).to(x.dtype)

    def tangent_project(self, x, g):
        return g - x @ sym(x.transpose(-1, -2) @ g)

    def check(self, x, atol: float = 1e-4) -> bool:
        m, n = x.shape[-2:]
        gram = x.transpose(-1, -2) @ x if n <= m else x @ x.transpose(-1, -2)
        eye = torch.eye(gram.shape[-1], dtype=gram.dtype, device=gram.device)
        return bool((gram - eye).abs().max() <= atol)


class Orthogonal(Manifold):
    """O(n) with skew-symmetric Lie-algebra tangents: exp(Q, Omega) = Q expm(Omega)
    (Orthogonal.lean:30-124)."""
    name = "orthogonal"

    def project(self, x):
        u, _, vh = torch.linalg.svd(x.float())
        return (u @ vh).to(x.dtype)

    def tangent_project(self, x, g):
        """Ambient gradient -> skew Omega with tangent Q Omega."""
        return skew(x.transpose(-1, -2) @ g)

    def to_ambient(self, x, omega):
        return x @ omega

    def inner(self, x, u, v):
        return (u * v).sum()

    def exp(self, x, omega):
        return x @ torch.linalg.matrix_exp(omega.float()).to(x.dtype)

    def retract(self, x, omega):
        return self.exp(x, omega)

    def check(self, x, atol: float = 1e-4) -> bool:
        eye = torch.eye(x.shape[-1], dtype=x.dtype, device=x.device)
        return bool((x.transpose(-1, -2) @ x - eye).abs().max() <= atol)


class Grassmann(EmbeddedManifold):
    """Subspaces represented by orthonormal bases Y (Grassmann.lean:35-131): horizontal tangents
    (I - Y Y^T) G, QR retraction, geodesic exp via the compact SVD, principal angles and log."""
    name = "grassmann"

    def project(self, x):
        return Stiefel().project(x)

    def tangent_project(self, x, g):
        return g - x @ (x.transpose(-1, -2) @ g)

    def exp(self, x, v):
        u, s, vh = torch.linalg.svd(v.float(), full_matrices=False)
        y = x.float() @ vh.transpose(-1, -2) @ torch.diag_embed(torch.cos(s)) @ vh + u @ torch.diag_embed(torch.sin(s)) @ vh
        return self.project(y.to(x.dtype))

    def principal_angles(self, x, y) -> torch.Tensor:
        s = torch.linalg.svdvals(x.float().transpose(-1, -2) @ y.float()).clamp(-1.0, 1.0)
        return torch.acos(s)

    def distance(self, x, y):
        return self.principal_angles(x, y).norm()

    def log(self, x, y):
        """Tangent at x pointing to y (y not orthogonal to x)."""
        xf, yf = x.float(), y.float()
        ytx = yf.transpose(-1, -2) @ xf
        at = yf.transpose(-1, -2) - ytx @ xf.transpose(-1, -2)
        bt = torch.linalg.solve(ytx, at)
        u, s, vh = torch.linalg.svd(bt.transpose(-1, -2), full_matrices=False)
        return (u @ torch.diag_embed(torch.atan(s)) @ vh).to(x.dtype)

    def check(self, x, atol: float = 1e-4) -> bool:
        return Stiefel().check(x, atol)


class Sphere(EmbeddedManifold):
    name = "sphere"

    def project(self, x):
        return x / x.norm().clamp_min(1e-12)

    def tangent_project(self, x, g):
        return g - x * (x * g).sum()

    def exp(self, x, v):
        n = v.norm()
        if float(n) < 1e-12:
            return x
        return torch.cos(n) * x + torch.sin(n) * v / n

    def distance(self, x, y):
        return torch.acos((x * y).sum().clamp(-1.0, 1.0))

    def check(self, x, atol: float = 1e-4) -> bool:
        return bool((x.norm() - 1.0).abs() <= atol)


class Oblique(EmbeddedManifold):
    """Matrices with unit-norm columns: a product of spheres."""
    name = "oblique"

    def project(self, x):
        return x / x.norm(dim=-2, keepdim=True).clamp_min(1e-12)

    def tangent_project(self, x, g):
        return g - x * (x * g).sum(dim=-2, keepdim=True)

    def check(self, x, atol: float = 1e-4) -> bool:
        return bool((x.norm(dim=-2) - 1.0).abs().max() <= atol)


class Positive(Manifold):
    """Entrywise positive tensors with the metric <u, v>_x = sum u v / x^2; exp(x, v) = x exp(v/x)."""
    name = "positive"

    def project(self, x):
        return x.clamp_min(1e-12)

    def inner(self, x, u, v):
        return (u * v / (x * x)).sum()

    def sharp(self, x, cot):
        return cot * x * x

    def flat(self, x, v):
        return v / (x * x)

    def exp(self, x, v):
        return x * torch.exp(v / x)

    def check(self, x, atol: float = 0.0) -> bool:
        return bool((x > 0).all())


class SymmetricPositiveDefinite(Manifold):
    """SPD matrices with the log-Euclidean structure: exp(X, V) = expm(logm X + V)
    (PositiveDefinite.lean; uses the checked matrix logarithm)."""
    name = "spd"

    @staticmethod
    def logm(x):
        w, v = torch.linalg.eigh(sym(x.float()))
        if (w <= 0).any():
            raise ValueError("SymmetricPositiveDefinite.logm: matrix is not positive definite")
        return (v @ torch.diag_embed(torch.log(w)) @ v.transpose(-1, -2)).to(x.dtype)

    @staticmethod
    def expm(a):
        w, v = torch.linalg.eigh(sym(a.float()))
        return (v @ torch.diag_embed(torch.exp(w)) @ v.transpose(-1, -2)).to(a.dtype)

    def project(self, x, floor: float = 1e-8):
        w, v = torch.linalg.eigh(sym(x.float()))
        return (v @ torch.diag_embed(w.clamp_min(floor)) @ v.transpose(-1, -2)).to(x.dtype)

    def tangent_project(self, x, g):
        return sym(g)

    def exp(self, x, v):
        return self.expm(self.logm(x) + sym(v))

    def distance(self, x, y):
        return (self.logm(x) - self.logm(y)).norm()

    def check(self, x, atol: float = 1e-5) -> bool:
        if (x - x.transpose(-1, -2)).abs().max() > atol:
            return False
        return bool((torch.linalg.eigvalsh(x.float()) > 0).all())


class PSDFixedRank(Manifold):
    """PSD matrices of rank k as Y Y^T with Y in R^{n x k} (PSD.lean): quotient by O(k); the
    horizontal projection removes the skew part of Y^T G solved from a Sylvester equation."""
    name = "psd_fixed_rank"

    def matrix(self, y):
        return y @ y.transpose(-1, -2)

    def tangent_project(self, y, g):
        yty = y.transpose(-1, -2) @ y
        rhs = y.transpose(-1, -2) @ g - g.transpose(-1, -2) @ y
        w, q = torch.linalg.eigh(yty.float())
        r = q.transpose(-1, -2) @ rhs.float() @ q
        om = q @ (r / (w[:, None] + w[None, :]).clamp_min(1e-12)) @ q.transpose(-1, -2)
        return g - y @ om.to(y.dtype)

    def retract(self, y, v):
        return y + v


class Elliptope(PSDFixedRank):
    """Rank-k correlation matrices: rows of Y have unit norm."""
    name = "elliptope"

    def project(self, y):
        return y / y.norm(dim=-1, keepdim=True).clamp_min(1e-12)

    def tangent_project(self, y, g):
        g = g - y * (y * g).sum(dim=-1, keepdim=True)
        return super().tangent_project(y, g)

    def retract(self, y, v):
        return self.project(y + v)

    def check(self, y, atol: float = 1e-4) -> bool:
        return bool((y.norm(dim=-1) - 1.0).abs().max() <= atol)


class FixedRankEmbedded(EmbeddedManifold):
    """Rank-k matrices embedded in R^{m x n}; projection = truncated SVD (FixedRank.lean)."""
    name = "fixed_rank"

    def __init__(self, rank: int):
        self.rank = rank

    def project(self, x):
        u, s, vh = torch.linalg.svd(x.float(), full_matrices=False)
        k = self.rank
        return ((u[..., :k] * s[..., None, :k]) @ vh[..., :k, :]).to(x.dtype)

    def tangent_project(self, x, g):
        u, s, vh = torch.linalg.svd(x.float(), full_matrices=False)
        u, vh = u[..., :self.rank], vh[..., :self.rank, :]
        pu, pv = u @ u.transpose(-1, -2), vh.transpose(-1, -2) @ vh
        gf = g.float()
        return (pu @ gf + gf @ pv - pu @ gf @ pv).to(g.dtype)

    def check(self, x, atol: float = 1e-4) -> bool:
        s = torch.linalg.svdvals(x.float())
        return bool((s[..., self.rank:] <= atol * max(1.0, float(s.max()))).all())


class PoincareBall(Manifold):
    """Unit ball with curvature -c: conformal factor lambda = 2 / (1 - c |x|^2), Mobius addition,
    exponential map, distance (PoincareBall.lean)."""
    name = "poincare_ball"

    def __init__(self, c: float = 1.0):
        self.c = c

    def project(self, x, eps: float = 1e-5):
        maxn = (1.0 - eps) / math.sqrt(self.c)
        n = x.norm(dim=-1, keepdim=True).clamp_min(1e-15)
        return torch.where(n > maxn, x / n * maxn, x)

    def lam(self, x):
        return 2.0 / (1.0 - self.c * (x * x).sum(-1, keepdim=True)).clamp_min(1e-15)

    def inner(self, x, u, v):
        return (self.lam(x) ** 2 * (u * v).sum(-1, keepdim=True)).sum()

    def sharp(self, x, cot):
        return cot / self.lam(x) ** 2

    def flat(self, x, v):
        return v * self.lam(x) ** 2

    def mobius_add(self, x, y):
        c = self.c
        xy = (x * y).sum(-1, keepdim=True)
        x2 = (x * x).sum(-1, keepdim=True)
        y2 = (y * y).sum(-1, keepdim=True)
        num = (1 + 2 * c * xy + c * y2) * x + (1 - c * x2) * y
        den = 1 + 2 * c * xy + c * c * x2 * y2
        return num / den.clamp_min(1e-15)

    def exp(self, x, v):
        sc = math.sqrt(self.c)
        n = v.norm(dim=-1, keepdim=True).clamp_min(1e-15)
        second = torch.tanh(sc * self.lam(x) * n / 2) * v / (sc * n)
        return self.project(self.mobius_add(x, second))

    def retract(self, x, v):
        return self.project(x + v)

    def distance(self, x, y):
        sc = math.sqrt(self.c)
        d = self.mobius_add(-x, y).norm(dim=-1).clamp(max=(1 - 1e-7) / sc)
        return (2 / sc) * torch.atanh(sc * d)

    def check(self, x, atol: float = 0.0) -> bool:
        return bool(((x * x).sum(-1) * self.c < 1.0).all())


class Hyperbolic(Manifold):
    """Hyperboloid model: <x, x>_L = -1 with the Minkowski inner product (Hyperbolic.lean)."""
    name = "hyperbolic"

    @staticmethod
    def minkowski_inner(u, v):
        return -(u[..., 0] * v[..., 0]) + (u[..., 1:] * v[..., 1:]).sum(-1)

    def project(self, x):
        sp = x[..., 1:]
        t = torch.sqrt(1.0 + (sp * sp).sum(-1, keepdim=True))
        return torch.cat([t, sp], dim=-1)

    def tangent_project(self, x, g):
        return g + self.minkowski_inner(x, g).unsqueeze(-1) * x

    def sharp(self, x, cot):
        g = cot.clone()
        g[..., 0] = -g[..., 0]          # raise the time-like index
        return self.tangent_project(x, g)

    def inner(self, x, u, v):
        return self.minkowski_inner(u, v).sum()

    def minkowski_norm(self, v):
        return torch.sqrt(self.minkowski_inner(v, v).abs())

    def exp(self, x, v):
        n = self.minkowski_norm(v).unsqueeze(-1).clamp_min(1e-15)
        return self.project(torch.cosh(n) * x + torch.sinh(n) * v / n)

    def distance(self, x, y):
        return torch.acosh((-self.minkowski_inner(x, y)).clamp_min(1.0))

    def check(self, x, atol: float = 1e-4) -> bool:
        return bool((self.minkowski_inner(x, x) + 1.0).abs().max() <= atol)


# ---- dual-map geometry ---------------------------------------------------------------------------------
class DualMapGeometry:
    """Steepest descent under a chosen norm: ``dual_map`` sends a cotangent to the tangent direction
    that maximises the pairing under ``tangent_norm`` (Optimizer.lean:48-77)."""

    def __init__(self, manifold: Manifold):
        self.m = manifold

    def tangent_norm(self, x, v) -> float:
        return float(self.m.norm(x, v))

    def cotangent_norm(self, x, g) -> float:
        return float(g.norm())

    def dual_map(self, x, g):
        return self.m.sharp(x, g)

    def steepest_direction(self, x, g):
        return self.dual_map(x, g)

    def dual_map_step(self, x, g, lr: float):
        return self.m.retract(x, self.m.scale_tangent(x, -lr, self.steepest_direction(x, g)))

    def dual_map_step_with_diagnostics(self, x, g, lr: float):
        d = self.steepest_direction(x, g)
        return (self.m.retract(x, self.m.scale_tangent(x, -lr, d)),
                StepDiagnostics(self.tangent_norm(x, d), self.cotangent_norm(x, g)))


@dataclass
class StepDiagnostics:
    tangent_norm: float
    cotangent_norm: float


class SignDualMap(DualMapGeometry):
    """The reference's float example: the step direction saturates to {-1, 0, 1}."""

    def __init__(self):
        super().__init__(Manifold())

    def dual_map(self, x, g):
        return torch.sign(g)


class SpectralDualMap(DualMapGeometry):
    """Matrix manifolds under the spectral norm: dual map = msign of the projected gradient, then
    projected back to the tangent space and normalised (the generic-manifold branch of
    DualOptimizer.stepGenericManifoldSingle, Tyr/Optim/DualOptimizer.lean:412)."""

    def __init__(self, manifold: Manifold, num_iters: int = 5):
        super().__init__(manifold)
        self.num_iters = num_iters

    def tangent_norm(self, x, v) -> float:
        return float(torch.linalg.matrix_norm(self._amb(x, v).float(), 2))

    def cotangent_norm(self, x, g) -> float:
        return float(torch.linalg.matrix_norm(g.float(), "nuc"))

    def _amb(self, x, v):
        return self.m.to_ambient(x, v) if isinstance(self.m, Orthogonal) else v

    def dual_map(self, x, g):
        from ..optim import polar_express as pe
        d = pe.apply(g.float(), pe.Config(self.num_iters)).to(g.dtype)
        t = self.m.tangent_project(x, d)
        n = t.norm()
        return t / n if float(n) > 0 else t
