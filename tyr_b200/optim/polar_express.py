"""Polar Express wrappers (Tyr/Optim/PolarExpress.lean:21-107) over :mod:`tyr_b200.ops.polar`."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import polar

COEFFICIENTS = polar.POLAR_EXPRESS_COEFFS


@dataclass
class Config:
    num_iters: int = 5


def apply(g: torch.Tensor, cfg: Config = Config()) -> torch.Tensor:
    """Matrix-sign approximation of ``g`` (keeps dtype); short side is orthogonalised."""
    if g.dim() < 2:
        raise ValueError("PolarExpress.apply requires a matrix")
    tall = g.shape[-2] > g.shape[-1]
    x = g.transpose(-1, -2) if tall else g
    y = polar.polar_express(x, cfg.num_iters)
    return y.transpose(-1, -2) if tall else y


def muon_orthogonalize(g: torch.Tensor, num_iters: int = 5) -> torch.Tensor:
    return polar.muon_orthogonalize(g, num_iters)


def apply_batch(gs, cfg: Config = Config()):
    """Same-shape matrices are stacked and orthogonalised in one batched call."""
    if not gs:
        return []
    stacked = torch.stack(list(gs))
    out = apply(stacked, cfg)
    return list(out.unbind(0))
