from .core import (GradientTransformation, scale, scale_by_adam, add_decayed_weights, trace, chain, adamw, sgd,  # noqa: F401
                   sgd_momentum, apply_updates, step, scale_by_schedule, adamw_schedule, sgd_schedule,
                   sgd_momentum_schedule, clip_by_global_norm)
from . import schedule, polar_express, normuon, distadam, dual, manifold_muon, riemannian  # noqa: F401
