"""Optax-style gradient transformations over tensor trees (Tyr/Optim.lean:100-314).

A ``GradientTransformation`` has ``init(params) -> state`` and
``update(params, grads, state) -> (updates, state)``; ``update`` returns transformed gradients,
not parameters, so transformations compose with ``chain``.  ``apply_updates`` adds the updates to
detached parameters and returns fresh trainable leaves.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Tuple

import torch

from ..struct import tree as ts

Schedule = Callable[[int], float]


@dataclass
class GradientTransformation:
    init: Callable[[Any], Any]
    update: Callable[[Any, Any, Any], Tuple[Any, Any]]


@dataclass
class EmptyState:
    pass


@dataclass
class ScaleByAdamState:
    count: int
    mu: Any
    nu: Any


@dataclass
class TraceState:
    trace: Any


@dataclass
class ChainState:
    fst: Any
    snd: Any


@dataclass
class ScaleByScheduleState:
    count: int


def _raw(t):
    return ts._raw(t)


def _like(t, r):
    return ts._like(t, r)


def _zeros_like(tree):
    return ts.tree_map(lambda t: _like(t, torch.zeros_like(_raw(t))), tree)


def scale(step_size: float) -> GradientTransformation:
    return GradientTransformation(lambda _: EmptyState(),
                                  lambda p, g, s: (ts.scale(g, step_size), s))


def scale_by_adam(b1: float = 0.9, b2: float = 0.999, eps: float = 1e-8) -> GradientTransformation:
    def init(model):
        return ScaleByAdamState(0, _zeros_like(model), _zeros_like(model))

    def update(_params, grads, state):
        ts._floating_check(grads)
        count = state.count + 1
        mu = ts.zip_with(lambda m, g: _like(m, _raw(m) * b1 + _raw(g).detach() * (1.0 - b1)), state.mu, grads)
        nu = ts.zip_with(lambda v, g: _like(v, _raw(v) * b2 + _raw(g).detach() ** 2 * (1.0 - b2)), state.nu, grads)
        bc1, bc2 = 1.0 - b1 ** count, 1.0 - b2 ** count
        upd = ts.zip_with(lambda m, v: _like(m, (_raw(m) / bc1) / (torch.sqrt(_raw(v) / bc2) + eps)), mu, nu)
        return upd, ScaleByAdamState(count, mu, nu)
    return GradientTransformation(init, update)


def add_decayed_weights(decay: float) -> GradientTransformation:
    def update(params, grads, state):
        return ts.zip_with(lambda p, g: _like(g, _raw(g) + _raw(p).detach() * decay), params, grads), state
    return GradientTransformation(lambda _: EmptyState(), update)


def trace(decay: float) -> GradientTransformation:
    def update(_params, grads, state):
        new = ts.zip_with(lambda t, g: _like(t, _raw(t) * decay + _raw(g)), state.trace, grads)
        return new, TraceState(new)
    return GradientTransformation(lambda m: TraceState(_zeros_like(m)), update)


def chain(t1: GradientTransformation, t2: GradientTransformation) -> GradientTransformation:
    def init(model):
        return ChainState(t1.init(model), t2.init(model))

    def update(params, grads, state):
        u1, s1 = t1.update(params, grads, state.fst)
        u2, s2 = t2.update(params, u1, state.snd)
        return u2, ChainState(s1, s2)
    return GradientTransformation(init, update)


def adamw(lr: float = 1e-3, b1: float = 0.9, b2: float = 0.999, eps: float = 1e-8,
          weight_decay: float = 0.01) -> GradientTransformation:
    """scale_by_adam -> add_decayed_weights -> scale(-lr)."""
    return chain(scale_by_adam(b1, b2, eps), chain(add_decayed_weights(weight_decay), scale(-lr)))


def sgd_momentum(lr: float, momentum: float = 0.9) -> GradientTransformation:
    return chain(trace(momentum), scale(-lr))


def sgd(lr: float) -> GradientTransformation:
    return scale(-lr)


def scale_by_schedule(schedule: Schedule) -> GradientTransformation:
    def update(_params, grads, state):
        return ts.scale(grads, schedule(state.count)), ScaleByScheduleState(state.count + 1)
    return GradientTransformation(lambda _: ScaleByScheduleState(0), update)


def adamw_schedule(lr_schedule: Schedule, b1: float = 0.9, b2: float = 0.999, eps: float = 1e-8,
                   weight_decay: float = 0.01) -> GradientTransformation:
    return chain(scale_by_adam(b1, b2, eps),
                 chain(add_decayed_weights(weight_decay), chain(scale_by_schedule(lr_schedule), scale(-1.0))))


def sgd_momentum_schedule(lr_schedule: Schedule, momentum: float = 0.9) -> GradientTransformation:
    return chain(trace(momentum), chain(scale_by_schedule(lr_schedule), scale(-1.0)))


def sgd_schedule(lr_schedule: Schedule) -> GradientTransformation:
    return chain(scale_by_schedule(lr_schedule), scale(-1.0))


def clip_by_global_norm(max_norm: float) -> GradientTransformation:
    """Gradient clipping (left as a TODO in the reference, Tyr/Optim.lean:308)."""
    def update(_params, grads, state):
        sq = ts.fold(lambda t, acc: acc + float(_raw(t).float().pow(2).sum()), 0.0, grads)
        norm = sq ** 0.5
        f = min(1.0, max_norm / (norm + 1e-6))
        return ts.scale(grads, f), state
    return GradientTransformation(lambda _: EmptyState(), update)


def apply_updates(params, updates):
    upd = ts.zip_with(lambda p, u: _like(p, _raw(p).detach() + _raw(u)), params, updates)
    return ts.make_leaf_params(upd)


def step(opt: GradientTransformation, params, grads, state):
    """Full optimizer step: returns (new_params, new_state)."""
    updates, new_state = opt.update(params, grads, state)
    return apply_updates(params, updates), new_state
