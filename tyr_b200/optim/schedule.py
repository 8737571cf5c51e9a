"""Schedules ``step -> value`` and their combinators (Tyr/Optim/Scheduler.lean:28-158)."""
from __future__ import annotations

import math
from typing import Callable

Schedule = Callable[[int], float]


def constant(value: float) -> Schedule:
    return lambda _: value


def cosine_decay(peak: float, total_steps: int, end_value: float = 0.0, warmup_steps: int = 0) -> Schedule:
    def f(step):
        if step < warmup_steps:
            return peak * (step / max(float(warmup_steps), 1.0))
        if step >= total_steps:
            return end_value
        progress = (step - warmup_steps) / max(float(total_steps - warmup_steps), 1.0)
        return end_value + 0.5 * (1.0 + math.cos(math.pi * progress)) * (peak - end_value)
    return f


def linear_decay(peak: float, total_steps: int, end_value: float = 0.0, warmup_steps: int = 0) -> Schedule:
    def f(step):
        if step < warmup_steps:
            return peak * (step / max(float(warmup_steps), 1.0))
        if step >= total_steps:
            return end_value
        progress = (step - warmup_steps) / max(float(total_steps - warmup_steps), 1.0)
        return peak - progress * (peak - end_value)
    return f


def step_decay(initial: float, gamma: float = 0.1, step_size: int = 30) -> Schedule:
    return lambda step: initial * gamma ** (step // step_size)


def one_cycle(peak: float, total_steps: int, min_value: float = 0.0, pct_start: float = 0.3) -> Schedule:
    def f(step):
        if step >= total_steps:
            return min_value
        warm = int(pct_start * total_steps)
        if step < warm:
            return min_value + (step / max(float(warm), 1.0)) * (peak - min_value)
        progress = (step - warm) / max(float(total_steps - warm), 1.0)
        return min_value + 0.5 * (1.0 + math.cos(math.pi * progress)) * (peak - min_value)
    return f


def warmup_plateau_cosine(peak: float, total_steps: int, warmup_steps: int, plateau_steps: int,
                          end_value: float = 0.0) -> Schedule:
    def f(step):
        decay_start = warmup_steps + plateau_steps
        if step < warmup_steps:
            return peak * (step / max(float(warmup_steps), 1.0))
        if step < decay_start:
            return peak
        if step >= total_steps:
            return end_value
        progress = (step - decay_start) / max(float(total_steps - decay_start), 1.0)
        return end_value + 0.5 * (1.0 + math.cos(math.pi * progress)) * (peak - end_value)
    return f


def exponential_decay(initial: float, gamma: float = 0.99) -> Schedule:
    return lambda step: initial * gamma ** step


def polynomial_decay(initial: float, total_steps: int, end_value: float = 0.0, power: float = 1.0) -> Schedule:
    def f(step):
        if step >= total_steps:
            return end_value
        return end_value + (1.0 - step / total_steps) ** power * (initial - end_value)
    return f


def warmup(peak: float, warmup_steps: int) -> Schedule:
    def f(step):
        if warmup_steps == 0 or step >= warmup_steps:
            return peak
        return peak * (step / warmup_steps)
    return f


def join(s1: Schedule, s2: Schedule, boundary: int) -> Schedule:
    return lambda step: s1(step) if step < boundary else s2(step)


def sequence(s1: Schedule, duration: int, s2: Schedule) -> Schedule:
    return lambda step: s1(step) if step < duration else s2(step - duration)


def scale_schedule(s: Schedule, factor: float) -> Schedule:
    return lambda step: s(step) * factor


def multiply(s1: Schedule, s2: Schedule) -> Schedule:
    return lambda step: s1(step) * s2(step)


def add(s1: Schedule, s2: Schedule) -> Schedule:
    return lambda step: s1(step) + s2(step)


def clamp(s: Schedule, lo: float, hi: float) -> Schedule:
    return lambda step: min(hi, max(lo, s(step)))


def linear_weight_decay(base_wd: float, total_steps: int) -> Schedule:
    return lambda step: 0.0 if step >= total_steps else base_wd * (1.0 - step / total_steps)


def cosine_weight_decay(base_wd: float, total_steps: int) -> Schedule:
    return lambda step: 0.0 if step >= total_steps else base_wd * 0.5 * (1.0 + math.cos(math.pi * step / total_steps))
