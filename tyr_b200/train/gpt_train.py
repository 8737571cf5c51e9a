"""Char-GPT training loop (Examples/GPT/Train.lean:20-260): cosine LR with warmup, random
contiguous-window batches, per-tensor gradient clipping, Optax-style AdamW step, leak gauge."""
from __future__ import annotations

import math
import time
from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch

from .. import optim
from ..models import gpt
from ..struct import tree as ts
from ..typed import Device, Tensor, get_live_tensors
from ..typed import ops as O


@dataclass
class TrainConfig:
    max_iters: int = 1000
    eval_interval: int = 100
    log_interval: int = 10
    learning_rate: float = 1e-3
    min_lr: float = 1e-4
    warmup_iters: int = 100
    lr_decay_iters: int = 1000
    grad_clip: float = 1.0
    batch_size: int = 4
    block_size: int = 64
    grad_accum_steps: int = 1
    device: Device = Device.CPU


def get_lr(cfg: TrainConfig, it: int) -> float:
    if it < cfg.warmup_iters:
        return cfg.learning_rate * (it / cfg.warmup_iters)
    if it > cfg.lr_decay_iters:
        return cfg.min_lr
    ratio = (it - cfg.warmup_iters) / (cfg.lr_decay_iters - cfg.warmup_iters)
    return cfg.min_lr + 0.5 * (1.0 + math.cos(math.pi * ratio)) * (cfg.learning_rate - cfg.min_lr)


def get_batch(data: torch.Tensor, batch_size: int, block_size: int, device: Device = Device.CPU, generator=None):
    """A random start, then ``batch_size`` consecutive windows; y is x shifted by one."""
    n = data.numel()
    required = batch_size * (block_size + 1)
    if batch_size == 0 or block_size == 0 or required > n:
        raise ValueError("GPT batch requires positive dimensions and enough tokens")
    start = int(torch.randint(0, n - required + 1, (), generator=generator))
    block = data[start:start + required].reshape(batch_size, block_size + 1)
    x, y = block[:, :block_size].contiguous(), block[:, 1:].contiguous()
    return Tensor.of_tensor(x.to(device.torch)), Tensor.of_tensor(y.to(device.torch))


def clip_gpt_grads(params, max_norm: float) -> None:
    for t in ts.leaves(params, include_frozen=False):
        O.clip_grad_norm_(t, max_norm)


def train_step(cfg: TrainConfig, params, opt_state, x: Tensor, y: Tensor, lr: float):
    ts.zero_grads(params)
    loss_t = gpt.loss(params, x, y, True)
    O.backward_loss(loss_t)
    if cfg.grad_clip > 0:
        clip_gpt_grads(params, cfg.grad_clip)
    loss_val = loss_t.item()
    grads = ts.grads(params)
    opt = optim.adamw(lr=lr)
    params, opt_state = optim.step(opt, params, grads, opt_state)
    return params, opt_state, loss_val


def train_loop(cfg: TrainConfig, params, data: torch.Tensor, log: Optional[Callable[[str], None]] = None,
               val_data: Optional[torch.Tensor] = None, generator=None):
    opt_state = optim.adamw(lr=cfg.learning_rate).init(params)
    losses = []
    t0 = time.time()
    for it in range(cfg.max_iters):
        x, y = get_batch(data, cfg.batch_size, cfg.block_size, cfg.device, generator)
        params, opt_state, l = train_step(cfg, params, opt_state, x, y, get_lr(cfg, it))
        losses.append(l)
        if log and it % cfg.log_interval == 0:
            log(f"iter {it}: loss {l:.4f}, lr {get_lr(cfg, it):.2e}, live tensors {get_live_tensors()}, "
                f"{(time.time() - t0) * 1000 / (it + 1):.1f} ms/iter")
        if log and val_data is not None and it > 0 and it % cfg.eval_interval == 0:
            with torch.no_grad():
                vx, vy = get_batch(val_data, cfg.batch_size, cfg.block_size, cfg.device, generator)
                log(f"iter {it}: val loss {gpt.loss(params, vx, vy, False).item():.4f}")
    return params, opt_state, losses
