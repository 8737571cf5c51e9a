"""Chat supervised fine-tuning: masked cross-entropy over assistant tokens, gradient accumulation derived from the
world size, linear LR decay, AdamW over the whole parameter tree, optional validation and ledger callbacks
(Tyr/Train/ChatSFT.lean)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .. import distributed as tdist
from ..data.task import ConversationBatch, TaskIterator, TokenizedConversation, collate
from ..optim import core as optim
from ..struct import tree as ts
from . import run_ledger as rl


@dataclass
class SFTConfig:
    num_epochs: int = 1
    num_iterations: Optional[int] = None
    device_batch_size: int = 4
    target_examples_per_step: int = 32
    embedding_lr: float = 0.2
    matrix_lr: float = 0.02
    init_lr_frac: float = 0.02
    max_seq_len: int = 2048
    eval_every: int = 100
    eval_steps: int = 100
    device: str = "cpu"
    log_interval: int = 10

    def grad_accum_steps(self, world_size: int = 1) -> int:
        per_step = self.device_batch_size * world_size
        steps = self.target_examples_per_step // per_step
        if steps <= 0:
            raise ValueError(f"SFT targetExamplesPerStep={self.target_examples_per_step} is smaller than "
                             f"deviceBatchSize*worldSize={per_step}")
        return steps


def linear_lr_multiplier(step: int, num_iterations: int) -> float:
    return 1.0 if num_iterations == 0 else 1.0 - step / num_iterations


@dataclass
class SFTState:
    step: int = 0
    epoch: int = 0
    best_val_loss: float = 1e10
    running_loss: float = 0.0
    total_tokens: int = 0


@dataclass
class SFTBatch:
    inputs: torch.Tensor      # int64 [B, S]
    targets: torch.Tensor     # int64 [B, S]
    mask: torch.Tensor        # float [B, S]
    num_valid_tokens: int

    @staticmethod
    def empty() -> "SFTBatch":
        z = torch.zeros(0, 0, dtype=torch.int64)
        return SFTBatch(z, z, torch.zeros(0, 0), 0)

    @staticmethod
    def of_conversation_batch(b: ConversationBatch) -> "SFTBatch":
        """inputs = tokens[:-1], targets = tokens[1:], mask = mask[1:] (aligned with the targets)."""
        if b.batch_size == 0 or b.seq_len < 2:
            return SFTBatch.empty()
        m = b.mask[:, 1:].contiguous()
        return SFTBatch(b.tokens[:, :-1].contiguous(), b.tokens[:, 1:].contiguous(), m, int(m.sum().item()))

    def to(self, device) -> "SFTBatch":
        return SFTBatch(self.inputs.to(device), self.targets.to(device), self.mask.to(device), self.num_valid_tokens)


def masked_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """Mean CE over positions with mask = 1: ``sum(ce * mask) / (sum(mask) + 1e-8)``."""
    if not (mask.dtype == torch.bool or mask.dtype.is_floating_point or not mask.dtype.is_complex):
        raise TypeError("maskedCrossEntropy requires a real numeric or Bool mask")
    V = logits.shape[-1]
    ce = F.cross_entropy(logits.reshape(-1, V).float(), targets.reshape(-1), reduction="none")
    m = mask.reshape(-1).float()
    return (ce * m).sum() / (m.sum() + 1e-8)


def prepare_sft_batch(convs: Sequence[TokenizedConversation], max_len: int, pad_token_id: int) -> SFTBatch:
    return SFTBatch.of_conversation_batch(collate(convs, max_len, pad_token_id))


def sft_forward(params, forward_fn, batch: SFTBatch) -> torch.Tensor:
    return masked_cross_entropy(forward_fn(params, batch.inputs), batch.targets, batch.mask)


@torch.no_grad()
def eval_validation_loss(params, val_data_fn: Callable[[], SFTBatch], forward_fn, eval_steps: int, device) -> Optional[float]:
    tot, n = 0.0, 0
    for _ in range(eval_steps):
        b = val_data_fn().to(device)
        if b.num_valid_tokens == 0:
            continue
        tot += float(sft_forward(params, forward_fn, b))
        n += 1
    return tot / n if n else None


def format_train_update(step: int, loss: float, lrm: float, num_tokens: int) -> str:
    return f"step {step:05d} | loss {loss:.4f} | lrm {lrm:.3f} | tokens {num_tokens}"


def format_validation_update(step: int, val_loss: float) -> str:
    return f"step {step:05d} | val loss {val_loss:.4f}"


@dataclass
class Callbacks:
    on_train_step: Callable[[int, float, float, int], None] = lambda step, loss, lrm, ntok: None
    on_validation: Callable[[int, float], None] = lambda step, loss: None

    def combine(self, other: "Callbacks") -> "Callbacks":
        def t(*a):
            self.on_train_step(*a); other.on_train_step(*a)

        def v(*a):
            self.on_validation(*a); other.on_validation(*a)
        return Callbacks(t, v)


def artifact_callbacks(artifacts: rl.RunArtifacts, scope: str = "sft") -> Callbacks:
    """Rows in metrics.jsonl for every logged train step and validation."""
    return Callbacks(
        lambda step, loss, lrm, ntok: rl.append_metric_event(artifacts, rl.MetricEvent(scope, step, [("train_loss", loss), ("lrm", lrm), ("tokens", ntok)])),
        lambda step, loss: rl.append_metric_event(artifacts, rl.MetricEvent(scope, step, [("val_loss", loss)])))


def train_loop(cfg: SFTConfig, params, opt_state, forward_fn: Callable, train_data_fn: Callable[[], SFTBatch],
               val_data_fn: Optional[Callable[[], SFTBatch]] = None, num_train_examples: int = 10000,
               callbacks: Optional[Callbacks] = None, loss_fn: Callable = masked_cross_entropy):
    """``forward_fn(params, inputs) -> logits [B, S, V]``.  Returns ``(params, opt_state, SFTState)``."""
    callbacks = callbacks or Callbacks()
    distributed = tdist.is_initialized()
    world = tdist.get_world_size() if distributed else 1
    n_iter = cfg.num_iterations if cfg.num_iterations is not None else (num_train_examples // cfg.target_examples_per_step) * cfg.num_epochs
    accum = cfg.grad_accum_steps(world)
    device = torch.device(cfg.device)
    cur = ts.make_leaf_params(params)
    state = SFTState()
    for step in range(n_iter):
        last = step == n_iter - 1
        state.step = step
        if val_data_fn is not None and (last or (step > 0 and cfg.eval_every > 0 and step % cfg.eval_every == 0)):
            vl = eval_validation_loss(cur, val_data_fn, forward_fn, cfg.eval_steps, device)
            if vl is not None:
                callbacks.on_validation(step, vl)
                state.best_val_loss = min(state.best_val_loss, vl)
        if last:
            break
        work = ts.make_leaf_params(cur)
        ts.zero_grads(work)
        acc_loss, n_tok = 0.0, 0
        for _ in range(accum):
            b = train_data_fn().to(device)
            if b.num_valid_tokens > 0:
                loss = loss_fn(forward_fn(work, b.inputs), b.targets, b.mask)
                (loss / accum).backward()
                acc_loss += float(loss.detach())
                n_tok += b.num_valid_tokens
        lrm = linear_lr_multiplier(step, n_iter)
        lr = cfg.embedding_lr * cfg.init_lr_frac * lrm
        grads = ts.tree_map(lambda p: p.grad if p.grad is not None else torch.zeros_like(p), work)
        if distributed:
            grads = tdist.all_reduce_grads(grads, tdist.ReduceOp.avg)
        with torch.no_grad():
            cur, opt_state = optim.step(optim.adamw(lr=lr, b1=0.9, b2=0.999), ts.detach(work), grads, opt_state)
        state.total_tokens += n_tok
        state.running_loss += acc_loss / accum
        if cfg.log_interval > 0 and step % cfg.log_interval == 0:
            callbacks.on_train_step(step, acc_loss / accum, lrm, n_tok)
    return cur, opt_state, state


def make_task_data_generator(it: TaskIterator) -> Callable[[], SFTBatch]:
    """Yields an SFT batch per call and rolls over epoch ends."""
    def gen() -> SFTBatch:
        for _ in range(2):
            b = it.next_batch()
            if b is not None:
                return SFTBatch.of_conversation_batch(b)
        return SFTBatch.empty()
    return gen


def train_sft(cfg: SFTConfig, params, forward_fn, train_iter: TaskIterator, val_iter: Optional[TaskIterator] = None,
              callbacks: Optional[Callbacks] = None):
    opt = optim.adamw(lr=cfg.embedding_lr * cfg.init_lr_frac)
    state = opt.init(ts.detach(params))
    return train_loop(cfg, params, state, forward_fn, make_task_data_generator(train_iter),
                      make_task_data_generator(val_iter) if val_iter is not None else None, train_iter.mixture.size(), callbacks)
