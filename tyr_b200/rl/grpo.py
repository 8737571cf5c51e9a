"""GRPO as used by nanochat: REINFORCE with mean-subtracted advantages over groups of sampled completions
(Tyr/RL/GRPO.lean).  Rollouts come from a user-supplied ``generate_one`` function; the policy-gradient loss is
``-sum(logp * A * mask) / (num_valid * num_passes * examples_per_rank)``."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .. import distributed as tdist
from ..optim import core as optim
from ..struct import tree as ts
from ..train import run_ledger as rl


@dataclass
class GRPOConfig:
    num_samples: int = 16
    max_new_tokens: int = 256
    temperature: float = 1.0
    top_k: Optional[int] = None
    examples_per_step: int = 16
    device_batch_size: int = 8
    embedding_lr: float = 0.2
    unembedding_lr: float = 0.004
    matrix_lr: float = 0.02
    init_lr_frac: float = 0.05
    weight_decay: float = 0.0
    eval_every: int = 100
    log_every: int = 10
    pad_token: int = 0
    eos_token: int = 2


def get_lr_multiplier(step: int, total_steps: int, init_lr_frac: float = 0.05) -> float:
    return init_lr_frac * (1.0 - step / total_steps)


def compute_advantages(rewards: Sequence[float]) -> List[float]:
    """A = r - mean(r); no division by the standard deviation."""
    if not rewards:
        return []
    mu = sum(rewards) / len(rewards)
    return [r - mu for r in rewards]


def compute_advantages_tensor(rewards: torch.Tensor) -> torch.Tensor:
    return rewards - rewards.mean()


@dataclass
class RewardResult:
    reward: float
    is_valid: bool = True


def math_reward(expected_answer: str, response: str) -> RewardResult:
    parts = response.split("####")
    if len(parts) < 2:
        return RewardResult(0.0)
    return RewardResult(1.0 if parts[1].strip() == expected_answer.strip() else 0.0)


def exact_match_reward(expected: str, response: str) -> RewardResult:
    return RewardResult(1.0 if response.strip() == expected.strip() else 0.0)


@dataclass
class Sample:
    response_tokens: List[int]
    response_text: str
    reward: float


@dataclass
class RolloutBatch:
    prompt_tokens: List[int]
    prompt_text: str
    samples: List[Sample]
    expected_answer: str


def compute_pg_loss(log_probs: torch.Tensor, advantages: torch.Tensor, mask: torch.Tensor, num_passes: int = 1,
                    examples_per_rank: int = 1) -> torch.Tensor:
    pg = (log_probs * advantages.unsqueeze(1) * mask).sum()
    pg = pg / (mask.sum() + 1e-8) / (num_passes * examples_per_rank)
    return -pg


def negate_to_log_prob(nll_per_token: torch.Tensor) -> torch.Tensor:
    return -nll_per_token


@dataclass
class GRPOState:
    step: int = 0
    total_steps: int = 1
    total_reward: float = 0.0
    num_rollouts: int = 0

    def get_lr(self, base_lr: float, init_lr_frac: float = 0.05) -> float:
        return base_lr * get_lr_multiplier(self.step, self.total_steps, init_lr_frac)


@dataclass
class StepResult:
    loss: float
    mean_reward: float
    num_sequences: int
    mean_sequence_length: float


def pad_sequence(seq: Sequence[int], target_len: int, pad_value: int) -> List[int]:
    return list(seq[:target_len]) + [pad_value] * max(0, target_len - len(seq))


def create_input_target(full_seq: Sequence[int], pad_token: int = 0) -> Tuple[List[int], List[int]]:
    return list(full_seq[:-1]), list(full_seq[1:])


def create_valid_mask(seq_len: int, padded_len: int) -> List[float]:
    return [1.0] * min(seq_len, padded_len) + [0.0] * max(0, padded_len - seq_len)


@dataclass
class BatchedRollout:
    inputs: torch.Tensor        # int64 [N, T]
    targets: torch.Tensor       # int64 [N, T]
    mask: torch.Tensor          # float [N, T]: 1 on response tokens only
    advantages: torch.Tensor    # float [N]
    rewards: torch.Tensor       # float [N]
    lengths: List[int]


def prepare_batched_rollouts(rollouts: Sequence[RolloutBatch], pad_token: int = 0) -> BatchedRollout:
    """One row per sample: prompt + response, shifted by one; the mask covers response targets only and advantages
    are computed inside each prompt's group."""
    seqs, masks, adv, rew = [], [], [], []
    for rb in rollouts:
        a = compute_advantages([s.reward for s in rb.samples])
        for s, ai in zip(rb.samples, a):
            full = list(rb.prompt_tokens) + list(s.response_tokens)
            seqs.append(full)
            # target position j predicts full[j + 1]; responses start at index len(prompt)
            masks.append([0.0] * (len(rb.prompt_tokens) - 1) + [1.0] * len(s.response_tokens))
            adv.append(ai)
            rew.append(s.reward)
    if not seqs:
        z = torch.zeros(0, 0, dtype=torch.int64)
        return BatchedRollout(z, z, torch.zeros(0, 0), torch.zeros(0), torch.zeros(0), [])
    T = max(len(s) for s in seqs) - 1
    inputs = torch.tensor([pad_sequence(s[:-1], T, pad_token) for s in seqs], dtype=torch.int64)
    targets = torch.tensor([pad_sequence(s[1:], T, pad_token) for s in seqs], dtype=torch.int64)
    mask = torch.tensor([pad_sequence(m, T, 0.0) for m in masks], dtype=torch.float32)
    return BatchedRollout(inputs, targets, mask, torch.tensor(adv), torch.tensor(rew), [len(s) for s in seqs])


def grpo_loss(forward_fn, params, batch: BatchedRollout, device, num_passes: int = 1, examples_per_rank: int = 1) -> torch.Tensor:
    logits = forward_fn(params, batch.inputs.to(device))
    V = logits.shape[-1]
    nll = F.cross_entropy(logits.reshape(-1, V).float(), batch.targets.to(device).reshape(-1), reduction="none").reshape(batch.targets.shape)
    return compute_pg_loss(negate_to_log_prob(nll), batch.advantages.to(device), batch.mask.to(device), num_passes, examples_per_rank)


def grpo_step(forward_fn, params, rollouts: Sequence[RolloutBatch], cfg: GRPOConfig, device="cpu") -> Tuple[StepResult, object]:
    """Loss and gradients for one batch of rollouts, processed in passes of ``device_batch_size`` rows."""
    batch = prepare_batched_rollouts(rollouts, cfg.pad_token)
    n = batch.inputs.shape[0]
    work = ts.make_leaf_params(params)
    ts.zero_grads(work)
    if n == 0:
        return StepResult(0.0, 0.0, 0, 0.0), ts.tree_map(torch.zeros_like, work)
    passes = (n + cfg.device_batch_size - 1) // cfg.device_batch_size
    total = 0.0
    for p in range(passes):
        sl = slice(p * cfg.device_batch_size, (p + 1) * cfg.device_batch_size)
        sub = BatchedRollout(batch.inputs[sl], batch.targets[sl], batch.mask[sl], batch.advantages[sl], batch.rewards[sl], batch.lengths[sl])
        loss = grpo_loss(forward_fn, work, sub, device, passes, max(1, len(rollouts)))
        loss.backward()
        total += float(loss.detach())
    grads = ts.tree_map(lambda p: p.grad if p.grad is not None else torch.zeros_like(p), work)
    res = StepResult(total, float(batch.rewards.mean()), n, sum(batch.lengths) / n)
    return res, grads


@dataclass
class PassKResult:
    pass1: float
    pass_k: float
    k: int


def compute_pass_k(rollouts: Sequence[RolloutBatch], k: int) -> PassKResult:
    n = len(rollouts)
    first = sum(1 for r in rollouts if r.samples and r.samples[0].reward > 0.5)
    anyk = sum(1 for r in rollouts if any(s.reward > 0.5 for s in r.samples[:k]))
    return PassKResult(first / n if n else 0.0, anyk / n if n else 0.0, k)


def format_train_update(result: StepResult, state: GRPOState) -> str:
    return (f"step {state.step:05d}/{state.total_steps} | loss {result.loss:.4f} | reward {result.mean_reward:.3f} | "
            f"seqs {result.num_sequences} | mean len {result.mean_sequence_length:.1f}")


def format_eval_update(p: PassKResult, step: int) -> str:
    return f"step {step:05d} | pass@1 {p.pass1:.3f} | pass@{p.k} {p.pass_k:.3f}"


@dataclass
class Callbacks:
    on_train_step: Callable[[StepResult, GRPOState], None] = lambda r, s: None
    on_eval: Callable[[PassKResult, int], None] = lambda p, step: None

    def combine(self, other: "Callbacks") -> "Callbacks":
        def a(*x):
            self.on_train_step(*x); other.on_train_step(*x)

        def b(*x):
            self.on_eval(*x); other.on_eval(*x)
        return Callbacks(a, b)


def artifact_callbacks(artifacts: rl.RunArtifacts, scope: str = "grpo") -> Callbacks:
    return Callbacks(
        lambda r, s: rl.append_metric_event(artifacts, rl.MetricEvent(scope, s.step, [("loss", r.loss), ("mean_reward", r.mean_reward),
                                                                                      ("num_sequences", r.num_sequences)])),
        lambda p, step: rl.append_metric_event(artifacts, rl.MetricEvent(scope, step, [("pass1", p.pass1), (f"pass{p.k}", p.pass_k)])))


@dataclass
class GenerationConfig:
    max_new_tokens: int = 256
    temperature: float = 1.0
    top_k: Optional[int] = None
    eos_token: int = 2


GenerateOneFn = Callable[[List[int], GenerationConfig, int], List[int]]
"""(prompt tokens, config, sample seed) -> response tokens"""


def generate_sample(generate_one: GenerateOneFn, decode, prompt_tokens, expected: str, gen_cfg: GenerationConfig, seed: int,
                    reward_fn=math_reward) -> Sample:
    toks = generate_one(list(prompt_tokens), gen_cfg, seed)
    text = decode(toks)
    return Sample(list(toks), text, reward_fn(expected, text).reward)


def generate_multiple_samples(generate_one, decode, prompt_tokens, expected, gen_cfg, num_samples: int, base_seed: int = 0,
                              reward_fn=math_reward) -> List[Sample]:
    return [generate_sample(generate_one, decode, prompt_tokens, expected, gen_cfg, base_seed + i, reward_fn) for i in range(num_samples)]


def create_rollout_batch(generate_one, encode, decode, prompt_text: str, expected: str, cfg: GRPOConfig, base_seed: int = 0,
                         reward_fn=math_reward) -> RolloutBatch:
    ptoks = encode(prompt_text)
    gen_cfg = GenerationConfig(cfg.max_new_tokens, cfg.temperature, cfg.top_k, cfg.eos_token)
    return RolloutBatch(ptoks, prompt_text, generate_multiple_samples(generate_one, decode, ptoks, expected, gen_cfg, cfg.num_samples,
                                                                      base_seed, reward_fn), expected)


@dataclass
class TrainResult:
    params: object
    opt_state: object
    state: GRPOState
    history: List[StepResult] = field(default_factory=list)


def train_loop_with_updates(cfg: GRPOConfig, params, forward_fn, make_generate_one: Callable[[object], GenerateOneFn], encode, decode,
                            prompts: Sequence[Tuple[str, str]], num_steps: int, device="cpu", callbacks: Optional[Callbacks] = None,
                            reward_fn=math_reward) -> TrainResult:
    """Each step: take ``examples_per_step / world`` prompts (rank-strided), sample groups with the CURRENT policy,
    compute the policy gradient, average it across ranks, AdamW update with the decaying LR (GRPO.lean:765-943)."""
    callbacks = callbacks or Callbacks()
    distributed = tdist.is_initialized()
    world, rank = (tdist.get_world_size(), tdist.get_rank()) if distributed else (1, 0)
    per_rank = max(1, cfg.examples_per_step // world)
    cur = ts.detach(params)
    opt_state = optim.adamw(lr=cfg.embedding_lr).init(cur)
    state = GRPOState(0, max(1, num_steps))
    hist = []
    for step in range(num_steps):
        state.step = step
        gen = make_generate_one(cur)
        rollouts = []
        for j in range(per_rank):
            pi = (step * cfg.examples_per_step + rank * per_rank + j) % len(prompts)
            text, expected = prompts[pi]
            rollouts.append(create_rollout_batch(gen, encode, decode, text, expected, cfg, base_seed=step * 1000 + j * cfg.num_samples, reward_fn=reward_fn))
        res, grads = grpo_step(forward_fn, cur, rollouts, cfg, device)
        if distributed:
            grads = tdist.all_reduce_grads(grads, tdist.ReduceOp.avg)
        lr = state.get_lr(cfg.embedding_lr, cfg.init_lr_frac)
        with torch.no_grad():
            cur, opt_state = optim.step(optim.adamw(lr=lr, weight_decay=cfg.weight_decay),
                                        cur, grads, opt_state)
        state.total_reward += res.mean_reward
        state.num_rollouts += res.num_sequences
        hist.append(res)
        if cfg.log_every > 0 and step % cfg.log_every == 0:
            callbacks.on_train_step(res, state)
        if cfg.eval_every > 0 and step > 0 and step % cfg.eval_every == 0:
            callbacks.on_eval(compute_pass_k(rollouts, cfg.num_samples), step)
    return TrainResult(cur, opt_state, state, hist)


def train_on_prompts_with_updates(cfg, params, forward_fn, make_generate_one, encode, decode, prompts, num_steps, **kw) -> TrainResult:
    return train_loop_with_updates(cfg, params, forward_fn, make_generate_one, encode, decode, prompts, num_steps, **kw)
