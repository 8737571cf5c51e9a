"""Token selection and the cached decode loop shared by all causal LMs (Tyr/Model/Generation.lean)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import torch


@dataclass(frozen=True)
class SamplingStrategy:
    """``greedy`` or ``multinomial(temperature, top_k, top_p)`` (Generation.lean:22-25)."""
    kind: str = "greedy"
    temperature: float = 1.0
    top_k: Optional[int] = None
    top_p: float = 1.0

    @staticmethod
    def greedy() -> "SamplingStrategy":
        return SamplingStrategy("greedy")

    @staticmethod
    def multinomial(temperature: float = 1.0, top_k: Optional[int] = None, top_p: float = 1.0) -> "SamplingStrategy":
        return SamplingStrategy("multinomial", temperature, top_k, top_p)


def top_k_filter(logits: torch.Tensor, k: Optional[int]) -> torch.Tensor:
    if k is None or k <= 0 or k >= logits.shape[-1]:
        return logits
    kth = torch.topk(logits, k, dim=-1).values[..., -1:]
    return logits.masked_fill(logits < kth, float("-inf"))


def top_p_filter(logits: torch.Tensor, p: float) -> torch.Tensor:
    """Keep the smallest prefix of the sorted distribution whose mass reaches ``p`` (the first token always stays)."""
    if p >= 1.0:
        return logits
    sorted_logits, idx = torch.sort(logits, dim=-1, descending=True)
    probs = torch.softmax(sorted_logits, dim=-1)
    cum = probs.cumsum(-1)
    drop = (cum - probs) >= p
    sorted_logits = sorted_logits.masked_fill(drop, float("-inf"))
    return torch.full_like(logits, float("-inf")).scatter(-1, idx, sorted_logits)


def sample_from_logits(logits: torch.Tensor, strategy: SamplingStrategy, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """logits fp32 [B, V] -> int64 [B]."""
    if logits.shape[-1] == 0:
        raise ValueError("greedy sampling requires a nonempty vocabulary")
    if strategy.kind == "greedy":
        return torch.argmax(logits, dim=-1)
    if strategy.temperature <= 0.0:
        raise ValueError(f"multinomial sampling requires temperature > 0, got {strategy.temperature}")
    scaled = logits if strategy.temperature == 1.0 else logits * (1.0 / strategy.temperature)
    filtered = top_p_filter(top_k_filter(scaled, strategy.top_k), strategy.top_p)
    return torch.multinomial(torch.softmax(filtered, dim=-1), 1, generator=generator).reshape(-1)


def token_in_set(tokens: torch.Tensor, values: Sequence[int]) -> torch.Tensor:
    mask = torch.zeros_like(tokens, dtype=torch.bool)
    for v in values:
        mask |= tokens == int(v)
    return mask


def apply_finished_eos(tokens: torch.Tensor, finished: torch.Tensor, eos: int) -> torch.Tensor:
    return torch.where(finished, torch.full_like(tokens, int(eos)), tokens)


StreamCallback = Callable[[int, torch.Tensor], None]


@torch.no_grad()
def generate_cached(prefill: Callable[[torch.Tensor], torch.Tensor], step: Callable[[torch.Tensor], torch.Tensor],
                    input_ids: torch.Tensor, max_new_tokens: int, strategy: SamplingStrategy = SamplingStrategy(),
                    eos_token_ids: Sequence[int] = (), on_step: Optional[StreamCallback] = None,
                    generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """``prefill(ids [B, S]) -> last logits [B, V]``; ``step(tok [B, 1]) -> logits [B, V]``.
    Finished rows keep emitting the first eos id; stops when every row finished or the budget is
    spent (Tyr/Model/Laguna/Model.lean:870-945)."""
    if input_ids.shape[1] == 0:
        raise ValueError("generate requires non-empty prompt sequence")
    if max_new_tokens == 0:
        return input_ids
    logits = prefill(input_ids)
    finished = torch.zeros(input_ids.shape[0], dtype=torch.bool, device=input_ids.device)
    ids = input_ids
    eos = list(eos_token_ids)
    for i in range(max_new_tokens):
        nxt_raw = sample_from_logits(logits.float(), strategy, generator)
        if eos:
            nxt = apply_finished_eos(nxt_raw, finished, eos[0])
            finished = finished | token_in_set(nxt_raw, eos)
        else:
            nxt = nxt_raw
        if on_step is not None:
            on_step(i, nxt)
        ids = torch.cat([ids, nxt.reshape(-1, 1)], dim=1)
        if i + 1 == max_new_tokens or (eos and bool(finished.all())):
            break
        logits = step(nxt.reshape(-1, 1))
    return ids
