"""Stable-prefix consensus for streaming ASR hypotheses: tokens become append-only "stable" text once the last
``confirm_windows`` hypotheses agree on them (minus a rollback margin), when the hypothesis stops changing, or at a
speech boundary; the rest stays mutable (Tyr/Text/StreamingConsensus.lean)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Sequence, Tuple


@dataclass
class ConsensusConfig:
    history_windows: int = 6
    confirm_windows: int = 3
    rollback_tokens: int = 2
    freeze_after_steps: int = 4
    mutable_tail_tokens_while_speech: int = 6


@dataclass
class TextDelta:
    stable_append: str = ""
    unstable_text: str = ""
    full_text: str = ""


def _lcp(a: Sequence[int], b: Sequence[int]) -> int:
    n = 0
    for x, y in zip(a, b):
        if x != y:
            break
        n += 1
    return n


def _consensus_prefix_last_k(hist: List[List[int]], k: int) -> int:
    if k == 0 or len(hist) < k:
        return 0
    w = hist[-k:]
    p = 0
    while p < min(len(h) for h in w) and all(h[p] == w[0][p] for h in w):
        p += 1
    return p


@dataclass
class ConsensusState:
    cfg: ConsensusConfig = field(default_factory=ConsensusConfig)
    stable_ids: List[int] = field(default_factory=list)
    unstable_ids: List[int] = field(default_factory=list)
    history: List[List[int]] = field(default_factory=list)
    last_ids: List[int] = field(default_factory=list)
    unchanged_steps: int = 0

    def update_with_signals(self, ids: Sequence[int], decode: Callable[[List[int]], str], speech_active: bool = True,
                            boundary: bool = False) -> TextDelta:
        cfg, ids = self.cfg, list(ids)
        hist = (self.history + [ids])[-cfg.history_windows:]
        sub = lambda a, b: max(0, a - b)
        c_prev = sub(_lcp(self.last_ids, ids), cfg.rollback_tokens)
        c_hist = sub(_consensus_prefix_last_k(hist, cfg.confirm_windows), cfg.rollback_tokens)
        cand0 = c_hist if len(hist) >= cfg.confirm_windows else c_prev
        unchanged = self.unchanged_steps + 1 if ids == self.last_ids else 0
        freeze = sub(len(ids), cfg.rollback_tokens) if cfg.freeze_after_steps > 0 and unchanged >= cfg.freeze_after_steps else 0
        bound = sub(len(ids), cfg.rollback_tokens) if boundary or not speech_active else 0
        cap = sub(len(ids), cfg.mutable_tail_tokens_while_speech) if speech_active else len(ids)
        cand = min(cap, max(cand0, freeze, bound))
        old = len(self.stable_ids)
        can_advance = _lcp(self.stable_ids, ids) == old          # never rewrite what was already emitted
        if can_advance:
            commit = max(old, cand)
            stable, unstable = ids[:min(commit, len(ids))], ids[commit:]
        else:
            stable, unstable = self.stable_ids, self.unstable_ids
        delta = TextDelta(decode(stable[old:]) if len(stable) > old else "", decode(unstable), decode(stable) + decode(unstable))
        self.stable_ids, self.unstable_ids, self.history, self.last_ids, self.unchanged_steps = stable, unstable, hist, ids, unchanged
        return delta

    def update(self, ids, decode) -> TextDelta:
        return self.update_with_signals(ids, decode, True, False)
