"""Batched generation engine with a per-row state machine: sampled tokens, tool blocks whose result is injected as
forced tokens, end-of-text handling (Examples/NanoChat/Generator/{State,TypedState,Engine}.lean)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

import torch

from ..models.generation import top_k_filter, top_p_filter
from .tools import ToolRegistry


@dataclass
class RowState:
    tokens: List[int]
    forced_tokens: List[int] = field(default_factory=list)
    in_tool_block: bool = False
    tool_input_tokens: List[int] = field(default_factory=list)
    current_tool: Optional[str] = None
    completed: bool = False
    generated_count: int = 0

    @staticmethod
    def from_prompt(prompt: Sequence[int]) -> "RowState":
        return RowState(list(prompt))

    def has_forced_tokens(self) -> bool:
        return bool(self.forced_tokens)

    def pop_forced_token(self) -> Optional[int]:
        return self.forced_tokens.pop(0) if self.forced_tokens else None

    def append_token(self, t: int) -> "RowState":
        self.tokens.append(t)
        self.generated_count += 1
        return self

    def enter_tool_block(self, name: str) -> Optional["RowState"]:
        """Invalid while already inside a tool block (the typed state machine rejects that transition)."""
        if self.in_tool_block:
            return None
        self.in_tool_block, self.tool_input_tokens, self.current_tool = True, [], name
        return self

    def accumulate_tool_token(self, t: int) -> Optional["RowState"]:
        if not self.in_tool_block:
            return None
        self.tool_input_tokens.append(t)
        return self

    def exit_tool_block(self, result_tokens: Sequence[int]) -> Optional["RowState"]:
        if not self.in_tool_block:
            return None
        self.in_tool_block, self.tool_input_tokens, self.current_tool = False, [], None
        self.forced_tokens += list(result_tokens)
        return self

    def mark_complete(self) -> "RowState":
        self.completed = True
        return self

    def last_token(self) -> Optional[int]:
        return self.tokens[-1] if self.tokens else None


@dataclass
class SpecialTokens:
    eot: int
    bot: int
    tool_start: int
    tool_end: int
    output_start: int
    output_end: int
    calc_start: int = -1
    calc_end: int = -1
    prover_start: int = -1
    prover_end: int = -1

    def is_tool_start(self, t: int) -> Optional[str]:
        return {self.tool_start: "generic", self.calc_start: "calculator", self.prover_start: "prover"}.get(t) if t >= 0 else None

    def is_tool_end(self, t: int) -> bool:
        return t >= 0 and t in (self.tool_end, self.calc_end, self.prover_end)

    def is_end_token(self, t: int) -> bool:
        return t == self.eot


@dataclass
class BatchState:
    rows: List[RowState]

    @staticmethod
    def from_prompts(prompts: Sequence[Sequence[int]]) -> "BatchState":
        return BatchState([RowState.from_prompt(p) for p in prompts])

    def all_complete(self) -> bool:
        return all(r.completed for r in self.rows)

    def completed_count(self) -> int:
        return sum(r.completed for r in self.rows)

    def get_next_tokens(self, sampled: Sequence[int]) -> List[int]:
        """Forced tokens (tool output) win over sampled ones."""
        out = []
        for r, s in zip(self.rows, sampled):
            f = r.pop_forced_token()
            out.append(int(s) if f is None else f)
        return out


@dataclass
class SamplingConfig:
    temperature: float = 1.0
    top_p: float = 0.9
    top_k: Optional[int] = None
    max_tokens: int = 256
    stop_tokens: Tuple[int, ...] = ()


def sample_with_config(logits: torch.Tensor, cfg: SamplingConfig, generator: Optional[torch.Generator] = None) -> List[int]:
    if cfg.temperature <= 0.0:
        return torch.argmax(logits, -1).tolist()
    scaled = logits.float() if cfg.temperature == 1.0 else logits.float() / cfg.temperature
    filtered = top_p_filter(top_k_filter(scaled, cfg.top_k), cfg.top_p)
    return torch.multinomial(torch.softmax(filtered, -1), 1, generator=generator).reshape(-1).tolist()


@dataclass
class Engine:
    special_tokens: SpecialTokens
    tool_registry: ToolRegistry = field(default_factory=ToolRegistry)
    sampling_config: SamplingConfig = field(default_factory=SamplingConfig)

    def process_token(self, state: RowState, token: int, decode, encode) -> RowState:
        st = self.special_tokens
        if st.is_end_token(token) or token in self.sampling_config.stop_tokens:
            return state.mark_complete().append_token(token)
        name = st.is_tool_start(token)
        if name is not None:
            state.enter_tool_block(name)
            return state.append_token(token)
        if state.in_tool_block and st.is_tool_end(token):
            res = self.tool_registry.dispatch(decode(state.tool_input_tokens))
            text = res.output if res.success else f"Error: {res.error or 'unknown'}"
            state.exit_tool_block([st.output_start] + list(encode(text)) + [st.output_end])
            return state.append_token(token)
        if state.in_tool_block:
            state.accumulate_tool_token(token)
        return state.append_token(token)

    def generate(self, prompts: Sequence[Sequence[int]], run_model: Callable[[List[int]], torch.Tensor], decode, encode,
                 generator: Optional[torch.Generator] = None) -> List[List[int]]:
        """``run_model(last_tokens) -> logits [B, V]`` advances the model by one token per row."""
        bs = BatchState.from_prompts(prompts)
        for _ in range(self.sampling_config.max_tokens):
            if bs.all_complete():
                break
            logits = run_model([r.last_token() or 0 for r in bs.rows])
            nxt = bs.get_next_tokens(sample_with_config(logits, self.sampling_config, generator))
            for r, t in zip(bs.rows, nxt):
                if not r.completed:
                    self.process_token(r, t, decode, encode)
        return [r.tokens for r in bs.rows]

    def generate_one(self, prompt, run_model, decode, encode, generator=None) -> List[int]:
        return self.generate([prompt], run_model, decode, encode, generator)[0]

    def generate_text(self, prompt_text: str, run_model, decode, encode, generator=None) -> str:
        p = list(encode(prompt_text))
        return decode(self.generate_one(p, run_model, decode, encode, generator)[len(p):])


@dataclass
class EngineConfig:
    temperature: float = 1.0
    top_p: float = 0.9
    top_k: Optional[int] = None
    max_tokens: int = 256

    def create(self, special_tokens: SpecialTokens) -> Engine:
        return Engine(special_tokens, ToolRegistry(), SamplingConfig(self.temperature, self.top_p, self.top_k, self.max_tokens))


def session_runner(session) -> Callable[[List[int]], torch.Tensor]:
    """Adapter from a cached session (``prefill`` / ``step``) to the engine's ``run_model``: the first call prefills
    nothing (the caller prefilled), every call feeds the rows' last tokens."""
    def run(last_tokens: List[int]) -> torch.Tensor:
        dev = session.p["embed"].device if hasattr(session, "p") else "cpu"
        return session.step(torch.tensor(last_tokens, device=dev))
    return run
