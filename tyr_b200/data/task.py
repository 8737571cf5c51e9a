"""Chat conversations, task mixtures, rendering with an assistant-only loss mask, collation, iterators
(Tyr/Data/Task.lean)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

import torch

SYSTEM, USER, ASSISTANT, TOOL = "system", "user", "assistant", "tool"


@dataclass
class ContentPart:
    type: str                      # "text" | "code:<lang>" | "tool_call:<name>" | "tool_result"
    content: str


@dataclass
class Message:
    role: str
    content: str = ""
    parts: List[ContentPart] = field(default_factory=list)

    @staticmethod
    def text(role: str, content: str) -> "Message":
        return Message(role, content)

    @staticmethod
    def user(content: str) -> "Message":
        return Message(USER, content)

    @staticmethod
    def assistant(content: str) -> "Message":
        return Message(ASSISTANT, content)

    @staticmethod
    def system(content: str) -> "Message":
        return Message(SYSTEM, content)


@dataclass
class Conversation:
    messages: List[Message] = field(default_factory=list)

    def add_message(self, m: Message) -> "Conversation":
        return Conversation(self.messages + [m])

    @staticmethod
    def from_messages(msgs: Sequence[Message]) -> "Conversation":
        return Conversation(list(msgs))


@dataclass
class TokenizedConversation:
    tokens: List[int]
    mask: List[int]                # 1 = train on this token
    source: Conversation


@dataclass
class TaskConfig:
    max_rows: int = 0
    seed: int = 42
    is_validation: bool = False


@dataclass
class LoadedTask:
    name: str
    conversations: List[Conversation]
    config: TaskConfig = field(default_factory=TaskConfig)

    def size(self) -> int:
        return len(self.conversations)

    def get(self, idx: int) -> Conversation:
        return self.conversations[idx] if 0 <= idx < len(self.conversations) else Conversation()


@dataclass
class MixtureEntry:
    task: LoadedTask
    weight: int = 1


_MASK64 = (1 << 64) - 1


def lcg_next(state: int) -> int:
    return (state * 6364136223846793005 + 1442695040888963407) & _MASK64


def shuffle_indices(arr: List, seed: int) -> List:
    """Fisher-Yates with the 64-bit LCG of the reference (Task.lean:137-151): the same seed gives the same order."""
    out = list(arr)
    state = seed & _MASK64
    for i in range(len(out) - 1):
        state = lcg_next(state)
        j = i + state % (len(out) - i)
        out[i], out[j] = out[j], out[i]
    return out


@dataclass
class TaskMixture:
    entries: List[MixtureEntry]
    index_map: List[Tuple[int, int]]
    seed: int = 42

    @staticmethod
    def create(entries: Sequence[MixtureEntry], seed: int = 42) -> "TaskMixture":
        idx = [(ti, ei) for ti, e in enumerate(entries) for _ in range(e.weight) for ei in range(e.task.size())]
        return TaskMixture(list(entries), shuffle_indices(idx, seed), seed)

    def size(self) -> int:
        return len(self.index_map)

    def get(self, idx: int) -> Conversation:
        ti, ei = self.index_map[idx]
        return self.entries[ti].task.get(ei)

    def to_conversation_mixture(self) -> "ConversationMixture":
        return ConversationMixture([self.get(i) for i in range(self.size())], self.seed)


@dataclass
class ConversationMixture:
    conversations: List[Conversation]
    seed: int = 42

    def size(self) -> int:
        return len(self.conversations)

    def get(self, idx: int) -> Conversation:
        return self.conversations[idx]

    def reshuffle(self, seed: int) -> "ConversationMixture":
        return ConversationMixture(shuffle_indices(self.conversations, seed), seed)


@dataclass
class ChatTokens:
    bos: int
    user_start: int
    user_end: int
    assistant_start: int
    assistant_end: int
    python_start: int
    python_end: int
    system_start: int = 0
    system_end: int = 0
    tool_start: int = 0
    tool_end: int = 0
    output_start: int = 0
    output_end: int = 0


def _merge_leading_system(msgs: List[Message]) -> List[Message]:
    if len(msgs) >= 2 and msgs[0].role == SYSTEM and msgs[1].role == USER:
        merged = Message(USER, msgs[0].content + "\n\n" + msgs[1].content, msgs[1].parts)
        return [merged] + msgs[2:]
    return msgs


def render_conversation(conv: Conversation, t: ChatTokens, encode: Callable[[str], List[int]]) -> TokenizedConversation:
    """Only assistant text, python/tool-call spans and the assistant end token are trained on (Task.lean:237-326)."""
    toks, mask = [t.bos], [0]

    def push(ids, m):
        toks.extend(ids)
        mask.extend([m] * len(ids))
    for msg in _merge_leading_system(conv.messages):
        if msg.role in (SYSTEM, USER):
            push([t.user_start], 0); push(encode(msg.content), 0); push([t.user_end], 0)
        elif msg.role == ASSISTANT:
            push([t.assistant_start], 0)
            if not msg.parts:
                push(encode(msg.content), 1)
            for part in msg.parts:
                kind = part.type
                if kind == "text" or (kind.startswith("code:") and kind != "code:python"):
                    push(encode(part.content), 1)
                elif kind == "code:python" or kind.startswith("tool_call"):
                    push([t.python_start], 1); push(encode(part.content), 1); push([t.python_end], 1)
                elif kind == "tool_result":
                    push([t.output_start], 0); push(encode(part.content), 0); push([t.output_end], 0)
            push([t.assistant_end], 1)
        elif msg.role == TOOL:
            push([t.output_start], 0); push(encode(msg.content), 0); push([t.output_end], 0)
    return TokenizedConversation(toks, mask, conv)


@dataclass
class ConversationBatch:
    batch_size: int
    seq_len: int
    tokens: torch.Tensor          # int64 [B, S]
    mask: torch.Tensor            # float32 [B, S]
    lengths: List[int]


def collate(convs: Sequence[TokenizedConversation], max_len: int, pad_token: int = 0) -> ConversationBatch:
    if not convs:
        return ConversationBatch(0, 0, torch.zeros(0, 0, dtype=torch.int64), torch.zeros(0, 0), [])
    S = max(min(len(c.tokens), max_len) for c in convs)
    toks = torch.full((len(convs), S), pad_token, dtype=torch.int64)
    mask = torch.zeros((len(convs), S), dtype=torch.float32)
    lens = []
    for i, c in enumerate(convs):
        n = min(len(c.tokens), S)
        toks[i, :n] = torch.tensor(c.tokens[:n], dtype=torch.int64)
        mask[i, :n] = torch.tensor(c.mask[:n], dtype=torch.float32)
        lens.append(n)
    return ConversationBatch(len(convs), S, toks, mask, lens)


class TaskIterator:
    """Batches of rendered conversations; returns ``None`` at an epoch end and reshuffles for the next one."""

    def __init__(self, mixture: ConversationMixture, batch_size: int, max_seq_len: int, chat_tokens: ChatTokens, encode):
        self.mixture, self.batch_size, self.max_seq_len = mixture, batch_size, max_seq_len
        self.chat_tokens, self.encode = chat_tokens, encode
        self.current_idx, self.epoch = 0, 0

    def next_batch(self) -> Optional[ConversationBatch]:
        if self.current_idx >= self.mixture.size():
            self.mixture = self.mixture.reshuffle(self.mixture.seed + self.epoch + 1)
            self.current_idx, self.epoch = 0, self.epoch + 1
            return None
        end = min(self.current_idx + self.batch_size, self.mixture.size())
        convs = [render_conversation(self.mixture.get(i), self.chat_tokens, self.encode) for i in range(self.current_idx, end)]
        self.current_idx = end
        return collate(convs, self.max_seq_len, self.chat_tokens.assistant_end)

    def reset(self):
        self.current_idx = 0

    def progress(self) -> float:
        return 1.0 if self.mixture.size() == 0 else self.current_idx / self.mixture.size()


class TaskTokenStream:
    """Rank-strided conversations appended to a token buffer; emits ``[B, S]`` input/target windows shifted by one
    (nanochat midtraining, Task.lean:461-575)."""

    def __init__(self, mixture: ConversationMixture, batch_size: int, seq_len: int, chat_tokens: ChatTokens, encode,
                 rank: int = 0, world_size: int = 1):
        self.mixture, self.batch_size, self.seq_len = mixture, batch_size, seq_len
        self.chat_tokens, self.encode = chat_tokens, encode
        self.rank, self.world_size = rank, max(1, world_size)
        self.cursor = rank % mixture.size() if mixture.size() else 0
        self.buffer: List[int] = []
        self.steps = 0
        self.last_wrapped = False
        self.last_progress = 0.0

    def next_gpt_batch(self):
        B, S = self.batch_size, self.seq_len
        if B == 0 or S == 0 or self.mixture.size() == 0:
            return None
        need = B * S + 1
        self.last_wrapped = False
        while len(self.buffer) < need:
            self.buffer.extend(render_conversation(self.mixture.get(self.cursor), self.chat_tokens, self.encode).tokens)
            nxt = self.cursor + self.world_size
            if nxt >= self.mixture.size():
                self.cursor, self.last_wrapped = nxt % self.mixture.size(), True
            else:
                self.cursor = nxt
        window = torch.tensor(self.buffer[:need], dtype=torch.int64)
        del self.buffer[:need - 1]                    # the last token of a window is the first input of the next
        self.steps += 1
        self.last_progress = self.cursor / self.mixture.size()
        return window[:-1].reshape(B, S), window[1:].reshape(B, S)

    def progress(self) -> float:
        return self.last_progress
