"""Evaluation tasks as an open interface, type-erased boxes and evaluable mixtures (Tyr/Data/TaskClass.lean)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

from .task import Conversation, ConversationMixture, shuffle_indices

CATEGORICAL, GENERATIVE = "categorical", "generative"


@dataclass
class EvalResult:
    correct: bool
    score: float
    expected: str
    predicted: str


class EvalTask:
    """Subclass and fill in; ``reward`` defaults to the evaluation score."""
    name: str = "task"

    def eval_type(self) -> str:
        return GENERATIVE

    def size(self) -> int:
        raise NotImplementedError

    def get_example(self, idx: int) -> Optional[Conversation]:
        raise NotImplementedError

    def evaluate(self, conv: Conversation, response: str) -> EvalResult:
        raise NotImplementedError

    def reward(self, conv: Conversation, response: str) -> float:
        return self.evaluate(conv, response).score


@dataclass
class BoxedTask:
    """Type-erased task: just the operations."""
    name: str
    eval_type: str
    size: int
    get_example: Callable[[int], Optional[Conversation]]
    evaluate: Callable[[Conversation, str], EvalResult]
    reward: Callable[[Conversation, str], float]


def box_task(task: EvalTask) -> BoxedTask:
    return BoxedTask(task.name, task.eval_type(), task.size(), task.get_example, task.evaluate, task.reward)


@dataclass
class TaskEntry:
    task: BoxedTask
    weight: int = 1


def entry(task: EvalTask, weight: int = 1) -> TaskEntry:
    return TaskEntry(box_task(task), weight)


@dataclass
class GenericTaskMixture:
    entries: List[TaskEntry]
    index_map: List[Tuple[int, int]]
    seed: int = 42

    @staticmethod
    def create(entries: Sequence[TaskEntry], seed: int = 42) -> "GenericTaskMixture":
        idx = [(ti, ei) for ti, e in enumerate(entries) for _ in range(e.weight) for ei in range(e.task.size)]
        return GenericTaskMixture(list(entries), shuffle_indices(idx, seed), seed)

    def size(self) -> int:
        return len(self.index_map)

    def get_example(self, index: int) -> Optional[Conversation]:
        if not 0 <= index < len(self.index_map):
            return None
        ti, ei = self.index_map[index]
        return self.entries[ti].task.get_example(ei)

    def evaluate(self, index: int, response: str) -> Optional[EvalResult]:
        conv = self.get_example(index)
        return None if conv is None else self.entries[self.index_map[index][0]].task.evaluate(conv, response)

    def reward(self, index: int, response: str) -> float:
        conv = self.get_example(index)
        return 0.0 if conv is None else self.entries[self.index_map[index][0]].task.reward(conv, response)

    def to_conversation_mixture(self) -> ConversationMixture:
        return ConversationMixture([c for c in (self.get_example(i) for i in range(self.size())) if c is not None], self.seed)

    def to_conversation_mixture_sharded(self, rank: int, world_size: int) -> ConversationMixture:
        return ConversationMixture([c for i in range(rank, self.size(), max(1, world_size))
                                    if (c := self.get_example(i)) is not None], self.seed)


def mixture_same(tasks: Sequence[BoxedTask], seed: int = 42) -> GenericTaskMixture:
    return GenericTaskMixture.create([TaskEntry(t, 1) for t in tasks], seed)


def mixture_weighted(entries: Sequence[TaskEntry], seed: int = 42) -> GenericTaskMixture:
    return GenericTaskMixture.create(entries, seed)
