"""Position-dependent containers (Tyr/TensorStruct/Indexed.lean:18,68): ``Select`` is a
Bool-indexed choice between two element types, ``IndexedList`` a list whose element type depends
on the position (e.g. layers that alternate between attention kinds)."""
from __future__ import annotations

from typing import Any, Callable, Generic, List, Sequence, TypeVar

A = TypeVar("A")
B = TypeVar("B")


class Select(Generic[A, B]):
    """``Select(True, a)`` holds an ``A``; ``Select(False, b)`` holds a ``B``."""
    __slots__ = ("flag", "value")

    def __init__(self, flag: bool, value):
        self.flag, self.value = bool(flag), value

    def match(self, on_true: Callable[[A], Any], on_false: Callable[[B], Any]):
        return on_true(self.value) if self.flag else on_false(self.value)


class IndexedList:
    """Elements whose kind is decided by ``kind_of(index)``; construction checks each element with
    ``check(kind, element)`` so a mismatching layer list is rejected when it is built."""

    def __init__(self, kind_of: Callable[[int], Any], items: Sequence, check: Callable[[Any, Any], bool] = None):
        self.kind_of = kind_of
        self.items: List = list(items)
        if check is not None:
            for i, it in enumerate(self.items):
                if not check(kind_of(i), it):
                    raise TypeError(f"IndexedList: element {i} does not have kind {kind_of(i)!r}")

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        return self.items[i]

    def kinds(self):
        return [self.kind_of(i) for i in range(len(self.items))]
