"""TensorStruct: generic traversal of tensor trees (the reference's ``TensorStruct`` class and
its ``deriving`` handlers, Tyr/TensorStruct.lean:155-704, Tyr/Module/Derive.lean:291-312).

A tensor tree is built from

* leaves: typed ``Tensor`` (or raw ``torch.Tensor``),
* ``Frozen(tensor)``: takes part in ``map`` (device/dtype moves) but not in gradient utilities,
* ``Static(value)``: metadata, skipped entirely,
* containers: ``@tensor_struct`` dataclasses, tuples, lists, dicts, ``Vector`` (fixed length),
  ``None`` (an absent optional), Python scalars / strings (metadata).

``map / map_m / zip_with / fold`` mirror the class methods; ``zip_with`` requires both trees to
have the same structure (``Vector`` lengths, dict keys, optional presence) and raises otherwise.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict, Generic, Iterable, List, Optional, Sequence, TypeVar

import torch

from ..typed import ops as O
from ..typed.tensor import Tensor

T = TypeVar("T")


class Static(Generic[T]):
    """Non-tensor data skipped by every traversal."""
    __slots__ = ("val",)

    def __init__(self, val: T):
        self.val = val

    def __eq__(self, other):
        return isinstance(other, Static) and self.val == other.val

    def __hash__(self):
        return hash(("Static", self.val)) if not isinstance(self.val, (dict, list)) else id(self)

    def __repr__(self):
        return f"Static({self.val!r})"


class Frozen:
    """A tensor that participates in the forward pass but is not trained."""
    __slots__ = ("tensor",)

    def __init__(self, tensor):
        self.tensor = tensor

    def map(self, f):
        return Frozen(f(self.tensor))

    def get(self):
        return self.tensor

    def __repr__(self):
        return f"Frozen({self.tensor!r})"


class Vector(Generic[T]):
    """Length-indexed array: ``zip_with`` on two vectors checks the lengths agree."""
    __slots__ = ("n", "data")

    def __init__(self, n: int, data: Sequence[T]):
        data = list(data)
        if len(data) != n:
            raise ValueError(f"Vector: expected {n} elements, got {len(data)}")
        self.n, self.data = n, data

    @staticmethod
    def replicate(n: int, a: T) -> "Vector[T]":
        return Vector(n, [a] * n)

    @staticmethod
    def empty() -> "Vector[T]":
        return Vector(0, [])

    def push(self, a: T) -> "Vector[T]":
        return Vector(self.n + 1, self.data + [a])

    def get(self, i: int) -> T:
        if not 0 <= i < self.n:
            raise IndexError(f"Vector index {i} out of range for length {self.n}")
        return self.data[i]

    def set(self, i: int, a: T) -> "Vector[T]":
        self.get(i)
        d = list(self.data)
        d[i] = a
        return Vector(self.n, d)

    def to_list(self) -> List[T]:
        return list(self.data)

    def __len__(self):
        return self.n

    def __iter__(self):
        return iter(self.data)

    def __repr__(self):
        return f"Vector({self.n}, {self.data!r})"


_STRUCT_FLAG = "__tensor_struct__"
_MODEL_FLAG = "__tyr_model__"


def tensor_struct(cls=None, *, model: bool = False):
    """Class decorator: makes a dataclass (creating it if needed) traversable.  ``model=True``
    additionally marks it as a ``Model`` (schema + flatten available, like ``deriving Model``)."""
    def wrap(c):
        if not dataclasses.is_dataclass(c):
            c = dataclasses.dataclass(c)
        setattr(c, _STRUCT_FLAG, True)
        if model:
            setattr(c, _MODEL_FLAG, True)
        return c
    return wrap(cls) if cls is not None else wrap


def model(cls):
    return tensor_struct(cls, model=True)


def is_leaf(x) -> bool:
    return isinstance(x, (Tensor, torch.Tensor))


def _is_meta(x) -> bool:
    return x is None or isinstance(x, (Static, bool, int, float, str, bytes, complex)) or callable(x) and not is_leaf(x) and not dataclasses.is_dataclass(x)


def _children(x):
    """(kind, keys, values, rebuild) for a container."""
    if isinstance(x, Frozen):
        return "frozen", [None], [x.tensor], lambda vs: Frozen(vs[0])
    if isinstance(x, Vector):
        return ("vector", x.n), list(range(x.n)), x.data, lambda vs: Vector(x.n, vs)
    if isinstance(x, tuple) and hasattr(x, "_fields"):
        return ("namedtuple", type(x)), list(x._fields), list(x), lambda vs: type(x)(*vs)
    if isinstance(x, tuple):
        return ("tuple", len(x)), list(range(len(x))), list(x), lambda vs: tuple(vs)
    if isinstance(x, list):
        return ("list", len(x)), list(range(len(x))), list(x), lambda vs: list(vs)
    if isinstance(x, dict):
        ks = list(x.keys())
        return ("dict", tuple(ks)), ks, [x[k] for k in ks], lambda vs: dict(zip(ks, vs))
    if dataclasses.is_dataclass(x) and not isinstance(x, type):
        fs = [f.name for f in dataclasses.fields(x)]
        return ("dataclass", type(x)), fs, [getattr(x, f) for f in fs], lambda vs: dataclasses.replace(x, **dict(zip(fs, vs)))
    return None


def tree_map(f: Callable, tree, *, include_frozen: bool = True):
    if is_leaf(tree):
        return f(tree)
    if _is_meta(tree):
        return tree
    ch = _children(tree)
    if ch is None:
        raise TypeError(f"TensorStruct: {type(tree).__name__} is not a tensor tree (wrap metadata in Static)")
    kind, _, vals, rebuild = ch
    if kind == "frozen" and not include_frozen:
        return tree
    return rebuild([tree_map(f, v, include_frozen=include_frozen) for v in vals])


map_ = tree_map
map_m = tree_map  # effects are ordinary Python; kept for API parity


def zip_with(f: Callable, a, b, *, include_frozen: bool = True):
    if is_leaf(a):
        if not is_leaf(b):
            raise TypeError("TensorStruct.zipWith: structures differ (leaf vs container)")
        return f(a, b)
    if _is_meta(a):
        return a
    ca, cb = _children(a), _children(b)
    if ca is None or cb is None or ca[0] != cb[0]:
        raise TypeError(f"TensorStruct.zipWith: structures differ ({type(a).__name__} vs {type(b).__name__})")
    if ca[0] == "frozen" and not include_frozen:
        return a
    return ca[3]([zip_with(f, x, y, include_frozen=include_frozen) for x, y in zip(ca[2], cb[2])])


def fold(f: Callable, init, tree, *, include_frozen: bool = True):
    acc = init
    for leaf in leaves(tree, include_frozen=include_frozen):
        acc = f(leaf, acc)
    return acc


def leaves(tree, *, include_frozen: bool = True) -> List:
    out = []

    def visit(t):
        if is_leaf(t):
            out.append(t)
        elif _is_meta(t):
            return
        else:
            ch = _children(t)
            if ch is None:
                raise TypeError(f"TensorStruct: {type(t).__name__} is not a tensor tree")
            if ch[0] == "frozen" and not include_frozen:
                return
            for v in ch[2]:
                visit(v)
    visit(tree)
    return out


def leaves_with_paths(tree, prefix: str = "", *, include_frozen: bool = True):
    """[(path, leaf, role)] with dotted paths; role is 'diff' or 'frozen'."""
    out = []

    def visit(t, path, role):
        if is_leaf(t):
            out.append((path, t, role))
        elif _is_meta(t):
            return
        else:
            kind, keys, vals, _ = _children(t)
            if kind == "frozen":
                if include_frozen:
                    visit(vals[0], path, "frozen")
                return
            for k, v in zip(keys, vals):
                visit(v, f"{path}.{k}" if path else str(k), role)
    visit(tree, prefix, "diff")
    return out


def with_leaves(template, new_leaves: Sequence, *, include_frozen: bool = True):
    """Rebuild ``template`` with leaves replaced in traversal order (count is checked)."""
    it = iter(new_leaves)
    n = [0]

    def nxt(_):
        n[0] += 1
        try:
            return next(it)
        except StopIteration:
            raise ValueError("TensorStruct.withLeaves: missing leaf") from None
    res = tree_map(nxt, template, include_frozen=include_frozen)
    if len(list(it)) != 0:
        raise ValueError("TensorStruct.withLeaves: unexpected extra leaves")
    return res


# -- utilities (TensorStruct namespace of the reference) -------------------------------------------
def _raw(t):
    return t.raw if isinstance(t, Tensor) else t


def _like(t, raw):
    return Tensor.of_raw(raw, t.spec, "TensorStruct") if isinstance(t, Tensor) else raw


def count(tree) -> int:
    return fold(lambda _, n: n + 1, 0, tree)


def grads(tree):
    """Independent gradient snapshots for all (non-frozen) leaves; missing gradients are zeros."""
    def g(t):
        r = _raw(t)
        gr = r.grad
        return _like(t, gr.detach().clone() if gr is not None else torch.zeros_like(r))
    return tree_map(g, tree, include_frozen=False)


def zero_grads(tree, set_to_none: bool = True) -> None:
    for t in leaves(tree):
        r = _raw(t)
        if set_to_none:
            r.grad = None
        elif r.grad is not None:
            r.grad.zero_()


def detach(tree):
    return tree_map(lambda t: _like(t, _raw(t).detach()), tree)


def requires_grad(tree, flag: bool):
    return tree_map(lambda t: _like(t, _raw(t).detach().requires_grad_(flag)), tree, include_frozen=False)


def make_leaf_params(tree):
    """Independent trainable leaf parameters throughout the tree (frozen leaves stay as they are)."""
    return tree_map(lambda t: _like(t, _raw(t).detach().clone().requires_grad_(True)), tree, include_frozen=False)


def grad(output, inputs, cotangent=None, retain_graph: Optional[bool] = None, create_graph: bool = False):
    """Differentiate ``output`` w.r.t. every leaf in ONE engine call; unused leaves get zeros."""
    ls = leaves(inputs, include_frozen=False)
    raws = [_raw(t) for t in ls]
    go = _raw(cotangent) if cotangent is not None else None
    rg = create_graph if retain_graph is None else retain_graph
    gs = torch.autograd.grad(_raw(output), raws, go, retain_graph=rg, create_graph=create_graph, allow_unused=True)
    if len(gs) != len(ls):
        raise RuntimeError("TensorStruct.grad: unexpected gradient leaves")
    new = [_like(t, g if g is not None else torch.zeros_like(r)) for t, r, g in zip(ls, raws, gs)]
    return with_leaves(inputs, new, include_frozen=False)


def functional_grad(f: Callable, inputs):
    """First derivatives of a scalar-valued function over a tensor tree.  Fresh differentiation
    variables live inside the call; only detached gradients escape; no ``.grad`` is mutated."""
    ls = leaves(inputs, include_frozen=False)
    for t in ls:
        if not _raw(t).dtype.is_floating_point:
            raise TypeError("functionalGrad: every differentiated leaf must be floating")
    fresh = [_like(t, _raw(t).detach().clone().requires_grad_(True)) for t in ls]
    out = f(with_leaves(inputs, fresh, include_frozen=False))
    gs = torch.autograd.grad(_raw(out), [_raw(t) for t in fresh], allow_unused=True)
    new = [_like(t, (g if g is not None else torch.zeros_like(_raw(t))).detach()) for t, g in zip(ls, gs)]
    return with_leaves(inputs, new, include_frozen=False)


def _floating_check(tree):
    for t in leaves(tree):
        if not _raw(t).dtype.is_floating_point:
            raise TypeError("FloatingTensorStruct: every leaf must have a real floating dtype")


def scale(tree, s: float):
    _floating_check(tree)
    return tree_map(lambda t: _like(t, _raw(t) * s), tree)


def add(a, b):
    _floating_check(a)
    return zip_with(lambda x, y: _like(x, _raw(x) + _raw(y)), a, b)


def sub(a, b):
    _floating_check(a)
    return zip_with(lambda x, y: _like(x, _raw(x) - _raw(y)), a, b)


def all_(p: Callable, tree) -> bool:
    return fold(lambda t, acc: acc and bool(p(t)), True, tree)


def any_(p: Callable, tree) -> bool:
    return fold(lambda t, acc: acc or bool(p(t)), False, tree)
