"""Schema / flatten / rebuild for tensor trees with leaf paths and roles
(Tyr/TensorStruct/Schema.lean:19-193).  The schema is what checkpoints and the safetensors type
provider agree on: ``[(path, shape, dtype, role)]`` in traversal order."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

import torch

from ..typed.dtype import DType
from ..typed.tensor import Tensor
from .tree import leaves_with_paths, with_leaves


@dataclass(frozen=True)
class LeafSchema:
    path: str
    shape: Tuple[int, ...]
    dtype: DType
    role: str  # "diff" | "frozen"


def schema_of(tree) -> List[LeafSchema]:
    out = []
    for path, leaf, role in leaves_with_paths(tree):
        raw = leaf.raw if isinstance(leaf, Tensor) else leaf
        out.append(LeafSchema(path, tuple(raw.shape), DType.of_torch(raw.dtype), role))
    return out


def flatten(tree) -> Dict[str, torch.Tensor]:
    """path -> raw tensor, in traversal order."""
    return {p: (l.raw if isinstance(l, Tensor) else l) for p, l, _ in leaves_with_paths(tree)}


def rebuild(template, tensors: Dict[str, torch.Tensor], strict: bool = True):
    """Replace the leaves of ``template`` by the tensors named by their paths, validating shape and
    dtype against the template's schema."""
    sch = schema_of(template)
    missing = [s.path for s in sch if s.path not in tensors]
    if missing:
        raise KeyError(f"rebuild: missing leaves {missing[:5]}{'...' if len(missing) > 5 else ''}")
    if strict:
        extra = set(tensors) - {s.path for s in sch}
        if extra:
            raise KeyError(f"rebuild: unexpected leaves {sorted(extra)[:5]}")
    new = []
    tleaves = leaves_with_paths(template)
    for s, (_, tl, _) in zip(sch, tleaves):
        t = tensors[s.path]
        if tuple(t.shape) != s.shape:
            raise ValueError(f"rebuild: {s.path} has shape {list(t.shape)}, expected {list(s.shape)}")
        if DType.of_torch(t.dtype) is not s.dtype:
            raise TypeError(f"rebuild: {s.path} has dtype {t.dtype}, expected {s.dtype}")
        new.append(Tensor.of_raw(t, tl.spec.with_device(tl.spec.device), "rebuild") if isinstance(tl, Tensor) and
                   tl.spec.device.torch == t.device else (Tensor.of_tensor(t) if isinstance(tl, Tensor) else t))
    return with_leaves(template, new)


def diff_schemas(a: Sequence[LeafSchema], b: Sequence[LeafSchema]) -> List[str]:
    """Human-readable differences (used by checkpoint resume checks)."""
    da, db = {s.path: s for s in a}, {s.path: s for s in b}
    out = []
    for p in da:
        if p not in db:
            out.append(f"missing in second: {p}")
        elif (da[p].shape, da[p].dtype) != (db[p].shape, db[p].dtype):
            out.append(f"{p}: {list(da[p].shape)} {da[p].dtype} vs {list(db[p].shape)} {db[p].dtype}")
    out += [f"missing in first: {p}" for p in db if p not in da]
    return out
