"""Tensor and module-tree inspection (the role of Tyr/Widget.lean outside an editor).

The reference renders ``#tensor`` / ``#module`` commands in the Lean infoview from two data models,
``TensorDisplayProps`` and a ``ModuleNode`` tree (Widget.lean:106-130, 773-830).  There is no infoview here, so the same
data models are produced for any tensor tree and rendered as plain text (``render_text``) or as a self-contained HTML
fragment with collapsible groups and a heat-map table for small tensors (``render_html``; ``Tensor._repr_html_`` and
``show`` use it, so notebooks display it directly).  Up to 10 000 values are sampled per tensor, as in the reference.
"""
from __future__ import annotations

import html
import math
from dataclasses import dataclass, field
from typing import Any, List, Optional, Sequence, Tuple, Union

import torch

MAX_VALUES = 10000


@dataclass
class TensorDisplayProps:
    shape: List[int]
    dtype: str
    device: str
    values: List[float]
    requires_grad: bool
    numel: int
    stats: str
    grad_values: Optional[List[float]] = None
    grad_stats: Optional[str] = None
    name: Optional[str] = None
    axis_names: Optional[List[str]] = None


@dataclass
class ModuleNode:
    """kind: "tensor" (``tensor`` set), "group" (``children`` set) or "static" (``value`` set)."""
    kind: str
    name: str
    tensor: Optional[TensorDisplayProps] = None
    children: List[Tuple[str, "ModuleNode"]] = field(default_factory=list)
    value: Optional[str] = None


@dataclass
class ModuleDisplayProps:
    root: ModuleNode


def _raw(t) -> torch.Tensor:
    return t.raw if hasattr(t, "raw") and isinstance(getattr(t, "raw"), torch.Tensor) else t


def _stats(x: torch.Tensor) -> str:
    if x.numel() == 0:
        return "empty"
    if x.dtype == torch.bool:
        return f"true={int(x.sum())}/{x.numel()}"
    if x.is_complex():
        x = x.abs()
    f = x.detach().to(torch.float64) if not x.dtype.is_floating_point or x.dtype.itemsize < 4 else x.detach().double()
    finite = f[torch.isfinite(f)]
    if finite.numel() == 0:
        return "no finite values"
    s = f"min={float(finite.min()):.4g} max={float(finite.max()):.4g} mean={float(finite.mean()):.4g} std={float(finite.std(unbiased=False)):.4g}"
    bad = f.numel() - finite.numel()
    return s + (f" non-finite={bad}" if bad else "")


def _values(x: torch.Tensor, limit: int = MAX_VALUES) -> List[float]:
    flat = x.detach().reshape(-1)[:limit]
    if flat.is_complex():
        flat = flat.abs()
    return flat.to("cpu", torch.float64).tolist()


def tensor_to_props(t, name: Optional[str] = None, axis_names: Sequence[str] = ()) -> TensorDisplayProps:
    x = _raw(t)
    grad = x.grad if (x.requires_grad and x.is_leaf) else None
    return TensorDisplayProps(
        shape=list(x.shape), dtype=str(x.dtype).replace("torch.", ""), device=str(x.device), values=_values(x),
        requires_grad=bool(x.requires_grad), numel=x.numel(), stats=_stats(x),
        grad_values=_values(grad) if grad is not None else None, grad_stats=_stats(grad) if grad is not None else None,
        name=name, axis_names=list(axis_names) or None)


def to_module_node(value: Any, name: str = "root") -> ModuleNode:
    """Any tensor tree (dataclasses marked ``@tensor_struct``, tuples, lists, dicts, ``Vector``, ``Frozen``, ``Static``,
    optionals, scalars) -> display tree."""
    from ..struct import tree as T
    if T.is_leaf(value):
        return ModuleNode("tensor", name, tensor=tensor_to_props(value, name))
    if value is None:
        return ModuleNode("group", f"{name} (none)")
    if isinstance(value, T.Static):
        return ModuleNode("static", name, value=repr(value.val))
    if isinstance(value, T.Frozen):
        inner = to_module_node(value.tensor, name)
        inner.name = f"{name} (frozen)"
        return inner
    ch = None if T._is_meta(value) else T._children(value)
    if ch is None:
        return ModuleNode("static", name, value=repr(value))
    kind, keys, vals, _ = ch
    tag = kind[0] if isinstance(kind, tuple) else kind
    label = name
    if tag in ("list", "tuple", "vector"):
        label = f"{name} [{len(vals)}]"
        keys = [f"[{k}]" for k in keys]
    elif tag == "dataclass":
        label = f"{name}: {type(value).__name__}"
    return ModuleNode("group", label, children=[(str(k), to_module_node(v, str(k))) for k, v in zip(keys, vals)])


def to_module_display_props(value: Any, name: str = "root") -> ModuleDisplayProps:
    return ModuleDisplayProps(to_module_node(value, name))


# ---- text --------------------------------------------------------------------------------------------------------------
def _tensor_line(p: TensorDisplayProps) -> str:
    g = " grad" if p.requires_grad else ""
    ax = f" axes={p.axis_names}" if p.axis_names else ""
    return f"{p.dtype}{p.shape} on {p.device}{g}{ax}  {p.stats}"


def render_text(node: Union[ModuleNode, ModuleDisplayProps, Any], indent: str = "") -> str:
    if isinstance(node, ModuleDisplayProps):
        node = node.root
    elif not isinstance(node, ModuleNode):
        node = to_module_node(node)
    if node.kind == "tensor":
        out = f"{indent}{node.name}: {_tensor_line(node.tensor)}"
        if node.tensor.grad_stats:
            out += f"\n{indent}  grad: {node.tensor.grad_stats}"
        return out
    if node.kind == "static":
        return f"{indent}{node.name} = {node.value}"
    lines = [f"{indent}{node.name}"]
    for _, child in node.children:
        lines.append(render_text(child, indent + "  "))
    return "\n".join(lines)


def count_parameters(node: Union[ModuleNode, ModuleDisplayProps]) -> int:
    if isinstance(node, ModuleDisplayProps):
        node = node.root
    if node.kind == "tensor":
        return node.tensor.numel
    return sum(count_parameters(c) for _, c in node.children)


# ---- HTML --------------------------------------------------------------------------------------------------------------
def _colour(v: float, lo: float, hi: float) -> str:
    if not math.isfinite(v):
        return "#000000"
    m = max(abs(lo), abs(hi), 1e-30)
    a = max(-1.0, min(1.0, v / m))
    # diverging blue (negative) - white - red (positive)
    if a >= 0:
        r, g, b = 255, int(255 * (1 - a)), int(255 * (1 - a))
    else:
        r, g, b = int(255 * (1 + a)), int(255 * (1 + a)), 255
    return f"#{r:02x}{g:02x}{b:02x}"


def _heatmap(p: TensorDisplayProps, max_cells: int = 4096) -> str:
    if not p.values or p.numel > max_cells or len(p.values) < p.numel:
        return ""
    cols = p.shape[-1] if p.shape else 1
    rows = max(1, p.numel // max(cols, 1))
    finite = [v for v in p.values if math.isfinite(v)] or [0.0]
    lo, hi = min(finite), max(finite)
    out = ['<table style="border-collapse:collapse;margin:4px 0">']
    for r in range(rows):
        out.append("<tr>")
        for c in range(cols):
            v = p.values[r * cols + c]
            out.append(f'<td title="{v:.6g}" style="width:6px;height:6px;padding:0;background:{_colour(v, lo, hi)}"></td>')
        out.append("</tr>")
    out.append("</table>")
    return "".join(out)


def render_html(node: Union[ModuleNode, ModuleDisplayProps, Any]) -> str:
    if isinstance(node, ModuleDisplayProps):
        node = node.root
    elif not isinstance(node, ModuleNode):
        node = to_module_node(node)
    esc = html.escape
    if node.kind == "tensor":
        p = node.tensor
        body = f"<code>{esc(node.name)}</code>: <code>{esc(_tensor_line(p))}</code>"
        if p.grad_stats:
            body += f"<br><small>grad: {esc(p.grad_stats)}</small>"
        return f'<div style="font-family:monospace">{body}{_heatmap(p)}</div>'
    if node.kind == "static":
        return f'<div style="font-family:monospace"><code>{esc(node.name)}</code> = <code>{esc(node.value or "")}</code></div>'
    inner = "".join(render_html(c) for _, c in node.children)
    n = count_parameters(node)
    return (f'<details open style="margin-left:12px;font-family:monospace"><summary>{esc(node.name)}'
            f' <small>({n:,} elements)</small></summary>{inner}</details>')


class Display:
    """Return value of :func:`show`: prints as text, renders as HTML in a notebook."""

    def __init__(self, props: ModuleDisplayProps):
        self.props = props

    def __repr__(self):
        return render_text(self.props)

    def _repr_html_(self):
        return render_html(self.props)


def show(value: Any, name: str = "root") -> Display:
    """``#tensor`` / ``#module`` for a Python session: ``show(model)`` or ``show(tensor, "w")``."""
    return Display(to_module_display_props(value, name))
