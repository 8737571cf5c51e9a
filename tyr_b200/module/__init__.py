"""Module layer (Tyr/Module/*.lean).

``Module`` / ``ModuleIO`` / ``ModuleCtx`` are protocols: a module is a tensor tree (a
``@tensor_struct`` dataclass) with a ``forward``; ``ModuleIO`` may have effects (dropout, sampling),
``ModuleCtx`` additionally takes a context such as ``TrainingCtx`` (Core.lean:77-139).  Layers:
``Linear`` (Kaiming init, PyTorch ``[out, in]`` weights), ``LayerNorm``, ``RMSNorm`` (2-D..5-D
inputs), ``Affine`` and ``Conv2d``; all are typed at the API boundary and route bf16 CUDA inputs
to the hand-written kernels.  ``module_display`` is the text form of ``deriving ToModuleDisplay``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Protocol, Tuple, runtime_checkable

import torch

from ..struct import Static, tensor_struct
from ..struct import tree as ts
from ..typed import DType, Device, StaticSpec, Tensor
from ..typed import neural as N
from ..typed import ops as O


@runtime_checkable
class Module(Protocol):
    def forward(self, x): ...


@runtime_checkable
class ModuleIO(Protocol):
    def forward(self, x): ...


@runtime_checkable
class ModuleCtx(Protocol):
    def forward(self, ctx, x): ...


@dataclass(frozen=True)
class TrainingCtx:
    training: bool = True
    dropout_p: float = 0.0

    @staticmethod
    def train() -> "TrainingCtx":
        return TrainingCtx(True)

    @staticmethod
    def eval() -> "TrainingCtx":
        return TrainingCtx(False, 0.0)

    def with_dropout(self, p: float) -> "TrainingCtx":
        return TrainingCtx(self.training, p if self.training else 0.0)


def apply(m, x):
    """``m |> x``."""
    return m.forward(x)


def apply_ctx(m, ctx, x):
    return m.forward(ctx, x)


@tensor_struct
class Linear:
    weight: Tensor
    bias: Optional[Tensor] = None

    @staticmethod
    def init(in_dim: int, out_dim: int, with_bias: bool = True, device: Device = Device.CPU,
             dtype: DType = DType.Float32, generator=None) -> "Linear":
        std = math.sqrt(2.0 / in_dim)
        w = O.parameter(O.mul_scalar(O.randn((out_dim, in_dim), dtype, device, generator=generator), std))
        b = O.parameter(O.zeros((out_dim,), dtype, device)) if with_bias else None
        return Linear(w, b)

    def forward(self, x: Tensor) -> Tensor:
        return O.linear(x, self.weight, self.bias)

    forward2d = forward
    forward3d = forward


@tensor_struct
class LayerNorm:
    weight: Tensor
    bias: Tensor
    eps: Static = field(default_factory=lambda: Static(1e-5))

    @staticmethod
    def init(dim: int, eps: float = 1e-5, device: Device = Device.CPU, dtype: DType = DType.Float32) -> "LayerNorm":
        return LayerNorm(O.parameter(O.ones((dim,), dtype, device)), O.parameter(O.zeros((dim,), dtype, device)), Static(eps))

    def forward(self, x: Tensor) -> Tensor:
        return O.layer_norm(x, self.weight, self.bias, self.eps.val)


@tensor_struct
class RMSNorm:
    weight: Tensor
    eps: Static = field(default_factory=lambda: Static(1e-6))

    @staticmethod
    def init(dim: int, eps: float = 1e-6, device: Device = Device.CPU, dtype: DType = DType.Float32) -> "RMSNorm":
        return RMSNorm(O.parameter(O.ones((dim,), dtype, device)), Static(eps))

    def forward(self, x: Tensor) -> Tensor:
        """Any rank 2..5: normalises the last dimension, result keeps the input dtype."""
        if not 2 <= x.spec.rank <= 5:
            raise TypeError(f"RMSNorm: expects a 2-D..5-D input, got rank {x.spec.rank}")
        return N.rms_norm_preserving(x, self.weight, self.eps.val)


@tensor_struct
class Affine:
    """y = x * scale + shift, broadcast over the last dimension."""
    scale: Tensor
    shift: Tensor

    @staticmethod
    def init(dim: int, device: Device = Device.CPU, dtype: DType = DType.Float32) -> "Affine":
        return Affine(O.parameter(O.ones((dim,), dtype, device)), O.parameter(O.zeros((dim,), dtype, device)))

    def forward(self, x: Tensor) -> Tensor:
        return O.add(O.mul(x, self.scale), self.shift)


@tensor_struct
class Conv2d:
    weight: Tensor
    bias: Optional[Tensor] = None
    stride: Static = field(default_factory=lambda: Static((1, 1)))
    padding: Static = field(default_factory=lambda: Static((0, 0)))

    @staticmethod
    def init(in_ch: int, out_ch: int, kernel: Tuple[int, int], stride=(1, 1), padding=(0, 0), with_bias: bool = True,
             device: Device = Device.CPU, dtype: DType = DType.Float32, generator=None) -> "Conv2d":
        fan_in = in_ch * kernel[0] * kernel[1]
        w = O.parameter(O.mul_scalar(O.randn((out_ch, in_ch) + tuple(kernel), dtype, device, generator=generator),
                                     math.sqrt(2.0 / fan_in)))
        b = O.parameter(O.zeros((out_ch,), dtype, device)) if with_bias else None
        return Conv2d(w, b, Static(tuple(stride)), Static(tuple(padding)))

    def forward(self, x: Tensor) -> Tensor:
        return O.conv2d(x, self.weight, self.bias, self.stride.val, self.padding.val)


@tensor_struct
class Dropout:
    """ModuleCtx example: behaves differently in training and inference."""
    p: Static = field(default_factory=lambda: Static(0.1))

    def forward(self, ctx: TrainingCtx, x: Tensor) -> Tensor:
        return O.dropout(x, ctx.dropout_p if ctx.dropout_p else self.p.val, ctx.training)


def module_display(m, name: str = "", indent: int = 0) -> str:
    """Text rendering of a module tree with leaf specs and parameter counts (the terminal form of
    the reference's infoview ``#module`` widget, Tyr/Widget.lean)."""
    pad = "  " * indent
    lines = []
    total = 0
    for path, leaf, role in ts.leaves_with_paths(m):
        raw = leaf.raw if isinstance(leaf, Tensor) else leaf
        total += raw.numel()
        lines.append(f"{pad}  {path}: {str(raw.dtype).replace('torch.', '')}{list(raw.shape)}"
                     f"{' (frozen)' if role == 'frozen' else ''}")
    head = f"{pad}{name or type(m).__name__} ({total:,} parameters)"
    return "\n".join([head] + lines)


def tensor_display(t, max_items: int = 8) -> str:
    """Terminal form of ``#tensor``: spec, statistics and the first values."""
    raw = t.raw if isinstance(t, Tensor) else t
    f = raw.detach().float().reshape(-1)
    stats = f"min={f.min():.4g} max={f.max():.4g} mean={f.mean():.4g} std={f.std():.4g}" if f.numel() > 1 else ""
    vals = ", ".join(f"{v:.4g}" for v in f[:max_items].tolist())
    return f"Tensor {str(raw.dtype).replace('torch.', '')}{list(raw.shape)} on {raw.device} {stats} [{vals}{', ...' if f.numel() > max_items else ''}]"
