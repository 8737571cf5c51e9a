"""``Tensor``: a torch tensor paired with the ``StaticSpec`` it claims.

Every native result re-enters through ``Tensor.of_raw`` which compares the runtime shape, dtype
and device with the claimed spec and raises on mismatch (the reference aborts:
Tyr/Basic.lean:115-138).  Existential packages ``SomeDTypeTensor`` / ``ShapePackedTensor`` carry
a tensor whose dtype / shape is only known at run time (Tyr/Typed/Tensor.lean:82,
Tyr/TensorStruct.lean:335).
"""
from __future__ import annotations

import threading
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import shape as sh
from .device import Device
from .dtype import DType
from .spec import StaticSpec

_live = [0]
_live_lock = threading.Lock()


class SpecMismatch(TypeError):
    """Raised when a runtime tensor does not have the shape/dtype/device its type claims."""


class Tensor:
    __slots__ = ("raw", "spec", "__weakref__")

    def __init__(self, raw: torch.Tensor, spec: StaticSpec, _checked: bool = False):
        if not _checked:
            _check(raw, spec, "Tensor")
        self.raw = raw
        self.spec = spec
        with _live_lock:
            _live[0] += 1

    def __del__(self):
        try:
            with _live_lock:
                _live[0] -= 1
        except Exception:
            pass

    # -- construction --------------------------------------------------------------------------
    @staticmethod
    def of_raw(raw: torch.Tensor, spec: StaticSpec, op: str = "ofRaw!") -> "Tensor":
        _check(raw, spec, op)
        return Tensor(raw, spec, _checked=True)

    @staticmethod
    def of_tensor(raw: torch.Tensor) -> "Tensor":
        """Admit a runtime tensor at the spec it actually has."""
        return Tensor(raw, spec_of(raw), _checked=True)

    @staticmethod
    def zeros_for(spec: StaticSpec) -> "Tensor":
        sh.validate_allocation(spec.shape)
        return Tensor(torch.zeros(spec.shape, dtype=spec.dtype.torch, device=spec.device.torch), spec, True)

    # -- views of the claim ------------------------------------------------------------------------
    @property
    def shape(self) -> sh.Shape:
        return self.spec.shape

    @property
    def dtype(self) -> DType:
        return self.spec.dtype

    @property
    def device(self) -> Device:
        return self.spec.device

    def at_dtype(self, dtype: DType) -> Optional["Tensor"]:
        """``self`` if it has exactly this dtype (no conversion)."""
        return self if self.spec.dtype is dtype else None

    def at_device(self, device: Device) -> Optional["Tensor"]:
        return self if self.spec.device == device else None

    def same_device(self, other: "Tensor") -> bool:
        return self.spec.device == other.spec.device

    def pack_dtype(self) -> "SomeDTypeTensor":
        return SomeDTypeTensor(self.spec.shape, self.spec.device, self)

    def pack_shape(self) -> "ShapePackedTensor":
        return ShapePackedTensor(self.spec.dtype, self.spec.device, self)

    # -- conversions -----------------------------------------------------------------------------
    def to(self, device: Device) -> "Tensor":
        return Tensor.of_raw(self.raw.to(device.torch), self.spec.with_device(device), "to")

    def cast(self, dtype: DType) -> "Tensor":
        return Tensor.of_raw(self.raw.to(dtype.torch), self.spec.with_dtype(dtype), "castDType")

    def item(self):
        if self.spec.numel != 1:
            raise ValueError(f"item: tensor of shape {list(self.shape)} is not a single element")
        return self.raw.item()

    def values(self):
        return self.raw.detach().cpu().reshape(-1).tolist()

    def __repr__(self):
        return f"Tensor(shape={list(self.shape)}, dtype={self.dtype}, device={self.device.kind!r})"

    def _repr_html_(self):
        """Notebook display: dtype / shape / device / statistics and a heat map for small tensors."""
        from ..utils import widget
        return widget.render_html(widget.to_module_node(self, "tensor"))

    def describe(self) -> str:
        """One line with dtype, shape, device and value statistics."""
        from ..utils import widget
        return widget.render_text(widget.to_module_node(self, "tensor"))

    # -- operator sugar (delegates to the typed ops so every result is spec-checked) -----------------
    def __add__(self, o):
        from . import ops
        return ops.add(self, o) if isinstance(o, Tensor) else ops.add_scalar(self, o)

    def __sub__(self, o):
        from . import ops
        return ops.sub(self, o) if isinstance(o, Tensor) else ops.sub_scalar(self, o)

    def __mul__(self, o):
        from . import ops
        return ops.mul(self, o) if isinstance(o, Tensor) else ops.mul_scalar(self, o)

    def __truediv__(self, o):
        from . import ops
        return ops.div(self, o) if isinstance(o, Tensor) else ops.div_scalar(self, o)

    def __matmul__(self, o):
        from . import ops
        return ops.matmul(self, o)

    def __neg__(self):
        from . import ops
        return ops.neg(self)


def spec_of(raw: torch.Tensor) -> StaticSpec:
    return StaticSpec(tuple(raw.shape), DType.of_torch(raw.dtype), Device.of_torch(raw.device))


def _check(raw: torch.Tensor, spec: StaticSpec, op: str) -> None:
    if not isinstance(raw, torch.Tensor):
        raise SpecMismatch(f"{op}: expected a tensor, got {type(raw).__name__}")
    if tuple(raw.shape) != spec.shape:
        raise SpecMismatch(f"{op}: runtime shape {list(raw.shape)} does not match the claimed {list(spec.shape)}")
    if raw.dtype != spec.dtype.torch:
        raise SpecMismatch(f"{op}: runtime dtype {raw.dtype} does not match the claimed {spec.dtype}")
    dev = Device.of_torch(raw.device)
    if dev != spec.device:
        raise SpecMismatch(f"{op}: runtime device {raw.device} does not match the claimed {spec.device}")


def get_live_tensors() -> int:
    """Leak gauge: number of typed tensors currently alive (cc/src/tyr.cpp:135,373)."""
    return _live[0]


@dataclass
class SomeDTypeTensor:
    """A tensor of known shape and device whose dtype is chosen at run time."""
    shape: sh.Shape
    device: Device
    tensor: Tensor

    @property
    def dtype(self) -> DType:
        return self.tensor.dtype

    def at_dtype(self, dtype: DType) -> Optional[Tensor]:
        return self.tensor.at_dtype(dtype)


@dataclass
class ShapePackedTensor:
    """A tensor of known dtype and device whose shape is chosen at run time."""
    dtype: DType
    device: Device
    tensor: Tensor

    @property
    def shape(self) -> sh.Shape:
        return self.tensor.shape

    def at_shape(self, shape: Sequence[int]) -> Optional[Tensor]:
        return self.tensor if tuple(shape) == self.tensor.shape else None


def real_floating_dtype(t: Tensor) -> DType:
    """``RealFloatingDType`` evidence for a runtime tensor, or a TypeError."""
    if not t.dtype.is_real_floating:
        raise TypeError(f"Expected a standard real floating dtype, got {t.dtype}")
    return t.dtype
