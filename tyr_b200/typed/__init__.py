"""Typed facade: tensors whose shape, dtype and device are part of their spec and are checked on
every operation (the reference's ``Tensor sigma``, Tyr/Basic.lean and Tyr/Typed/*)."""
from .dtype import DType, promote, promote_scalar  # noqa: F401
from .device import Device, DeviceKind, get_best_device  # noqa: F401
from .spec import StaticSpec, TensorSpec  # noqa: F401
from .tensor import Tensor, SomeDTypeTensor, ShapePackedTensor, SpecMismatch, get_live_tensors  # noqa: F401
from . import shape, ops, neural  # noqa: F401
