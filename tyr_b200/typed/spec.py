"""Tensor specs: ``TensorSpec`` (shape + dtype) and ``StaticSpec`` (shape + dtype + device) with
the result-spec algebra of common operations (Tyr/Typed/Spec.lean, Tyr/Typed/Tensor.lean:42-55,
Tyr/Basic/Types.lean:269-273)."""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional

from . import shape as sh
from .device import Device, pointwise_result
from .dtype import DType, promote, promote_scalar


@dataclass(frozen=True)
class TensorSpec:
    shape: sh.Shape
    dtype: DType

    @staticmethod
    def scalar(dtype: DType) -> "TensorSpec":
        return TensorSpec((), dtype)

    @property
    def rank(self) -> int:
        return len(self.shape)

    @property
    def numel(self) -> int:
        return sh.numel(self.shape)

    def with_shape(self, shape) -> "TensorSpec":
        return replace(self, shape=tuple(shape))

    def with_dtype(self, dtype: DType) -> "TensorSpec":
        return replace(self, dtype=dtype)


def pointwise_dtype_opt(lhs: TensorSpec, rhs: TensorSpec) -> Optional[DType]:
    """Zero-dimensional operands promote weakly (Tyr/Typed/Spec.lean:118-122)."""
    if lhs.rank == 0 and rhs.rank > 0:
        return promote_scalar(rhs.dtype, lhs.dtype)
    if lhs.rank > 0 and rhs.rank == 0:
        return promote_scalar(lhs.dtype, rhs.dtype)
    return promote(lhs.dtype, rhs.dtype)


def pointwise_opt(lhs: TensorSpec, rhs: TensorSpec) -> Optional[TensorSpec]:
    s = sh.broadcast_shapes_opt(lhs.shape, rhs.shape)
    d = pointwise_dtype_opt(lhs, rhs)
    if s is None or d is None:
        return None
    return TensorSpec(s, d)


def division_opt(lhs: TensorSpec, rhs: TensorSpec) -> Optional[TensorSpec]:
    r = pointwise_opt(lhs, rhs)
    return None if r is None else TensorSpec(r.shape, r.dtype.divide_result)


def matmul_opt(lhs: TensorSpec, rhs: TensorSpec) -> Optional[TensorSpec]:
    s = sh.matmul_shape_opt(lhs.shape, rhs.shape)
    if s is None or lhs.dtype is not rhs.dtype:
        return None
    return TensorSpec(s, lhs.dtype)


def sum_spec(spec: TensorSpec) -> TensorSpec:
    return TensorSpec((), spec.dtype.sum_result)


def mean_spec(spec: TensorSpec) -> TensorSpec:
    return TensorSpec((), spec.dtype.mean_result)


def prod_spec(spec: TensorSpec) -> TensorSpec:
    return TensorSpec((), spec.dtype.prod_result)


def check_shape(expected, actual) -> None:
    if tuple(expected) != tuple(actual):
        raise ValueError(f"Expected shape {list(expected)}, got {list(actual)}")


def check_compatible(expected: TensorSpec, actual: TensorSpec) -> None:
    check_shape(expected.shape, actual.shape)
    if expected.dtype is not actual.dtype:
        raise TypeError(f"Expected dtype {expected.dtype}, got {actual.dtype}")


@dataclass(frozen=True)
class StaticSpec:
    """Exact shape, dtype and actual placement of a tensor; every field is required."""
    shape: sh.Shape
    dtype: DType
    device: Device = Device.CPU

    def __post_init__(self):
        object.__setattr__(self, "shape", tuple(int(d) for d in self.shape))

    @property
    def tensor_spec(self) -> TensorSpec:
        return TensorSpec(self.shape, self.dtype)

    @property
    def rank(self) -> int:
        return len(self.shape)

    @property
    def numel(self) -> int:
        return sh.numel(self.shape)

    def with_shape(self, shape) -> "StaticSpec":
        return replace(self, shape=tuple(shape))

    def with_dtype(self, dtype: DType) -> "StaticSpec":
        return replace(self, dtype=dtype)

    def with_device(self, device: Device) -> "StaticSpec":
        return replace(self, device=device)

    @property
    def sum_spec(self) -> "StaticSpec":
        return StaticSpec((), self.dtype.sum_result, self.device)

    def pointwise(self, other: "StaticSpec") -> Optional["StaticSpec"]:
        ts = pointwise_opt(self.tensor_spec, other.tensor_spec)
        dev = pointwise_result(self.device, self.rank, other.device, other.rank)
        if ts is None or dev is None:
            return None
        return StaticSpec(ts.shape, ts.dtype, dev)

    def division(self, other: "StaticSpec") -> Optional["StaticSpec"]:
        r = self.pointwise(other)
        return None if r is None else r.with_dtype(r.dtype.divide_result)
