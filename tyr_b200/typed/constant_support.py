"""Evidence that the constant factories can build exact 0 / 1 / identity values at a (dtype, device) pair
(Tyr/ConstantSupport.lean, Tyr/ConstantSupport/Types.lean; native probe cc/src/tyr.cpp:3159-3184).

The reference keeps this apart from dtype recognition and promotion: knowing a dtype's name says nothing about
whether ``zeros`` / ``ones`` / ``eye`` and the conversion from Float32 work for it on a given device.  A small static
table covers the combinations that always work; everything else is *acquired* at run time by building 2 x 2 zero, one
and identity tensors through the same paths the factories use and comparing them, on the host in Float32, with exact
references.  Quantised-without-parameters and shell formats fail here instead of deep inside a model.

The witness is deliberately opaque (``ConstantSupported`` cannot be constructed by user code) and carries no claim
about any other kernel.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from .device import Device
from .dtype import DType

_ALWAYS = frozenset({DType.UInt8, DType.Int8, DType.Int16, DType.Int32, DType.Int64, DType.Float16, DType.Float32,
                     DType.Bool})
_CPU_ONLY = frozenset({DType.BFloat16, DType.Float64, DType.Complex32, DType.Complex64, DType.Complex128,
                       DType.Float8E4M3FN, DType.Float8E5M2, DType.Float8E5M2FNUZ, DType.Float8E4M3FNUZ,
                       DType.UInt16, DType.UInt32, DType.UInt64})

_TOKEN = object()


def static_constant_support(dtype: DType, device: Device) -> bool:
    """Conservative built-in table: accelerator-dependent formats need run-time acquisition."""
    if dtype in _ALWAYS:
        return True
    if dtype in _CPU_ONLY:
        return device.is_cpu
    return False


class ConstantSupported:
    """Witness for one exact (dtype, device).  Obtain it from :func:`acquire_constant_support`."""
    __slots__ = ("dtype", "device", "static")

    def __init__(self, dtype: DType, device: Device, static: bool, _token=None):
        if _token is not _TOKEN:
            raise TypeError("ConstantSupported is acquired with acquire_constant_support(dtype, device)")
        object.__setattr__(self, "dtype", dtype)
        object.__setattr__(self, "device", device)
        object.__setattr__(self, "static", static)

    def __setattr__(self, *_):
        raise AttributeError("ConstantSupported is immutable")

    def __repr__(self):
        return f"ConstantSupported({self.dtype.name}, {self.device!r}, {'static' if self.static else 'runtime'})"


_CACHE: Dict[Tuple[DType, Device], ConstantSupported] = {}


def _probe(dtype: DType, device: Device) -> None:
    try:
        td = dtype.torch
    except TypeError as e:
        raise IOError(f"DType.acquireConstantSupport: {e}") from None
    place = device.torch
    zeros = torch.zeros(2, 2, dtype=torch.float32)
    ones = torch.ones(2, 2, dtype=torch.float32)
    ident = torch.eye(2, dtype=torch.float32)

    def check(expected, actual):
        if actual.dtype != td or actual.device.type != place.type:
            raise IOError("DType.acquireConstantSupport: constant conversion returned incorrect dtype or placement")
        if not torch.equal(expected, actual.to("cpu").to(torch.float32)):
            raise IOError(f"DType.acquireConstantSupport: dtype cannot represent exact zero and one constants: {dtype.name}")

    try:
        # the factory paths themselves, not just "this dtype exists"
        check(zeros, torch.zeros(2, 2, dtype=torch.float32, device=place).to(td))
        check(ones, torch.ones(2, 2, dtype=torch.float32, device=place).to(td))
        check(ident, ident.to(td).to(place))
    except IOError:
        raise
    except Exception as e:      # missing kernels, quantised dtypes without parameters, ...
        raise IOError(f"DType.acquireConstantSupport: {dtype.name} on {device!r}: {e}") from None


def acquire_constant_support(dtype: DType, device: Device) -> ConstantSupported:
    """Static table first; otherwise allocate the small probes on ``device`` and verify exact values.  Raises ``IOError``
    when the pair is not usable.  Witnesses are cached per (dtype, device)."""
    key = (dtype, device)
    hit = _CACHE.get(key)
    if hit is not None:
        return hit
    if static_constant_support(dtype, device):
        w = ConstantSupported(dtype, device, True, _TOKEN)
    else:
        _probe(dtype, device)
        w = ConstantSupported(dtype, device, False, _TOKEN)
    _CACHE[key] = w
    return w


def require(support: ConstantSupported, dtype: DType, device: Device) -> None:
    """Guard used by factories that take a witness: it must be for exactly this dtype and device."""
    if not isinstance(support, ConstantSupported) or support.dtype is not dtype or support.device != device:
        raise TypeError(f"constant factory for {dtype.name} on {device!r} given {support!r}")
