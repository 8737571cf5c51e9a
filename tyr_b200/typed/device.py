"""Devices and the device-compatibility rules of typed ops.

``Device.CPU`` always exists; an accelerator ``Device`` can only be obtained through the runtime
acquisition ``Device.cuda(i)``, which checks availability and the ordinal and performs a probe
allocation (Tyr/Basic/Types.lean:208-251, cc/src/tyr.cpp:3187-3203).  The result rules mirror
Tyr/Typed/Device.lean:20-110: operands of matmul/cat must share a device, pointwise ops accept
a rank-0 CPU tensor next to an accelerator tensor, selections follow the selected operands.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

_ACQUIRE_TOKEN = object()


@dataclass(frozen=True)
class DeviceKind:
    """A placement description; it grants no access to a runtime device."""
    kind: str            # "cpu" | "cuda" | "mps"
    index: int = 0

    @staticmethod
    def CUDA(i: int) -> "DeviceKind":
        return DeviceKind("cuda", int(i))

    CPU: "DeviceKind" = None  # filled in below
    MPS: "DeviceKind" = None

    def __repr__(self):
        return f"DeviceKind.CUDA({self.index})" if self.kind == "cuda" else f"DeviceKind.{self.kind.upper()}"


DeviceKind.CPU = DeviceKind("cpu")
DeviceKind.MPS = DeviceKind("mps")


class Device:
    """An acquired runtime placement."""
    __slots__ = ("kind",)
    CPU: "Device" = None

    def __init__(self, kind: DeviceKind, _token=None):
        if kind.kind != "cpu" and _token is not _ACQUIRE_TOKEN:
            raise PermissionError("accelerator devices are acquired with Device.cuda(i) / Device.mps()")
        object.__setattr__(self, "kind", kind)

    def __setattr__(self, *a):
        raise AttributeError("Device is immutable")

    @staticmethod
    def cuda(index: int = 0) -> "Device":
        if not torch.cuda.is_available():
            raise RuntimeError("CUDA is not available")
        if not 0 <= index < torch.cuda.device_count():
            raise RuntimeError(f"CUDA device ordinal {index} out of range (have {torch.cuda.device_count()})")
        torch.empty(0, device=f"cuda:{index}")  # probe allocation
        return Device(DeviceKind.CUDA(index), _ACQUIRE_TOKEN)

    @staticmethod
    def mps() -> "Device":
        raise RuntimeError("MPS is not available on this platform")

    @staticmethod
    def of_torch(d: torch.device) -> "Device":
        d = torch.device(d)
        if d.type == "cpu":
            return Device.CPU
        if d.type == "cuda":
            return Device(DeviceKind.CUDA(d.index if d.index is not None else torch.cuda.current_device()),
                          _ACQUIRE_TOKEN)
        raise RuntimeError(f"unsupported device {d}")

    @property
    def torch(self) -> torch.device:
        k = self.kind
        return torch.device("cpu") if k.kind == "cpu" else torch.device(k.kind, k.index)

    @property
    def is_cpu(self) -> bool:
        return self.kind.kind == "cpu"

    @property
    def is_cuda(self) -> bool:
        return self.kind.kind == "cuda"

    def __eq__(self, other):
        return isinstance(other, Device) and self.kind == other.kind

    def __hash__(self):
        return hash(self.kind)

    def __repr__(self):
        return f"Device({self.kind!r})"


Device.CPU = Device(DeviceKind.CPU)


def get_best_device() -> Device:
    """``TYR_DEVICE`` override, else CUDA 0 when present, else CPU (Tyr/Torch.lean:29)."""
    req = os.environ.get("TYR_DEVICE", "").lower()
    if req.startswith("cuda"):
        idx = int(req.split(":")[1]) if ":" in req else 0
        return Device.cuda(idx)
    if req == "cpu":
        return Device.CPU
    if torch.cuda.is_available():
        return Device.cuda(0)
    return Device.CPU


def same_result(devices: Sequence[Device]) -> Optional[Device]:
    """All operands on one device (matmul, cat, ...)."""
    if not devices:
        return None
    first = devices[0]
    return first if all(d == first for d in devices) else None


def pointwise_result(lhs: Device, lhs_rank: int, rhs: Device, rhs_rank: int) -> Optional[Device]:
    """A rank-0 CPU tensor may be combined with an accelerator tensor."""
    if lhs == rhs:
        return lhs
    if lhs.is_cpu and lhs_rank == 0:
        return rhs
    if rhs.is_cpu and rhs_rank == 0:
        return lhs
    return None


def selection_result(cond: Device, a: Device, a_rank: int, b: Device, b_rank: int) -> Optional[Device]:
    """``where``: the condition lives with the selected operands."""
    r = pointwise_result(a, a_rank, b, b_rank)
    if r is None:
        return None
    return r if cond == r else None
