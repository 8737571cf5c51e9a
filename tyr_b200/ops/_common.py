"""Helpers shared by the op wrappers: raw pointers, current stream, return-code checks and the
device-side error record that bounded waits write into."""
from __future__ import annotations

import ctypes

import torch

from .._native import kernels

_err_words = {}
# Number of native kernel launches issued through the wrappers (each checked call = one launch).
LAUNCH_COUNT = [0]


def ptr(t):
    """Raw device/host pointer of a tensor (None -> NULL)."""
    if t is None:
        return None
    return ctypes.c_void_p(t.data_ptr())


def cur_stream(device=None):
    """Current torch stream of ``device`` as a raw handle.  Also binds that device to the calling
    host thread inside the kernel library (autograd worker threads start without one)."""
    idx = torch.device(device).index if device is not None else None
    if idx is None:
        idx = torch.cuda.current_device()
    rc = kernels().tyr_bind_device(idx)
    if rc != 0:
        raise RuntimeError(f"tyr_bind_device({idx}) failed with CUDA error {rc}")
    return ctypes.c_void_p(torch.cuda.current_stream(idx).cuda_stream)


def check(rc: int, what: str):
    LAUNCH_COUNT[0] += 1
    if rc != 0:
        raise RuntimeError(f"tyr_b200 native call {what} failed with code {rc}")


def err_word(device) -> torch.Tensor:
    """Per-device int32[4] record {code, block, detail, spare} written by kernels on a timeout."""
    idx = torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    w = _err_words.get(idx)
    if w is None:
        w = torch.zeros(4, dtype=torch.int32, device=f"cuda:{idx}")
        _err_words[idx] = w
    return w


def raise_on_device_error(device=None):
    """Synchronises, reads the error record and raises if a kernel reported a bounded-wait
    timeout or a bounds violation.  Call between steps (it is a host sync)."""
    if device is None:
        device = torch.cuda.current_device()
    w = err_word(device)
    vals = w.tolist()
    if vals[0] != 0:
        w.zero_()
        raise RuntimeError(
            f"device error record: code={vals[0]} block={vals[1]} detail={vals[2]} "
            "(1=mbarrier timeout, 2=peer flag timeout, 3=bounds, 4=tmem)")


def is_cuda(*ts) -> bool:
    return any(t is not None and t.is_cuda for t in ts)


def lib():
    return kernels()
