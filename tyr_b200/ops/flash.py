"""Bindings for the tcgen05 flash-attention kernels (csrc/attention_fwd.cu, attention_bwd.cu).

Tensors are addressed as ``[B, T, H, D]`` views through explicit (batch, row, head) element
strides, so the packed ``[rows, 3, H, D]`` projection of the training path and the usual
``[B, H, T, D]`` layout are both consumed without a copy.  Supported: bf16, head_dim 128,
causal (with offset for cached prefixes), sliding window, GQA, arbitrary sequence lengths.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from .._native import register_signatures
from ._common import check, cur_stream, err_word, lib, ptr

_ENABLED = os.environ.get("TYR_FLASH", "1") != "0"


@register_signatures
def _sigs(lib_):
    import ctypes
    P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    for name, args in (
        ("tyr_flash_fwd", [P, P, P, P, P, I, I, I, I, I, I] + [L] * 12 + [I, I, I, F, P, P]),
        ("tyr_flash_bwd", [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, ctypes.POINTER(L), I, I, I, F, P, P]),
    ):
        fn = getattr(lib_, name, None)
        if fn is not None:
            fn.argtypes = args
            fn.restype = ctypes.c_int
    fn = getattr(lib_, "tyr_flash_bwd_workspace_bytes", None)
    if fn is not None:
        fn.argtypes = [I, I, I]
        fn.restype = L


def has_fwd() -> bool:
    return _ENABLED and hasattr(lib(), "tyr_flash_fwd")


def has_bwd() -> bool:
    return _ENABLED and hasattr(lib(), "tyr_flash_bwd")


def _bthd_strides(x_bthd: torch.Tensor):
    """x is a [B, T, H, D] view; returns (batch, row, head) strides in elements."""
    assert x_bthd.stride(3) == 1
    return x_bthd.stride(0), x_bthd.stride(1), x_bthd.stride(2)


def _ok_view(x: torch.Tensor) -> bool:
    return (x.stride(3) == 1 and all(s % 8 == 0 for s in x.stride()[:3]) and x.data_ptr() % 16 == 0)


def flash_fwd_bthd(q, k, v, *, causal: bool, window: Optional[int], scale: Optional[float],
                   q_offset: Optional[int] = None, out: Optional[torch.Tensor] = None,
                   need_lse: bool = True):
    """q: [B, Tq, Hq, D]; k, v: [B, Tk, Hkv, D] (views).  Returns (o [B, Tq, Hq, D], lse [B, Hq, Tq])."""
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    if out is None:
        out = torch.empty((B, Tq, Hq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, Tq), dtype=torch.float32, device=q.device) if need_lse else None
    if q_offset is None:
        q_offset = Tk - Tq
    sc = scale if scale is not None else 1.0 / math.sqrt(D)
    check(lib().tyr_flash_fwd(ptr(q), ptr(k), ptr(v), ptr(out), ptr(lse), B, Hq, Hkv, Tq, Tk, D,
                              *_bthd_strides(q), *_bthd_strides(k), *_bthd_strides(v),
                              *_bthd_strides(out), 1 if causal else 0, int(window or 0), q_offset, sc,
                              ptr(err_word(q.device)), cur_stream(q.device)), "flash_fwd")
    return out, lse


def flash_bwd_bthd(do, q, k, v, o, lse, *, causal, window, scale, q_offset=None):
    """Gradients (dq, dk, dv) as [B, T, H, D] views, packed into one [B, T, 3, H, D] buffer (returned fourth) when
    Hq == Hkv and Tq == Tk, else three separate buffers.  Every operand is a strided [B, T, H, D] view."""
    import ctypes
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    if q_offset is None:
        q_offset = Tk - Tq
    sc = scale if scale is not None else 1.0 / math.sqrt(D)
    if Hq == Hkv and Tq == Tk:
        buf = torch.empty((B, Tq, 3, Hq, D), dtype=q.dtype, device=q.device)
        dq, dk, dv = buf[:, :, 0], buf[:, :, 1], buf[:, :, 2]
    else:
        buf = None
        dq = torch.empty((B, Tq, Hq, D), dtype=q.dtype, device=q.device)
        dk = torch.empty((B, Tk, Hkv, D), dtype=q.dtype, device=q.device)
        dv = torch.empty((B, Tk, Hkv, D), dtype=q.dtype, device=q.device)
    ws = torch.empty(int(lib().tyr_flash_bwd_workspace_bytes(B, Hq, Tq)), dtype=torch.uint8, device=q.device)
    strides = (ctypes.c_longlong * 24)(*[x for t in (q, k, v, o, do, dq, dk, dv) for x in _bthd_strides(t)])
    check(lib().tyr_flash_bwd(ptr(do), ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), ptr(dq), ptr(dk), ptr(dv), ptr(ws),
                              B, Hq, Hkv, Tq, Tk, D, strides, 1 if causal else 0, int(window or 0), q_offset, sc,
                              ptr(err_word(q.device)), cur_stream(q.device)), "flash_bwd")
    return dq, dk, dv, buf


def supported(q, k, v, causal, window) -> bool:
    """[B, H, T, D] inputs (forward only: used by the inference paths)."""
    if not has_fwd() or torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        return False
    if q.shape[-1] != 128 or q.dtype != torch.bfloat16 or q.shape[1] % k.shape[1] != 0:
        return False
    return all(_ok_view(t.transpose(1, 2)) for t in (q, k, v))


def flash_attention(q, k, v, *, causal=True, window=None, scale=None):
    """[B, H, T, D] in, [B, H, T, D] out (a transposed view of a [B, T, H, D] buffer)."""
    o, _ = flash_fwd_bthd(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal=causal,
                          window=window, scale=scale, need_lse=False)
    return o.transpose(1, 2)


_TRAIN = os.environ.get("TYR_FLASH_TRAIN", "1") != "0"


def supported_packed(H, D, T, causal, window) -> bool:
    """Training path (forward + backward through these kernels, reading q / k / v from the packed projection and writing
    the three gradients into one packed buffer).  ``TYR_FLASH_TRAIN=0`` falls back to the library's fused attention."""
    return _TRAIN and has_fwd() and has_bwd() and D == 128


class _FlashPackedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, B, T, H, D, causal, window, scale):
        x = qkv.view(B, T, 3, H, D)
        q, k, v = x[:, :, 0], x[:, :, 1], x[:, :, 2]
        o, lse = flash_fwd_bthd(q, k, v, causal=causal, window=window, scale=scale)
        ctx.save_for_backward(qkv, o, lse)
        ctx.cfg = (B, T, H, D, causal, window, scale)
        return o.view(B * T, H * D)

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse = ctx.saved_tensors
        B, T, H, D, causal, window, scale = ctx.cfg
        x = qkv.view(B, T, 3, H, D)
        q, k, v = x[:, :, 0], x[:, :, 1], x[:, :, 2]
        do = do.contiguous().view(B, T, H, D)
        _, _, _, buf = flash_bwd_bthd(do, q, k, v, o, lse, causal=causal, window=window, scale=scale)
        return buf.view(B * T, 3 * H * D), None, None, None, None, None, None, None


def flash_attention_packed(qkv, B, T, H, D, *, causal=True, window=None, scale=None):
    return _FlashPackedFn.apply(qkv, B, T, H, D, causal, window, scale)
