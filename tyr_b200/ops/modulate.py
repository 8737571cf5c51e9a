"""Adaptive LayerNorm modulation and gated residual (csrc/modulate.cu), with fp32 PyTorch fallbacks."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from .._native import register_signatures
from ._common import check, cur_stream, lib, ptr


@register_signatures
def _sigs(lib_):
    import ctypes
    P, I, L, Fl = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    for name, args in (("tyr_layernorm_modulate", [P, P, P, P, L, I, I, L, Fl, P]),
                       ("tyr_gate_residual", [P, P, P, P, L, I, I, L, P])):
        fn = getattr(lib_, name, None)
        if fn is not None:
            fn.argtypes = args
            fn.restype = ctypes.c_int


def _mod_ok(x, *mods):
    D = x.shape[-1]
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 3 and D % 8 == 0 and x.is_contiguous()):
        return False
    strides = set()
    for m in mods:
        if m is None:
            continue
        if m.dtype != torch.bfloat16 or m.stride(-1) != 1 or m.data_ptr() % 16 or m.shape != (x.shape[0], D):
            return False
        strides.add(m.stride(0) if x.shape[0] > 1 else 0)
    return len(strides) <= 1 and all(s % 8 == 0 for s in strides)


def layernorm_modulate(x: torch.Tensor, scale: Optional[torch.Tensor], shift: Optional[torch.Tensor], eps: float = 1e-6) -> torch.Tensor:
    """x: [B, S, D]; scale, shift: [B, D] (views of a modulation tensor are fine).  ``(1 + scale) * LN(x) + shift``."""
    if _mod_ok(x, scale, shift):
        B, S, D = x.shape
        y = torch.empty_like(x)
        ref = scale if scale is not None else shift
        bstride = ref.stride(0) if (ref is not None and B > 1) else 0
        check(lib().tyr_layernorm_modulate(ptr(x), ptr(scale), ptr(shift), ptr(y), B * S, S, D, bstride, eps,
                                           cur_stream(x.device)), "layernorm_modulate")
        return y
    y = F.layer_norm(x.float(), (x.shape[-1],), eps=eps)
    if scale is not None:
        y = y * (1.0 + scale.float().unsqueeze(1))
    if shift is not None:
        y = y + shift.float().unsqueeze(1)
    return y.to(x.dtype)


def gate_residual(x: torch.Tensor, y: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """``x + gate[:, None, :] * y``."""
    if _mod_ok(x, gate) and y.is_contiguous() and y.dtype == x.dtype and y.shape == x.shape:
        B, S, D = x.shape
        out = torch.empty_like(x)
        check(lib().tyr_gate_residual(ptr(x), ptr(y), ptr(gate), ptr(out), B * S, S, D, gate.stride(0) if B > 1 else 0,
                                      cur_stream(x.device)), "gate_residual")
        return out
    return (x.float() + gate.float().unsqueeze(1) * y.float()).to(x.dtype)
