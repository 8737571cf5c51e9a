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
                       ("tyr_gate_residual", [P, P, P, P, L, I, I, L, P]),
                       ("tyr_flux_qk_post", [P, L, L, P, L, L, P, P, P, P, L, I, I, I, I, I, I, Fl, P])):
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


def flux_qk_post_supported(src: torch.Tensor, head_dim: int) -> bool:
    return (src.is_cuda and src.dtype == torch.bfloat16 and head_dim == 128 and src.dim() == 3 and src.stride(-1) == 1
            and getattr(lib(), "tyr_flux_qk_post", None) is not None)


def flux_qk_post(src: torch.Tensor, dst: torch.Tensor, wq: torch.Tensor, wk: torch.Tensor, cos: torch.Tensor,
                 sin: torch.Tensor, num_heads: int, *, dst_row0: int = 0, copy_v: bool = False, eps: float = 1e-6) -> None:
    """Per-head ``RoPE(RMSNorm(q) * wq)`` and the same for k, from the fused projection ``src`` ([B, S, >= 3*H*128] rows:
    q | k | v) into ``dst`` (same column layout, rows ``dst_row0 ...``); ``copy_v`` also moves v.  ``dst`` may be ``src``
    (in place, v untouched).  cos / sin: fp32 [B or 1, S, 64].  Reference: Tyr/Model/Flux/Layers.lean (QKNorm + RoPE)."""
    B, S, _ = src.shape
    H = num_heads
    assert dst.dim() == 3 and dst.stride(-1) == 1 and dst.shape[0] == B and dst.shape[1] >= dst_row0 + S
    assert cos.dtype == torch.float32 and cos.shape[-2:] == (S, 64) and cos.is_contiguous() and sin.is_contiguous()
    cs_sb = cos.stride(0) if (cos.dim() == 3 and cos.shape[0] > 1) else 0
    wq = wq.to(torch.bfloat16).contiguous()
    wk = wk.to(torch.bfloat16).contiguous()
    check(lib().tyr_flux_qk_post(ptr(src), src.stride(0), src.stride(1), ptr(dst), dst.stride(0), dst.stride(1), ptr(wq),
                                 ptr(wk), ptr(cos), ptr(sin), cs_sb, B, S, H, 128, dst_row0, 1 if copy_v else 0, eps,
                                 cur_stream(src.device)), "flux_qk_post")
