"""Rotary embedding kernels (csrc/rope.cu).

``rotary_freqs(seq, head_dim, base)`` reproduces cc/src/tyr.cpp:2776-2802 (cos/sin of shape
``[seq, head_dim/2]``); ``apply_rotary`` is the half-split rotation of cc/src/tyr.cpp:2823-2856.
``qkv_post`` is the fused NanoChat attention prologue: RoPE, then per-head RMSNorm of q and k,
and the value-embedding blend ``v = (1-m) v + m ve`` (Examples/NanoChat/ModdedGPT.lean:301-327).
"""
from __future__ import annotations

from typing import Optional

import torch

from ._common import check, cur_stream, lib, ptr
from .norm import EPS, rms_norm_ref


def rotary_freqs(seq_len: int, head_dim: int, base: float = 10000.0, device="cpu"):
    ch = torch.arange(0, head_dim, 2, dtype=torch.float32, device=device)
    inv = 1.0 / torch.pow(torch.tensor(base, dtype=torch.float32, device=device), ch / head_dim)
    t = torch.arange(seq_len, dtype=torch.float32, device=device)
    fr = torch.outer(t, inv)
    return fr.cos(), fr.sin()


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [batch, seq, heads, head_dim]; cos/sin: [seq, head_dim/2]."""
    d = x.shape[3] // 2
    x1, x2 = x[..., :d].float(), x[..., d:2 * d].float()
    c = cos[None, :, None, :].to(x.device)
    s = sin[None, :, None, :].to(x.device)
    return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=3).to(x.dtype)


def qkv_post_ref(qkv, ve, mix, cos, sin, T, H, D, eps=EPS):
    rows = qkv.shape[0]
    x = qkv.float().reshape(rows // T, T, 3, H, D)
    q = rms_norm_ref(apply_rotary(x[:, :, 0], cos, sin), eps)
    k = rms_norm_ref(apply_rotary(x[:, :, 1], cos, sin), eps)
    v = x[:, :, 2]
    if ve is not None:
        m = mix.float().reshape(())
        v = (1.0 - m) * v + m * ve.float().reshape(rows // T, T, H, D)
    return torch.stack([q, k, v], dim=2).reshape(rows, 3 * H * D).to(qkv.dtype)


class _QkvPostFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, ve, mix, cos, sin, T, H, D, eps):
        qkv = qkv.contiguous()
        rows = qkv.shape[0]
        if qkv.is_cuda:
            out = torch.empty_like(qkv)
            vec = ve.contiguous() if ve is not None else None
            check(lib().tyr_qkv_post_fwd(ptr(qkv), ptr(vec), ptr(mix), ptr(cos), ptr(sin), ptr(out),
                                         rows, T, H, D, eps, cur_stream(qkv.device)), "qkv_post_fwd")
        else:
            vec = ve
            out = qkv_post_ref(qkv, ve, mix, cos, sin, T, H, D, eps)
        ctx.save_for_backward(qkv, vec, mix, cos, sin)
        ctx.dims = (T, H, D, eps)
        return out

    @staticmethod
    def backward(ctx, dy):
        qkv, ve, mix, cos, sin = ctx.saved_tensors
        T, H, D, eps = ctx.dims
        rows = qkv.shape[0]
        if qkv.is_cuda:
            dy = dy.contiguous()
            dqkv = torch.empty_like(qkv)
            dve = torch.empty_like(ve) if ve is not None else None
            dmix = torch.zeros((), dtype=torch.float32, device=qkv.device) if ve is not None else None
            check(lib().tyr_qkv_post_bwd(ptr(qkv), ptr(ve), ptr(mix), ptr(cos), ptr(sin), ptr(dy),
                                         ptr(dqkv), ptr(dve), ptr(dmix), rows, T, H, D, eps,
                                         cur_stream(qkv.device)), "qkv_post_bwd")
            if dmix is not None and mix is not None:
                dmix = dmix.reshape(mix.shape)
            return dqkv, dve, dmix, None, None, None, None, None, None
        with torch.enable_grad():
            q_ = qkv.detach().float().requires_grad_(True)
            ve_ = ve.detach().float().requires_grad_(True) if ve is not None else None
            mix_ = mix.detach().float().requires_grad_(True) if mix is not None else None
            out = qkv_post_ref(q_, ve_, mix_, cos, sin, T, H, D, eps)
            ins = [t for t in (q_, ve_, mix_) if t is not None]
            gs = list(torch.autograd.grad(out, ins, dy.float(), allow_unused=True))
        dq = gs.pop(0).to(qkv.dtype)
        dve = gs.pop(0).to(ve.dtype) if ve is not None else None
        dmix = gs.pop(0) if (mix is not None and gs) else None
        return dq, dve, dmix, None, None, None, None, None, None


def qkv_post(qkv: torch.Tensor, ve: Optional[torch.Tensor], mix: Optional[torch.Tensor],
             cos: torch.Tensor, sin: torch.Tensor, T: int, H: int, D: int, eps: float = EPS):
    """qkv: [rows, 3*H*D] (rows = batch*T); ve: [rows, H*D] or None; mix: fp32 scalar tensor."""
    if mix is not None:
        mix = mix.float()
    return _QkvPostFn.apply(qkv, ve, mix, cos, sin, T, H, D, eps)


def rope_norm(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, *, weight=None,
              positions: Optional[torch.Tensor] = None, rot: Optional[int] = None,
              eps: float = EPS, one_plus_w: bool = False) -> torch.Tensor:
    """x: [rows, H, D] (bf16 on CUDA).  Optional per-head RMSNorm(weight) BEFORE the rotation of
    the first ``rot`` channels; cos/sin: [P, rot/2]; positions: int32 [rows]."""
    rows, H, D = x.shape
    rot = D if rot is None else rot
    if x.is_cuda and x.dtype == torch.bfloat16:
        xc = x if x.stride(2) == 1 and x.stride(1) == D else x.contiguous()      # rows may be slices of a wider projection
        y = torch.empty((rows, H, D), dtype=x.dtype, device=x.device)
        pos = positions.to(torch.int32).contiguous() if positions is not None else None
        w = weight.to(torch.bfloat16).contiguous() if weight is not None else None
        T = cos.shape[0]
        check(lib().tyr_rope_norm(ptr(xc), ptr(y), ptr(w), ptr(cos.float().contiguous()),
                                  ptr(sin.float().contiguous()), ptr(pos), xc.stride(0), H * D, rows, T, H, D, rot,
                                  eps, 1 if one_plus_w else 0, cur_stream(x.device)), "rope_norm")
        return y
    xf = x.float()
    if weight is not None:
        w = weight.float() + (1.0 if one_plus_w else 0.0)
        xf = (rms_norm_ref(xf, eps).to(x.dtype).float() * w).to(x.dtype).float()
    pos = positions.long() if positions is not None else torch.arange(rows, device=x.device) % cos.shape[0]
    c = cos.float()[pos][:, None, :]
    s = sin.float()[pos][:, None, :]
    hr = rot // 2
    x1, x2 = xf[..., :hr], xf[..., hr:rot]
    out = torch.cat([x1 * c - x2 * s, x1 * s + x2 * c, xf[..., rot:]], dim=-1)
    return out.to(x.dtype)
