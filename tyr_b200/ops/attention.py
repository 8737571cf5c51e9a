"""Attention front-ends.

``attention_packed`` consumes the packed ``[rows, 3, H, D]`` projection produced by
``qkv_post`` and returns ``[rows, H*D]``.  On CUDA with bf16 inputs it runs the hand-written
tcgen05 flash-attention kernels (csrc/attention_fwd.cu / attention_bwd.cu) when they are built;
the bounded math path below is the CPU oracle and mirrors the reference dispatcher
(cc/include/tyr_attention.h:58-130): causal, sliding window (a query at position i sees keys
in (i - window, i]), GQA by head grouping, explicit key-padding / edge masks.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


def _mask(Tq: int, Tk: int, causal: bool, window: Optional[int], device, q_offset: int = 0):
    if not causal and window is None:
        return None
    qi = torch.arange(Tq, device=device)[:, None] + q_offset
    ki = torch.arange(Tk, device=device)[None, :]
    m = torch.ones(Tq, Tk, dtype=torch.bool, device=device)
    if causal:
        m &= ki <= qi
    if window is not None:
        m &= ki > qi - window
    return m


def attention_ref(q, k, v, *, causal=True, window: Optional[int] = None,
                  scale: Optional[float] = None, key_padding_mask=None, edge_mask=None,
                  q_offset: Optional[int] = None):
    """q: [B, Hq, Tq, D]; k, v: [B, Hkv, Tk, D]; fp32 math; GQA when Hq is a multiple of Hkv."""
    B, Hq, Tq, D = q.shape
    Hkv, Tk = k.shape[1], k.shape[2]
    if Hq % Hkv != 0:
        raise ValueError(f"attention: {Hq} query heads are not a multiple of {Hkv} kv heads")
    rep = Hq // Hkv
    kf = k.float().repeat_interleave(rep, dim=1)
    vf = v.float().repeat_interleave(rep, dim=1)
    s = torch.matmul(q.float(), kf.transpose(-1, -2)) * (scale if scale is not None else 1.0 / math.sqrt(D))
    if q_offset is None:
        q_offset = Tk - Tq
    m = _mask(Tq, Tk, causal, window, q.device, q_offset)
    if m is not None:
        s = s.masked_fill(~m, float("-inf"))
    if key_padding_mask is not None:  # [B, Tk] True = keep
        s = s.masked_fill(~key_padding_mask[:, None, None, :].bool(), float("-inf"))
    if edge_mask is not None:  # [B, Tq, Tk] True = keep
        s = s.masked_fill(~edge_mask[:, None].bool(), float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    return torch.matmul(p, vf).to(q.dtype)


def attention(q, k, v, *, causal=True, window: Optional[int] = None, scale: Optional[float] = None,
              key_padding_mask=None, edge_mask=None):
    """General attention entry ([B, H, T, D] layout)."""
    from . import flash
    if (q.is_cuda and q.dtype == torch.bfloat16 and key_padding_mask is None and edge_mask is None
            and flash.supported(q, k, v, causal, window)):
        return flash.flash_attention(q, k, v, causal=causal, window=window, scale=scale)
    if q.is_cuda and key_padding_mask is None and edge_mask is None and window is None:
        Hq, Hkv = q.shape[1], k.shape[1]
        is_causal = causal and q.shape[2] == k.shape[2]
        if causal and not is_causal:
            return attention_ref(q, k, v, causal=True, scale=scale)
        return F.scaled_dot_product_attention(q, k, v, is_causal=is_causal, scale=scale,
                                              enable_gqa=(Hq != Hkv))
    return attention_ref(q, k, v, causal=causal, window=window, scale=scale,
                         key_padding_mask=key_padding_mask, edge_mask=edge_mask)


class _SdpaPackedFn(torch.autograd.Function):
    """Library attention on the packed projection without autograd's per-slice zero-fill: the
    inner graph is kept and differentiated once, and the three gradients are written straight
    into one packed buffer."""

    @staticmethod
    def forward(ctx, qkv, B, T, H, D, causal, scale):
        x = qkv.detach().view(B, T, 3, H, D)
        with torch.enable_grad():
            q = x[:, :, 0].transpose(1, 2).requires_grad_(True)
            k = x[:, :, 1].transpose(1, 2).requires_grad_(True)
            v = x[:, :, 2].transpose(1, 2).requires_grad_(True)
            o = F.scaled_dot_product_attention(q, k, v, is_causal=causal, scale=scale)
        ctx.inner = (q, k, v, o)
        ctx.dims = (B, T, H, D)
        return o.detach().transpose(1, 2).reshape(B * T, H * D)

    @staticmethod
    def backward(ctx, do):
        q, k, v, o = ctx.inner
        B, T, H, D = ctx.dims
        do4 = do.view(B, T, H, D).transpose(1, 2)
        dq, dk, dv = torch.autograd.grad(o, (q, k, v), do4)
        out = torch.empty((B, T, 3, H, D), dtype=do.dtype, device=do.device)
        out[:, :, 0].copy_(dq.transpose(1, 2))
        out[:, :, 1].copy_(dk.transpose(1, 2))
        out[:, :, 2].copy_(dv.transpose(1, 2))
        ctx.inner = None
        return out.view(B * T, 3 * H * D), None, None, None, None, None, None


def attention_packed(qkv: torch.Tensor, B: int, T: int, H: int, D: int, *, causal: bool = True,
                     window: Optional[int] = None, scale: Optional[float] = None) -> torch.Tensor:
    """qkv: [B*T, 3*H*D] packed (q | k | v, heads inner) -> [B*T, H*D]."""
    from . import flash
    if qkv.is_cuda and qkv.dtype == torch.bfloat16 and flash.supported_packed(H, D, T, causal, window):
        return flash.flash_attention_packed(qkv, B, T, H, D, causal=causal, window=window, scale=scale)
    if qkv.is_cuda and window is None:
        return _SdpaPackedFn.apply(qkv, B, T, H, D, causal, scale)
    x = qkv.view(B, T, 3, H, D)
    q, k, v = (x[:, :, i].transpose(1, 2) for i in range(3))
    o = attention_ref(q, k, v, causal=causal, window=window, scale=scale)
    return o.transpose(1, 2).reshape(B * T, H * D)
