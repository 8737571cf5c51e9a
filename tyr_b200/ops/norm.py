"""RMSNorm family on the hand-written kernels in csrc/norm.cu.

``lincomb_rmsnorm(tensors, scalars)`` returns ``(out, normed)`` where
``out = sum_i scalars[i] * tensors[i]`` and ``normed = rms_norm(out)`` (eps 1e-6, fp32
accumulate, no weight) - the residual-stream update of the modded-nanogpt block fused with the
pre-norm that follows (Examples/NanoChat/ModdedGPT.lean:586-611, Tyr/Typed/Neural.lean:38-43).
Gradients flow to every tensor and to the scalars (a 1-D fp32 tensor).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from ._common import check, cur_stream, lib, ptr

EPS = 1e-6


def rms_norm_ref(x: torch.Tensor, eps: float = EPS) -> torch.Tensor:
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)


def _fwd_native(ts, scal, want_out, want_normed, eps):
    t0 = ts[0]
    D = t0.shape[-1]
    rows = t0.numel() // D
    out = torch.empty_like(t0) if want_out else None
    normed = torch.empty_like(t0) if want_normed else None
    p = [ptr(t) for t in ts] + [None] * (4 - len(ts))
    check(lib().tyr_lincomb_rmsnorm_fwd(p[0], p[1], p[2], p[3], ptr(scal), len(ts), rows, D,
                                        ptr(out), ptr(normed), eps, cur_stream(t0.device)),
          "lincomb_rmsnorm_fwd")
    return out, normed


class _LincombNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, scal, eps, want_normed, *ts):
        ts = [t.contiguous() for t in ts]
        if ts[0].is_cuda:
            out, normed = _fwd_native(ts, scal, True, want_normed, eps)
        else:
            acc = sum((scal[i] if scal is not None else 1.0) * t.float() for i, t in enumerate(ts))
            out = acc.to(ts[0].dtype)
            normed = rms_norm_ref(out, eps).to(out.dtype) if want_normed else None
        ctx.save_for_backward(scal, out, *ts)
        ctx.eps = eps
        ctx.n = len(ts)
        if want_normed:
            return out, normed
        ctx.mark_non_differentiable()
        return out, None

    @staticmethod
    def backward(ctx, d_out, d_normed):
        scal, out, *ts = ctx.saved_tensors
        n = ctx.n
        need_scal = scal is not None and ctx.needs_input_grad[0]
        if out.is_cuda:
            dts = [torch.empty_like(t) if ctx.needs_input_grad[3 + i] else None for i, t in enumerate(ts)]
            dscal = torch.zeros(n, dtype=torch.float32, device=out.device) if need_scal else None
            P = ctypes.c_void_p
            tarr = (P * 4)(*[t.data_ptr() for t in ts] + [None] * (4 - n))
            darr = (P * 4)(*[(d.data_ptr() if d is not None else None) for d in dts] + [None] * (4 - n))
            d_out_c = d_out.contiguous() if d_out is not None else None
            d_normed_c = d_normed.contiguous() if d_normed is not None else None
            D = out.shape[-1]
            check(lib().tyr_lincomb_rmsnorm_bwd(tarr, darr, ptr(scal), ptr(dscal), ptr(out),
                                                ptr(d_out_c), ptr(d_normed_c), n, out.numel() // D, D,
                                                ctx.eps, cur_stream(out.device)), "lincomb_rmsnorm_bwd")
        else:
            g = d_out.float() if d_out is not None else torch.zeros_like(out, dtype=torch.float32)
            if d_normed is not None:
                o = out.float()
                D = o.shape[-1]
                rstd = torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + ctx.eps)
                dot = (o * d_normed.float()).sum(-1, keepdim=True)
                g = g + rstd * d_normed.float() - o * (rstd ** 3) * dot / D
            dts = [((scal[i] if scal is not None else 1.0) * g).to(t.dtype) if ctx.needs_input_grad[3 + i] else None
                   for i, t in enumerate(ts)]
            dscal = torch.stack([(g * t.float()).sum() for t in ts]) if need_scal else None
        return (dscal, None, None, *dts)


def lincomb_rmsnorm(tensors: Sequence[torch.Tensor], scalars: Optional[torch.Tensor] = None,
                    eps: float = EPS, want_normed: bool = True):
    """Returns ``(out, normed)``; ``scalars`` is an fp32 tensor with ``len(tensors)`` entries."""
    if not 1 <= len(tensors) <= 4:
        raise ValueError("lincomb_rmsnorm takes 1..4 tensors")
    if scalars is not None and scalars.dtype != torch.float32:
        scalars = scalars.float()
    return _LincombNormFn.apply(scalars, eps, want_normed, *tensors)


def rms_norm(x: torch.Tensor, eps: float = EPS) -> torch.Tensor:
    """Weight-free RMSNorm that keeps the input dtype (bf16 on the GPU path)."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        return lincomb_rmsnorm([x], None, eps)[1]
    return rms_norm_ref(x, eps).to(x.dtype)


def rms_norm_weighted(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float = EPS, *,
                      one_plus_w: bool = False, gate: Optional[torch.Tensor] = None,
                      residual: Optional[torch.Tensor] = None, return_residual: bool = False):
    """Inference RMSNorm: ``y = norm(x [+ residual]) * w`` (``1 + w`` when ``one_plus_w``),
    optionally multiplied by ``silu(gate)``.  cc/src/tyr.cpp:3766-3772 plus the Qwen3.5 variants."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        xc = x.contiguous()
        D = xc.shape[-1]
        y = torch.empty_like(xc)
        r = residual.contiguous() if residual is not None else None
        r_out = torch.empty_like(xc) if (residual is not None and return_residual) else None
        w = weight.to(torch.bfloat16).contiguous() if weight is not None else None
        g = gate.contiguous() if gate is not None else None
        check(lib().tyr_rmsnorm_weighted(ptr(xc), ptr(w), ptr(g), ptr(r), ptr(r_out), ptr(y),
                                         xc.numel() // D, D, eps, 1 if one_plus_w else 0,
                                         cur_stream(x.device)), "rmsnorm_weighted")
        return (y, r_out) if return_residual else y
    xf = x.float()
    if residual is not None:
        xf = xf + residual.float()
        r_out = xf.to(x.dtype)
        xf = r_out.float()
    y = rms_norm_ref(xf, eps)
    if weight is not None:
        w = weight.float() + (1.0 if one_plus_w else 0.0)
        y = y * w
    if gate is not None:
        y = y * torch.nn.functional.silu(gate.float())
    y = y.to(x.dtype)
    return (y, r_out) if (return_residual and residual is not None) else y
