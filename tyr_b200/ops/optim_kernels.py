"""Bindings for the fused optimizer kernels in csrc/optim.cu (with fp32 torch fallbacks that
double as the numerics oracle on CPU)."""
from __future__ import annotations

from typing import Optional

import torch

from ._common import check, cur_stream, lib, ptr


def adamw_step_(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, *, lr: float,
                beta1: float, beta2: float, eps: float, weight_decay: float, step: int,
                p_bf16: Optional[torch.Tensor] = None, grad_scale: float = 1.0):
    """Bias-corrected AdamW with decoupled weight decay, in place on fp32 ``p``, ``m``, ``v``
    (Tyr/Optim/DistAdam.lean:109-158).  ``p_bf16`` receives the refreshed bf16 working copy."""
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    if p.is_cuda:
        assert p.dtype == torch.float32 and m.dtype == torch.float32 and v.dtype == torch.float32
        assert p.is_contiguous() and g.is_contiguous() and m.is_contiguous() and v.is_contiguous()
        check(lib().tyr_adamw_step(ptr(p), ptr(p_bf16), ptr(g), ptr(m), ptr(v), p.numel(), lr, beta1,
                                   beta2, eps, weight_decay, bc1, bc2, grad_scale,
                                   1 if g.dtype == torch.bfloat16 else 0, cur_stream(p.device)),
              "adamw_step")
        return
    gf = g.float() * grad_scale
    m.mul_(beta1).add_(gf, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    p.mul_(1 - lr * weight_decay).addcdiv_(m / bc1, (v / bc2).sqrt() + eps, value=-lr)
    if p_bf16 is not None:
        p_bf16.copy_(p)


def muon_momentum_(g: torch.Tensor, mom: torch.Tensor, u: torch.Tensor, sumsq: torch.Tensor,
                   mu: float, grad_scale: float = 1.0):
    """Stacked [B, R, C]: mom = mu*mom + (1-mu)*g ; u = bf16((1-mu)*g + mu*mom) ;
    sumsq[b] += ||u_b||_F^2 (Tyr/Optim/NorMuon.lean:196-203, 240-243)."""
    B = g.shape[0]
    per = g[0].numel()
    if g.is_cuda:
        assert g.is_contiguous() and mom.is_contiguous() and u.is_contiguous()
        check(lib().tyr_muon_momentum(ptr(g), ptr(mom), ptr(u), ptr(sumsq), per, B, mu, grad_scale,
                                      1 if g.dtype == torch.bfloat16 else 0, cur_stream(g.device)),
              "muon_momentum")
        return
    gf = g.float() * grad_scale
    mom.mul_(mu).add_(gf, alpha=1 - mu)
    uu = ((1 - mu) * gf + mu * mom).to(u.dtype)
    u.copy_(uu)
    sumsq.add_(uu.float().reshape(B, -1).pow(2).sum(1))


def scale_by_inv_norm_(x: torch.Tensor, sumsq: torch.Tensor, eps: float = 1e-7):
    """x[b] /= (sqrt(sumsq[b]) + eps) on a stacked bf16 batch (cc/src/tyr_polar.cpp:292-293)."""
    B = x.shape[0]
    if x.is_cuda:
        check(lib().tyr_scale_by_inv_norm(ptr(x), ptr(sumsq), x[0].numel(), B, eps,
                                          cur_stream(x.device)), "scale_by_inv_norm")
        return
    inv = 1.0 / (sumsq.sqrt() + eps)
    x.copy_((x.float() * inv.reshape(B, *([1] * (x.dim() - 1)))).to(x.dtype))


def muon_apply_(p: torch.Tensor, o: torch.Tensor, lr: float, weight_decay: float,
                p_bf16: Optional[torch.Tensor] = None):
    """p = p*(1 - lr*wd) - bf16(lr * o) on fp32 master weights; refreshes the bf16 copy."""
    if p.is_cuda:
        assert p.is_contiguous() and o.is_contiguous()
        check(lib().tyr_muon_apply(ptr(p), ptr(p_bf16), ptr(o), p.numel(), lr, weight_decay,
                                   cur_stream(p.device)), "muon_apply")
        return
    upd = (o.to(torch.bfloat16).float() * lr).to(torch.bfloat16).float()
    p.mul_(1 - lr * weight_decay).sub_(upd)
    if p_bf16 is not None:
        p_bf16.copy_(p)
