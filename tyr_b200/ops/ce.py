"""Soft-capped cross-entropy fused with the language-model head.

``lm_head_ce`` never materialises the ``[tokens, vocab]`` fp32 logits the reference builds
(linear -> softcap -> cross_entropy, Examples/NanoChat/ModdedGPT.lean:626-650 and
cc/src/tyr.cpp:2063-2072).  It walks the tokens in row chunks: tcgen05 GEMM -> bf16 logits chunk
-> ``softcap_ce`` kernel (loss + in-place gradient) -> the two gradient GEMMs.  The gradients are
therefore produced during the forward pass; backward only rescales them.
"""
from __future__ import annotations

from typing import Optional

import torch

from ._common import check, cur_stream, lib, ptr
from .gemm import gemm


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """cap * tanh(x / cap) (cc/src/tyr.cpp:2769-2773)."""
    return cap * torch.tanh(x / cap)


def softcap_ce_ref(logits: torch.Tensor, targets: torch.Tensor, cap: float,
                   ignore_index: int = -100):
    z = logits.float()
    if cap > 0:
        z = softcap(z, cap)
    return torch.nn.functional.cross_entropy(z, targets, reduction="none", ignore_index=ignore_index)


def softcap_ce_(logits: torch.Tensor, targets: torch.Tensor, cap: float, gscale: float = 1.0,
                gscale_dev: Optional[torch.Tensor] = None, ignore_index: int = -100,
                write_grad: bool = True, bad_count: Optional[torch.Tensor] = None) -> torch.Tensor:
    """In place: ``logits`` (bf16 [rows, V]) is overwritten by
    ``gscale * gscale_dev * dloss/dlogits``.  Returns the per-row losses (fp32).  Targets outside
    ``[0, V)`` give zero loss and zero gradient and are counted in ``bad_count``."""
    rows, V = logits.shape
    if logits.is_cuda:
        loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        check(lib().tyr_softcap_ce(ptr(logits), ptr(targets), ptr(loss), ptr(bad_count), rows, V,
                                   logits.stride(0), cap, gscale, ptr(gscale_dev), ignore_index,
                                   1 if write_grad else 0, cur_stream(logits.device)), "softcap_ce")
        return loss
    with torch.enable_grad():
        l = logits.detach().float().requires_grad_(True)
        valid = (targets != ignore_index) & (targets >= 0) & (targets < V)
        t = torch.where(valid, targets, torch.full_like(targets, ignore_index))
        loss = softcap_ce_ref(l, t, cap, ignore_index)
        if write_grad:
            (g,) = torch.autograd.grad(loss.sum(), l)
            g = g * gscale
            if gscale_dev is not None:
                g = g * gscale_dev.float()
            logits.copy_(g.to(logits.dtype))
    return loss.detach()


class _LmHeadCeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, targets, cap, chunk_rows, loss_scale, ignore_index):
        N, d = x.shape
        need_grad = x.requires_grad or w.requires_grad
        count = (targets != ignore_index).sum().clamp(min=1).float()
        inv = (loss_scale / count).reshape(1)  # device scalar: no host sync
        dx = torch.empty_like(x) if need_grad else None
        mg = getattr(w, "main_grad", None)
        dw32 = None
        if need_grad and w.requires_grad and mg is None:
            dw32 = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        dw_target = mg if mg is not None else dw32
        losses = torch.empty(N, dtype=torch.float32, device=x.device)
        bad = torch.zeros(1, dtype=torch.int32, device=x.device) if x.is_cuda else None
        for r0 in range(0, N, chunk_rows):
            r1 = min(N, r0 + chunk_rows)
            xc = x[r0:r1]
            logits = gemm(xc, w, a_layout="K", b_layout="K")
            losses[r0:r1] = softcap_ce_(logits, targets[r0:r1], cap, 1.0, inv, ignore_index,
                                        write_grad=need_grad, bad_count=bad)
            if need_grad:
                gemm(logits, w, a_layout="K", b_layout="MN", out=dx[r0:r1])
                if dw_target is not None:
                    gemm(logits, xc, a_layout="MN", b_layout="MN", out=dw_target, accumulate=True)
            del logits
        loss = losses.sum() * inv[0]
        if mg is not None and need_grad:
            w.grad_ready = True
        ctx.save_for_backward(dx, dw32)
        ctx.bad_count = bad
        return loss

    @staticmethod
    def backward(ctx, g):
        dx, dw32 = ctx.saved_tensors
        gx = gw = None
        if dx is not None and ctx.needs_input_grad[0]:
            gx = (dx.float() * g).to(dx.dtype)
        if dw32 is not None:
            gw = (dw32 * g).to(torch.bfloat16 if dw32.is_cuda else dw32.dtype)
        return gx, gw, None, None, None, None, None


def lm_head_ce(x: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, cap: float = 15.0,
               chunk_rows: int = 8192, loss_scale: float = 1.0, ignore_index: int = -100):
    """Mean (over non-ignored targets) soft-capped cross-entropy of ``softcap(x @ w^T)``.

    x: [tokens, d]; w: [vocab, d]; targets: int64 [tokens].  ``loss_scale`` (for example
    1/grad_accum_steps) is folded into the gradients while they are produced.  When ``w`` carries
    a ``main_grad`` fp32 buffer its gradient is accumulated there during the forward pass, so the
    upstream gradient given to backward must then be 1."""
    return _LmHeadCeFn.apply(x, w, targets, cap, chunk_rows, loss_scale, ignore_index)
