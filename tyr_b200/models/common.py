"""Shared inference building blocks for the decoder families (Laguna, Qwen3, Qwen3.5, Gemma4, ...).

* ``lin``: bias-free/biased projection; prefill-sized bf16 batches go to the tcgen05 GEMM, batches of up to 16 rows
  to the weight-streaming kernel, the sizes in between to the library GEMM.
* rotary tables (plain / YaRN / partial), HF rotate-half application.
* ``KVCache``: static and ring (sliding-window) stores with in-place writes; the session owns the
  tensors (Tyr/Model/Laguna/Model.lean:351-406, Tyr/Model/Qwen/Model.lean KVCache).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..ops.gemm import gemm as _gemm
from ..ops import decode_gemm as _decode_gemm
from ..ops import skinny as _skinny
from ..ops.attention import attention
from ..ops.norm import rms_norm_weighted

TCGEN05_MIN_ROWS = 128


def lin(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None, act: Optional[str] = None) -> torch.Tensor:
    """``act(x @ w^T + b)`` with ``w: [out, in]``.  No autograd on the tensor-core path (inference)."""
    rows = x.numel() // x.shape[-1]
    if (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and rows >= TCGEN05_MIN_ROWS
            and not torch.is_grad_enabled() and w.shape[1] % 8 == 0 and w.shape[0] % 8 == 0 and w.is_contiguous()):
        y = _gemm(x.reshape(rows, -1).contiguous(), w, a_layout="K", b_layout="K",
                       act=act if b is None else None).reshape(*x.shape[:-1], w.shape[0])
        if b is not None:
            y = y + b
            if act == "relu":
                y = F.relu(y)
        return y
    if rows <= _skinny.MAX_ROWS and x.is_cuda and not torch.is_grad_enabled():
        x2 = x.reshape(rows, -1)
        if _skinny.supported(x2, w):
            y = _skinny.skinny_linear(x2, w, b).reshape(*x.shape[:-1], w.shape[0])
            return F.relu(y) if act == "relu" else (F.relu(y).square() if act == "relu2" else y)
    if rows <= _decode_gemm.MAX_ROWS and x.is_cuda and b is None and act is None and not torch.is_grad_enabled():
        x2 = x.reshape(rows, -1)
        if _decode_gemm.supported(x2, w):                # 17 .. 64 rows, matrices with enough 128-row tiles (ops/decode_gemm.py)
            return _decode_gemm.decode_linear(x2, w).reshape(*x.shape[:-1], w.shape[0])
    y = F.linear(x, w.to(x.dtype), None if b is None else b.to(x.dtype))
    if act == "relu":
        y = F.relu(y)
    elif act == "relu2":
        y = F.relu(y).square()
    return y


def swiglu_mlp(x, gate_w, up_w, down_w):
    rows = x.numel() // x.shape[-1]
    if rows <= _decode_gemm.MAX_ROWS and x.is_cuda and not torch.is_grad_enabled():
        x2 = x.reshape(rows, -1)
        if _decode_gemm.supported(x2, gate_w, up_w, min_tiles=_decode_gemm.GATED_MIN_ROW_TILES):
            # 17 .. 64 rows and a wide MLP: weights on the 128-row side of the tensor core, SwiGLU in the epilogue
            return lin(_decode_gemm.decode_swiglu(x2, gate_w, up_w).reshape(*x.shape[:-1], gate_w.shape[0]), down_w)
    if rows <= _skinny.MAX_ROWS and x.is_cuda and not torch.is_grad_enabled():
        x2 = x.reshape(rows, -1)
        if _skinny.swiglu_supported(x2, gate_w, up_w):          # decode: gate and up in one pass, SwiGLU in the epilogue
            return lin(_skinny.skinny_swiglu(x2, gate_w, up_w).reshape(*x.shape[:-1], gate_w.shape[0]), down_w)
    return lin(F.silu(lin(x, gate_w)) * lin(x, up_w), down_w)


def norm_w(x, w, eps, one_plus_w: bool = False, residual=None, return_residual: bool = False):
    """Weighted RMSNorm; with ``residual`` the norm is taken of ``x + residual`` in the same kernel and, with
    ``return_residual``, the sum comes back as the second result (the new residual stream)."""
    return rms_norm_weighted(x, w, eps, one_plus_w=one_plus_w, residual=residual, return_residual=return_residual)


# ---- rotary ---------------------------------------------------------------------------------------
def plain_inv_freq(half: int, base: float) -> List[float]:
    dim = 2.0 * half
    return [base ** (-(2.0 * j / dim)) for j in range(half)]


def yarn_correction_range(dim: int, base: float, max_pos: int, beta_fast: float, beta_slow: float) -> Tuple[int, int]:
    def corr(rot):
        return dim * math.log(max_pos / (rot * 2.0 * math.pi)) / (2.0 * math.log(base))
    low = min(max(math.floor(corr(beta_fast)), 0.0), dim - 1.0)
    high = min(max(math.ceil(corr(beta_slow)), 0.0), dim - 1.0)
    return int(low), int(high)


def yarn_inv_freq(half: int, base: float, factor: float, max_pos: int, beta_fast: float, beta_slow: float) -> List[float]:
    """HF ``_compute_yarn_parameters`` in double precision (Tyr/Model/Laguna/Rope.lean:85-121)."""
    dim = 2 * half
    low, high = yarn_correction_range(dim, base, max_pos, beta_fast, beta_slow)
    denom = max(float(high - low), 1.0)
    out = []
    for j in range(half):
        pos_freq = base ** (2.0 * j / dim)
        ramp = min(max((j - low) / denom, 0.0), 1.0)
        out.append((1.0 / (factor * pos_freq)) * ramp + (1.0 / pos_freq) * (1.0 - ramp))
    return out


def cos_sin_tables(inv_freq: Sequence[float], max_len: int, scale: float = 1.0, device="cpu"):
    """fp32 ``[max_len, half]`` tables computed in double precision."""
    f = torch.tensor(list(inv_freq), dtype=torch.float64)
    ang = torch.arange(max_len, dtype=torch.float64)[:, None] * f[None, :]
    return (torch.cos(ang) * scale).float().to(device), (torch.sin(ang) * scale).float().to(device)


def apply_rotary_partial(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [B, S, H, D]; cos/sin: [S, half] (or [B, S, half]).  HF rotate-half over the first ``2*half``
    channels; the tail passes through (Tyr/Model/Laguna/Rope.lean:177-194)."""
    half = cos.shape[-1]
    c = cos.unsqueeze(-2) if cos.dim() == 3 else cos[None, :, None, :]
    s = sin.unsqueeze(-2) if sin.dim() == 3 else sin[None, :, None, :]
    x1, x2, rest = x[..., :half].float(), x[..., half:2 * half].float(), x[..., 2 * half:]
    o1 = x1 * c - x2 * s
    o2 = x2 * c + x1 * s
    return torch.cat([o1.to(x.dtype), o2.to(x.dtype), rest], dim=-1)


def head_norm(x: torch.Tensor, w: torch.Tensor, eps: float, one_plus_w: bool = False) -> torch.Tensor:
    """Per-head RMSNorm over the last dim of [B, S, H, D]."""
    return rms_norm_weighted(x, w, eps, one_plus_w=one_plus_w)


# ---- KV caches -----------------------------------------------------------------------------------------
@dataclass
class KVCache:
    """K/V stores ``[B, Hkv, cap, D]``.  ``ring`` stores keep the last ``cap`` positions at slot
    ``position % cap``; RoPE is already applied so slot order is irrelevant to a single query."""
    k: torch.Tensor
    v: torch.Tensor
    ring: bool = False
    length: int = 0           # absolute positions written so far

    @staticmethod
    def allocate(batch: int, kv_heads: int, cap: int, head_dim: int, device, dtype, ring: bool = False) -> "KVCache":
        if cap <= 0:
            raise ValueError("cache capacity must be positive")
        shape = (batch, kv_heads, cap, head_dim)
        return KVCache(torch.zeros(shape, device=device, dtype=dtype), torch.zeros(shape, device=device, dtype=dtype), ring)

    @property
    def cap(self) -> int:
        return self.k.shape[2]

    def write(self, k_new: torch.Tensor, v_new: torch.Tensor) -> None:
        """Append ``[B, Hkv, S, D]`` at absolute position ``self.length``."""
        S, cap, pos = k_new.shape[2], self.cap, self.length
        if not self.ring:
            if pos + S > cap:
                raise ValueError(f"KV cache overflow: {pos}+{S} > {cap}")
            self.k[:, :, pos:pos + S].copy_(k_new)
            self.v[:, :, pos:pos + S].copy_(v_new)
        else:
            keep = min(S, cap)
            src0 = S - keep
            slot = (pos + src0) % cap
            first = min(keep, cap - slot)
            self.k[:, :, slot:slot + first].copy_(k_new[:, :, src0:src0 + first])
            self.v[:, :, slot:slot + first].copy_(v_new[:, :, src0:src0 + first])
            if first < keep:
                self.k[:, :, :keep - first].copy_(k_new[:, :, src0 + first:])
                self.v[:, :, :keep - first].copy_(v_new[:, :, src0 + first:])
        self.length = pos + S

    def view(self) -> Tuple[torch.Tensor, torch.Tensor]:
        n = min(self.length, self.cap)
        return self.k[:, :, :n], self.v[:, :, :n]

    def clone(self) -> "KVCache":
        return KVCache(self.k.clone(), self.v.clone(), self.ring, self.length)

    def nbytes(self) -> int:
        return self.k.numel() * self.k.element_size() * 2


def cached_attention(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, cache: Optional[KVCache],
                     window: Optional[int], scale: Optional[float] = None) -> torch.Tensor:
    """q: [B, H, S, D]; k_new/v_new: [B, Hkv, S, D].  Prefill (cache empty or absent) attends over the
    fresh K/V with causal / window masking; a decode step (S == 1) attends over everything retained."""
    S = q.shape[2]
    if cache is None:
        return attention(q, k_new, v_new, causal=True, window=window, scale=scale)
    fresh = cache.length == 0
    cache.write(k_new, v_new)
    if fresh:
        return attention(q, k_new, v_new, causal=True, window=window, scale=scale)
    if S != 1:
        if cache.ring:
            raise ValueError("chunked prefill into a ring cache is not supported")
        k, v = cache.view()
        return attention(q, k, v, causal=True, window=window, scale=scale)
    k, v = cache.view()
    if window is not None and not cache.ring and k.shape[2] > window:
        k, v = k[:, :, -window:], v[:, :, -window:]
    return attention(q, k, v, causal=False, scale=scale)
