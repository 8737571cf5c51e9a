"""Typed neural-network ops (Tyr/Typed/Neural.lean): RMSNorm family, the attention family with
head-count evidence, rotary embeddings, STFT, and file IO helpers.  GPU bf16 inputs reach the
hand-written kernels of :mod:`tyr_b200.ops`; everything else takes the fp32 oracle path."""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .. import ops as K
from . import shape as sh
from .device import Device
from .dtype import DType
from .spec import StaticSpec
from .tensor import Tensor


def _fail(op: str, msg: str):
    raise TypeError(f"{op}: {msg}")


def rms_norm(x: Tensor, eps: float = 1e-6) -> Tensor:
    """RMS normalisation accumulated in Float32; the result dtype is Float32
    (Tyr/Typed/Neural.lean:38-43)."""
    if not x.dtype.is_real_floating:
        _fail("rmsNorm", f"expects a real floating dtype, got {x.dtype}")
    if x.raw.is_cuda and x.dtype is DType.BFloat16:
        raw = K.rms_norm(x.raw, eps).float()
    else:
        raw = K.rms_norm_ref(x.raw, eps)
    return Tensor.of_raw(raw, x.spec.with_dtype(DType.Float32), "rmsNorm")


def rms_norm_preserving(x: Tensor, weight: Tensor, eps: float = 1e-6) -> Tensor:
    """Normalise in Float32, round back to the input dtype, then multiply the weight (HF order)."""
    if weight.shape != x.shape[-len(weight.shape):]:
        _fail("rmsNormPreserving", f"weight {list(weight.shape)} does not match {list(x.shape)}")
    raw = K.rms_norm_weighted(x.raw, weight.raw, eps)
    return Tensor.of_raw(raw, x.spec, "rmsNormPreserving")


def rms_norm_weighted(x: Tensor, weight: Tensor, eps: float = 1e-6) -> Tensor:
    """(x_f32 * rsqrt(mean(x^2) + eps)) * w, result promoted like the native op
    (cc/src/tyr.cpp:3766-3772)."""
    xf = x.raw.float()
    raw = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.raw
    return Tensor.of_tensor(raw)


def rotary_freqs(seq_len: int, head_dim: int, base: float = 10000.0, device: Device = Device.CPU) -> Tuple[Tensor, Tensor]:
    """(cos, sin) of shape [seq_len, head_dim/2] (cc/src/tyr.cpp:2776-2802)."""
    c, s = K.rotary_freqs(seq_len, head_dim, base, device=device.torch)
    spec = StaticSpec((seq_len, head_dim // 2), DType.Float32, device)
    return Tensor.of_raw(c, spec, "rotaryFreqs"), Tensor.of_raw(s, spec, "rotaryFreqs")


def apply_rotary(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """x: [batch, seq, heads, head_dim]; half-split rotation (cc/src/tyr.cpp:2823-2856)."""
    if x.spec.rank != 4 or cos.shape != (x.shape[1], x.shape[3] // 2) or sin.shape != cos.shape:
        _fail("applyRotary", f"x {list(x.shape)} needs cos/sin of shape [{x.shape[1]}, {x.shape[3] // 2}]")
    return Tensor.of_raw(K.apply_rotary(x.raw, cos.raw, sin.raw), x.spec, "applyRotary")


def _heads(op: str, q: Tensor, k: Tensor, v: Tensor):
    """``AttentionHeads`` evidence: 4-D [B, H, T, D], kv heads divide query heads, K/V agree."""
    if q.spec.rank != 4 or k.spec.rank != 4 or v.spec.rank != 4:
        _fail(op, "expects [batch, heads, seq, head_dim] operands")
    if k.shape != v.shape[:3] + (k.shape[3],) or k.shape[:3] != v.shape[:3]:
        _fail(op, f"key {list(k.shape)} and value {list(v.shape)} disagree")
    if q.shape[0] != k.shape[0] or q.shape[3] != k.shape[3]:
        _fail(op, f"query {list(q.shape)} and key {list(k.shape)} disagree")
    if k.shape[1] == 0 or q.shape[1] % k.shape[1] != 0:
        _fail(op, f"{q.shape[1]} query heads are not a multiple of {k.shape[1]} key/value heads")
    if not (q.dtype is k.dtype is v.dtype):
        _fail(op, "query, key and value must share a dtype")
    return StaticSpec(q.shape[:3] + (v.shape[3],), q.dtype, q.device)


def attention(q: Tensor, k: Tensor, v: Tensor, causal: bool = False) -> Tensor:
    spec = _heads("attention", q, k, v)
    if q.shape[1] != k.shape[1]:
        _fail("attention", "head counts differ; use attention_gqa")
    return Tensor.of_raw(K.attention(q.raw, k.raw, v.raw, causal=causal), spec, "attention")


def attention_gqa(q: Tensor, k: Tensor, v: Tensor, causal: bool = False, scale: Optional[float] = None) -> Tensor:
    spec = _heads("attentionGQA", q, k, v)
    return Tensor.of_raw(K.attention(q.raw, k.raw, v.raw, causal=causal, scale=scale), spec, "attentionGQA")


def attention_window(q: Tensor, k: Tensor, v: Tensor, causal: bool, dropout: bool, window: int) -> Tensor:
    """Sliding window: query i sees keys in (i - window, i] (cc/include/tyr_attention.h:104-128)."""
    spec = _heads("attentionWindow", q, k, v)
    if window <= 0:
        _fail("attentionWindow", "window must be positive")
    return Tensor.of_raw(K.attention(q.raw, k.raw, v.raw, causal=causal, window=window), spec, "attentionWindow")


def attention_gqa_mask(q: Tensor, k: Tensor, v: Tensor, key_padding_mask: Tensor, causal: bool = False) -> Tensor:
    """Key-padding mask [batch, keys], True = attend."""
    spec = _heads("attentionGQAMask", q, k, v)
    if key_padding_mask.shape != (k.shape[0], k.shape[2]):
        _fail("attentionGQAMask", f"mask {list(key_padding_mask.shape)} must be [batch, keys]")
    raw = K.attention(q.raw, k.raw, v.raw, causal=causal, key_padding_mask=key_padding_mask.raw)
    return Tensor.of_raw(raw, spec, "attentionGQAMask")


def attention_edge_mask(q: Tensor, k: Tensor, v: Tensor, edge_mask: Tensor) -> Tensor:
    """Edge mask [batch, queries, keys], True = attend."""
    spec = _heads("attentionEdgeMask", q, k, v)
    if edge_mask.shape != (q.shape[0], q.shape[2], k.shape[2]):
        _fail("attentionEdgeMask", f"mask {list(edge_mask.shape)} must be [batch, queries, keys]")
    raw = K.attention(q.raw, k.raw, v.raw, causal=False, edge_mask=edge_mask.raw)
    return Tensor.of_raw(raw, spec, "attentionEdgeMask")


def attention_gqa_qkv(q: Tensor, k: Tensor, v: Tensor) -> Tensor:
    """Decode form: the queries are the LAST rows of the key sequence (causal with offset)."""
    spec = _heads("attentionGQAQKV", q, k, v)
    return Tensor.of_raw(K.attention(q.raw, k.raw, v.raw, causal=True), spec, "attentionGQAQKV")


def split_heads(x: Tensor) -> Tensor:
    """[B, T, H, D] -> [B, H, T, D]."""
    return Tensor.of_raw(x.raw.transpose(1, 2), x.spec.with_shape(sh.transpose_shape(x.shape, 1, 2)), "splitHeads")


join_heads = split_heads


def hann_window(n: int, device: Device = Device.CPU) -> Tensor:
    return Tensor.of_raw(torch.hann_window(n, device=device.torch), StaticSpec((n,), DType.Float32, device), "hannWindow")


def stft(x: Tensor, n_fft: int, hop: int, window: Tensor) -> Tensor:
    """1-D signal -> complex spectrogram [n_fft/2+1, frames] (centered, reflect padding)."""
    raw = torch.stft(x.raw, n_fft, hop, n_fft, window.raw, center=True, pad_mode="reflect", return_complex=True)
    return Tensor.of_tensor(raw)


def istft(spec: Tensor, n_fft: int, hop: int, window: Tensor, length: Optional[int] = None) -> Tensor:
    return Tensor.of_tensor(torch.istft(spec.raw, n_fft, hop, n_fft, window.raw, center=True, length=length))


def timestep_embedding(t: Tensor, dim: int, max_period: float = 10000.0, time_factor: float = 1000.0) -> Tensor:
    """Sinusoidal embedding [batch, dim] = cat(cos, sin) of t*time_factor*freqs (cc/src/tyr.cpp:2862)."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.raw.device) / half)
    args = (t.raw.float() * time_factor)[:, None] * freqs[None]
    emb = torch.cat([torch.cos(args), torch.sin(args)], dim=-1)
    if dim % 2:
        emb = torch.cat([emb, torch.zeros_like(emb[:, :1])], dim=-1)
    return Tensor.of_raw(emb, StaticSpec((t.shape[0], dim), DType.Float32, t.device), "timestepEmbedding")
