"""tcgen05 flash-attention bindings (filled in by csrc/attention_*.cu)."""
from __future__ import annotations

import torch

_ENABLED = False


def supported(q, k, v, causal, window) -> bool:
    return False


def supported_packed(H, D, T, causal, window) -> bool:
    return False


def flash_attention(q, k, v, *, causal=True, window=None, scale=None):  # pragma: no cover
    raise NotImplementedError


def flash_attention_packed(qkv, B, T, H, D, *, causal=True, window=None, scale=None):  # pragma: no cover
    raise NotImplementedError
