"""One-token attention over a K/V store with the append fused in and the position read on the device
(csrc/decode_attention.cu), so that a decode step has no host-dependent shapes and can be replayed from a CUDA graph.

The CPU path states the same contract in plain PyTorch and is the oracle of the numerics tests."""
from __future__ import annotations

import ctypes
import math
from typing import Dict, Optional, Tuple

import torch

from .._native import register_signatures
from ._common import check, cur_stream, err_word, lib, ptr

_workspaces: Dict[Tuple, torch.Tensor] = {}


@register_signatures
def _sigs(lib_):
    P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    fn = getattr(lib_, "tyr_decode_attention", None)
    if fn is not None:
        fn.argtypes = [P, P, P, P, P, P, P, P, L, L, L, I, I, I, I, I, I, I, I, I, F, P, P]
        fn.restype = I
        g = getattr(lib_, "tyr_decode_attention_gated", None)
        if g is not None:
            g.argtypes = [P, P, P, P, P, P, P, P, L, L, L, I, I, I, I, I, I, I, I, I, F, P, L, L, I, P, P]
            g.restype = I
        lib_.tyr_decode_attention_workspace_bytes.argtypes = [I, I, I, I, I]
        lib_.tyr_decode_attention_workspace_bytes.restype = L


def pick_splits(B: int, Hkv: int, keys: int) -> int:
    """Enough CTAs to fill 148 SMs a few times over, but at least 256 keys per split."""
    want = -(-592 // max(1, B * Hkv))
    return max(1, min(want, 32, -(-keys // 256)))


def geometry_supported(Hq: int, Hkv: int, D: int) -> bool:
    """Up to 16 query heads per K/V head at head dim 64 / 128, up to 8 at head dim 256."""
    return D in (64, 128, 256) and Hkv > 0 and Hq % Hkv == 0 and Hq // Hkv <= (8 if D == 256 else 16)


def supported(q: torch.Tensor, Hkv: int) -> bool:
    B, Hq, D = q.shape
    return q.is_cuda and q.dtype == torch.bfloat16 and geometry_supported(Hq, Hkv, D)


def _rows_ok(t: torch.Tensor, D: int) -> bool:
    return t.stride(2) == 1 and t.stride(1) == D and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0


def decode_attention(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     pos: torch.Tensor, *, ring: bool = False, window: Optional[int] = None, scale: Optional[float] = None,
                     append: bool = True, splits: Optional[int] = None, head_gate: Optional[torch.Tensor] = None,
                     elem_gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q: [B, Hq, D]; k_new, v_new: [B, Hkv, D] (the new position, RoPE applied); stores ``[B, Hkv, cap, D]``;
    ``pos``: int32 tensor holding the absolute position of the new token.  Writes the new K/V at slot ``pos`` (``pos % cap``
    for a ring store) when ``append`` and returns the attention of the new query over the retained keys (all of a ring
    store; the last ``window`` positions of a plain one), ``[B, Hq, D]``.  ``head_gate`` ([B, Hq]) multiplies each head's
    output by ``softplus(gate)``, ``elem_gate`` ([B, Hq, D]) each element by ``sigmoid(gate)``; on the GPU the gate is
    applied inside the kernel's final write."""
    B, Hq, D = q.shape
    Hkv, cap = k_cache.shape[1], k_cache.shape[2]
    sc = scale if scale is not None else 1.0 / math.sqrt(D)
    if not q.is_cuda:
        p = int(pos.reshape(-1)[0])
        if p < 0 or (not ring and p >= cap):
            raise ValueError(f"decode position {p} outside a store of {cap} slots")
        slot = p % cap if ring else p
        if append:
            k_cache[:, :, slot] = k_new
            v_cache[:, :, slot] = v_new
        if ring:
            lo, hi = 0, min(p + 1, cap)
        else:
            lo, hi = (max(0, p + 1 - window) if window else 0), p + 1
        k, v = k_cache[:, :, lo:hi].float().clone(), v_cache[:, :, lo:hi].float().clone()
        k[:, :, slot - lo], v[:, :, slot - lo] = k_new.float(), v_new.float()
        G = Hq // Hkv
        s = torch.einsum("bhgd,bhkd->bhgk", q.float().reshape(B, Hkv, G, D), k) * sc
        o = torch.einsum("bhgk,bhkd->bhgd", torch.softmax(s, -1), v).reshape(B, Hq, D)
        if head_gate is not None:
            o = o * torch.nn.functional.softplus(head_gate.float()).unsqueeze(-1)
        if elem_gate is not None:
            o = o * torch.sigmoid(elem_gate.float())
        return o.to(q.dtype)
    if not supported(q, Hkv):
        raise ValueError(f"decode_attention: unsupported geometry Hq={Hq} Hkv={Hkv} D={D} dtype={q.dtype}")
    if not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise ValueError("decode_attention: K/V stores must be contiguous")
    q, k_new, v_new = (t if _rows_ok(t, D) else t.contiguous() for t in (q, k_new, v_new))
    keys = cap if ring or not window else min(cap, window)
    if splits is None:
        splits = pick_splits(B, Hkv, keys)
    key = (q.device.index, B, Hq, Hkv, D, splits)
    ws = _workspaces.get(key)
    if ws is None:
        ws = _workspaces[key] = torch.zeros(lib().tyr_decode_attention_workspace_bytes(B, Hq, Hkv, D, splits) // 4, dtype=torch.int32, device=q.device)
    out = torch.empty((B, Hq, D), dtype=q.dtype, device=q.device)
    gate, mode = None, 0
    if head_gate is not None:
        gate, mode = head_gate, 1
        assert gate.shape == (B, Hq) and gate.dtype == torch.bfloat16 and elem_gate is None
        gs = (gate.stride(0), gate.stride(1))
    elif elem_gate is not None:
        gate, mode = elem_gate, 2
        assert gate.shape == (B, Hq, D) and gate.dtype == torch.bfloat16 and gate.stride(2) == 1
        gs = (gate.stride(0), gate.stride(1))
    if gate is None:
        check(lib().tyr_decode_attention(ptr(q), ptr(k_new), ptr(v_new), ptr(k_cache), ptr(v_cache), ptr(pos), ptr(out), ptr(ws),
                                         q.stride(0), k_new.stride(0), v_new.stride(0), B, Hq, Hkv, D, cap, 1 if ring else 0, int(window or 0),
                                         splits, 1 if append else 0, sc, ptr(err_word(q.device)), cur_stream(q.device)), "decode_attention")
    else:
        check(lib().tyr_decode_attention_gated(ptr(q), ptr(k_new), ptr(v_new), ptr(k_cache), ptr(v_cache), ptr(pos), ptr(out), ptr(ws),
                                               q.stride(0), k_new.stride(0), v_new.stride(0), B, Hq, Hkv, D, cap, 1 if ring else 0,
                                               int(window or 0), splits, 1 if append else 0, sc, ptr(gate), gs[0], gs[1], mode,
                                               ptr(err_word(q.device)), cur_stream(q.device)), "decode_attention_gated")
    return out
