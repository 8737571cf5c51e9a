"""Linear layers for 17 .. 64 rows on the tensor-core weight-streaming kernel (csrc/decode_gemm.cu).

The weights fill the 128-row side of ``tcgen05.mma`` and the tokens the narrow side, so a CTA streams 128 weight rows once
and re-reads the activations from L2 once per 128 rows.  ``decode_linear``: ``x W^T``; ``decode_swiglu``:
``silu(x Wg^T) * (x Wu^T)`` with both matrices streamed once.  A launch uses one CTA per 128 weight rows, so it pays off
when the matrix has enough rows to occupy most SMs (``MIN_ROW_TILES``); smaller matrices stay on the library GEMM.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .._native import register_signatures
from ._common import check, cur_stream, err_word, lib, ptr

MIN_ROWS, MAX_ROWS = 17, 64
# CTAs (of 128 weight rows) below which a product stays where it was.  Alone, a plain product ties with the library GEMM
# (within 3 % either way from 40 tiles on); inside a decode step it is ahead, because its weight loads start while the kernel
# in front of it still runs: Qwen3.5-27B widths, 8 layers, batch 32: 2.19 ms per step with the library for plain products,
# 2.10 ms from 40 tiles on, 2.11 ms from 16.  The gated form replaces three launches and is ahead of both alternatives from
# 64 tiles on.
MIN_ROW_TILES = int(os.environ.get("TYR_DECODE_GEMM_MIN_TILES", "40"))
# ... and above which a plain product goes back to the library: one CTA per tile means several waves for a vocabulary-sized
# matrix (784 tiles: the Laguna decode step was 0.4 % slower with this kernel for the lm_head than with the library).
MAX_ROW_TILES = int(os.environ.get("TYR_DECODE_GEMM_MAX_TILES", "296"))
GATED_MIN_ROW_TILES = int(os.environ.get("TYR_DECODE_GEMM_GATED_MIN_TILES", "64"))
_ENABLED = os.environ.get("TYR_DECODE_GEMM", "1") != "0"


@register_signatures
def _sigs(lib_):
    P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    fn = getattr(lib_, "tyr_decode_gemm_bf16", None)
    if fn is not None:
        fn.argtypes = [P, P, P, P, L, L, L, I, I, I, I, P, P]
        fn.restype = I


def _operand_ok(t: torch.Tensor) -> bool:
    return (t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0
            and t.data_ptr() % 16 == 0)


def supported(x2: torch.Tensor, w: torch.Tensor, w2: Optional[torch.Tensor] = None, min_tiles: Optional[int] = None) -> bool:
    if not (_ENABLED and x2.is_cuda and hasattr(lib(), "tyr_decode_gemm_bf16")):
        return False
    M, K = x2.shape
    N = w.shape[0]
    tiles = (N + 127) // 128
    if not (MIN_ROWS <= M <= MAX_ROWS and K % 64 == 0 and K >= 64 and tiles >= (MIN_ROW_TILES if min_tiles is None else min_tiles)):
        return False
    if min_tiles is None and w2 is None and tiles > MAX_ROW_TILES:
        return False
    if w2 is not None and not (_operand_ok(w2) and w2.shape == w.shape and w2.stride(0) == w.stride(0)):
        return False
    return _operand_ok(x2) and _operand_ok(w) and w.shape[1] == K


def _run(x2, w, w2, out, split: int = 0):
    M, K = x2.shape
    N = w.shape[0]
    y = torch.empty((M, N), dtype=torch.bfloat16, device=x2.device) if out is None else out
    assert y.shape == (M, N) and y.dtype == torch.bfloat16 and y.stride(1) == 1
    check(lib().tyr_decode_gemm_bf16(ptr(x2), ptr(w), ptr(w2), ptr(y), x2.stride(0), w.stride(0), y.stride(0), M, N, K, split,
                                     ptr(err_word(x2.device)), cur_stream(x2.device)), "decode_gemm_bf16")
    return y


def decode_linear(x2: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, split: int = 0) -> torch.Tensor:
    """x2 [17..64, K] bf16, w [N, K] bf16 (rows may be strided) -> [M, N] bf16, fp32 accumulation.  ``split``: CTAs of a
    thread-block cluster that share one 128-row tile's contraction (0: chosen from the shape so that one wave fills the SMs)."""
    if not x2.is_cuda:
        y = (x2.float() @ w.float().T).to(x2.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    return _run(x2, w, None, out, split)


def decode_swiglu(x2: torch.Tensor, gate_w: torch.Tensor, up_w: torch.Tensor, out: Optional[torch.Tensor] = None, split: int = 0) -> torch.Tensor:
    """silu(x2 gate_w^T) * (x2 up_w^T) as [M, N] bf16."""
    if not x2.is_cuda:
        y = (torch.nn.functional.silu(x2.float() @ gate_w.float().T) * (x2.float() @ up_w.float().T)).to(x2.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    return _run(x2, gate_w, up_w, out, split)
