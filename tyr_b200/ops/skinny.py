"""Decode-sized linear layers (1..32 rows) on the weight-streaming kernel (csrc/skinny_gemm.cu)."""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .._native import register_signatures
from ._common import check, cur_stream, lib, ptr

MAX_ROWS = 32
_workspaces = {}


def _workspace(device, M: int, N: int) -> torch.Tensor:
    """fp32 [M * N] scratch of the split reduction; zero between calls (the finishing kernel re-zeroes what it read)."""
    key = (device.index, M * N)
    ws = _workspaces.get(key)
    if ws is None:
        ws = _workspaces[key] = torch.zeros(M * N, dtype=torch.float32, device=device)
    return ws


@register_signatures
def _sigs(lib_):
    P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    fn = getattr(lib_, "tyr_skinny_gemm_bf16", None)
    if fn is not None:
        fn.argtypes = [P, P, P, P, P, L, L, L, I, I, I, P]
        fn.restype = I
        lib_.tyr_skinny_gemm_splits.argtypes = [I, I]
        lib_.tyr_skinny_gemm_splits.restype = I
    fn = getattr(lib_, "tyr_skinny_swiglu_bf16", None)
    if fn is not None:
        fn.argtypes = [P, P, P, P, L, L, L, I, I, I, P]
        fn.restype = I


LINEAR_MAX_ROWS = 16     # plain products above this many rows go to the library GEMM (measured 2.5x faster at 32 rows)


def supported(x2: torch.Tensor, w: torch.Tensor, max_rows: int = LINEAR_MAX_ROWS) -> bool:
    M, K = x2.shape
    # 9..16 rows with a long contraction leave too few loads in flight per warp; the library GEMM is faster there
    return (x2.is_cuda and x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 1 <= M <= min(max_rows, MAX_ROWS) and (M <= 8 or K <= 8192) and K >= 32 and K % 32 == 0
            and x2.stride(1) == 1 and w.stride(1) == 1 and x2.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x2.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def skinny_linear(x2: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x2: [M <= 32, K] bf16, w: [N, K] bf16 (rows may be strided) -> [M, N] bf16 with fp32 accumulation; ``out`` (rows may be
    strided, e.g. a window of a symmetric-heap buffer) receives the result when given."""
    M, K = x2.shape
    N = w.shape[0]
    if not x2.is_cuda:
        y = x2.float() @ w.float().T
        y = (y if bias is None else y + bias.float()).to(x2.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    y = torch.empty((M, N), dtype=torch.bfloat16, device=x2.device) if out is None else out
    assert y.shape == (M, N) and y.dtype == torch.bfloat16 and y.stride(1) == 1
    b = None if bias is None else bias.to(torch.bfloat16).contiguous()
    ws = _workspace(x2.device, M, N) if lib().tyr_skinny_gemm_splits(N, K) > 1 else None
    check(lib().tyr_skinny_gemm_bf16(ptr(x2), ptr(w), ptr(b), ptr(y), ptr(ws), x2.stride(0), w.stride(0), y.stride(0), M, N, K, cur_stream(x2.device)), "skinny_gemm_bf16")
    return y


_SWIGLU = os.environ.get("TYR_SKINNY_SWIGLU", "1") != "0"


def swiglu_supported(x2: torch.Tensor, gate_w: torch.Tensor, up_w: torch.Tensor) -> bool:
    # the gated form replaces a library product plus two element-wise launches and stays ahead of them up to 32 rows
    return (_SWIGLU and supported(x2, gate_w, MAX_ROWS) and supported(x2, up_w, MAX_ROWS) and gate_w.shape == up_w.shape and gate_w.stride(0) == up_w.stride(0)
            and hasattr(lib(), "tyr_skinny_swiglu_bf16"))


def skinny_swiglu(x2: torch.Tensor, gate_w: torch.Tensor, up_w: torch.Tensor) -> torch.Tensor:
    """x2: [M <= 32, K] bf16 -> silu(x2 gate_w^T) * (x2 up_w^T) as [M, N] bf16: both matrices streamed once, one launch."""
    M, K = x2.shape
    N = gate_w.shape[0]
    if not x2.is_cuda:
        return (torch.nn.functional.silu(x2.float() @ gate_w.float().T) * (x2.float() @ up_w.float().T)).to(x2.dtype)
    y = torch.empty((M, N), dtype=torch.bfloat16, device=x2.device)
    check(lib().tyr_skinny_swiglu_bf16(ptr(x2), ptr(gate_w), ptr(up_w), ptr(y), x2.stride(0), gate_w.stride(0), N, M, N, K, cur_stream(x2.device)),
          "skinny_swiglu")
    return y
