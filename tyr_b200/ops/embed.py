"""Embedding-table gradient from rows sorted by token id (csrc/embed.cu)."""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch

from .._native import register_signatures
from ._common import check, cur_stream, lib, ptr


@register_signatures
def _sigs(lib_):
    P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    fn = getattr(lib_, "tyr_embed_grad_sorted", None)
    if fn is not None:
        fn.argtypes = [P, P, P, P, I, I, L, I, P]
        fn.restype = I


def sort_tokens(idx: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(sorted ids, order) of a flat int64 token vector; one sort serves every table indexed by the same tokens."""
    sorted_ids, order = torch.sort(idx.reshape(-1))
    return sorted_ids.contiguous(), order.contiguous()


def embedding_grad_(grad_table: torch.Tensor, dy: torch.Tensor, idx: torch.Tensor, sorted_ids=None, order=None) -> None:
    """grad_table[idx[n]] += dy[n] (fp32 table [V, d], dy [N, d]).  bf16 rows on the GPU go through the sorted
    segment-sum kernel; everything else through ``index_add_``."""
    flat = dy.reshape(-1, dy.shape[-1])
    if (flat.is_cuda and flat.dtype == torch.bfloat16 and grad_table.dtype == torch.float32 and grad_table.is_contiguous()
            and flat.shape[1] % 8 == 0 and flat.stride(1) == 1 and flat.stride(0) % 8 == 0 and flat.data_ptr() % 16 == 0
            and hasattr(lib(), "tyr_embed_grad_sorted")):
        if sorted_ids is None or order is None:
            sorted_ids, order = sort_tokens(idx)
        N, d = flat.shape
        check(lib().tyr_embed_grad_sorted(ptr(flat), ptr(order), ptr(sorted_ids), ptr(grad_table), N, d, flat.stride(0),
                                          grad_table.shape[0], cur_stream(flat.device)), "embed_grad_sorted")
        return
    grad_table.index_add_(0, idx.reshape(-1), flat.to(grad_table.dtype))
