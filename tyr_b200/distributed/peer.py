"""Reduce-scatter / all-gather / all-reduce over the symmetric heap with the repository's own kernels.

The public optimizer steps (``optim/distadam.step_distributed``, ``optim/normuon.step_distributed_group`` and
``step_distributed_owner``) follow the reference's sequence of collectives (Tyr/Optim/DistAdam.lean:185-267,
Tyr/Optim/NorMuon.lean:346-425).  With ``distributed.enable_peer_collectives()`` those collectives stop being NCCL calls:
every rank copies its operand into a staging buffer of the heap, a device-side flag barrier (bounded waits, error word
instead of a hang) makes the copies visible, and one kernel pulls the pieces it needs from the peers with 16-byte loads over
NVLink (``tyr_peer_sum``: sum of one slice over all ranks; ``tyr_peer_gather``: every rank's piece).  A second barrier keeps
the staging buffer from being overwritten while a peer still reads it.  fp32 operands go through unchanged; bf16 / fp16
operands are staged and summed in fp32 and rounded once at the end.

The trainer's own data-parallel step does not come through here: ``parallel/dp.py`` fuses the optimizer into the exchange.
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence

import torch

from .._native import kernels, register_signatures
from ..ops._common import check, cur_stream, err_word
from .symm import FlagBarrier, SymmetricHeap


@register_signatures
def _sigs(lib):
    P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    PP = ctypes.POINTER(ctypes.c_void_p)
    fn = getattr(lib, "tyr_peer_gather", None)
    if fn is not None:
        fn.argtypes = [PP, I, L, P, L, P]
        fn.restype = ctypes.c_int


_FLOAT = (torch.float32, torch.bfloat16, torch.float16)


class PeerCollectives:
    def __init__(self, rank: int, world_size: int, device, capacity_bytes: int = 256 << 20, group=None):
        self.rank, self.world = rank, world_size
        self.device = torch.device(device)
        self.capacity = capacity_bytes // 16 * 4          # fp32 elements, a multiple of 4
        self.heap = SymmetricHeap(self.capacity * 4 + (1 << 16), rank, world_size, self.device, group)
        self.staging = self.heap.alloc((self.capacity,), torch.float32)
        self.barrier = FlagBarrier(self.heap, n_slots=2)
        self._table = self.heap.peer_table_at(self.heap.offset_bytes(self.staging))

    # ------------------------------------------------------------------------------------------------------------
    def supports(self, t: torch.Tensor, copies: int = 1) -> bool:
        """``copies``: how many tensors of this size the operation stages (the list forms stage ``world``)."""
        return (t.is_cuda and t.device == self.device and t.dtype in _FLOAT and t.numel() > 0
                and self._pad4(t.numel()) * copies <= self.capacity)

    @staticmethod
    def _pad4(n: int) -> int:
        return (n + 3) // 4 * 4

    def _err(self):
        return ctypes.c_void_p(err_word(self.device).data_ptr())

    def _publish(self):
        self.barrier.barrier_device_seq(0, self._err())

    def _release(self):
        self.barrier.barrier_device_seq(1, self._err())

    def _sum(self, off: int, n: int, scale: float) -> torch.Tensor:
        out = torch.empty(n, dtype=torch.float32, device=self.device)
        check(kernels().tyr_peer_sum(self._table, self.world, off, ctypes.c_void_p(out.data_ptr()), n, scale,
                                     cur_stream(self.device)), "peer_sum")
        return out

    # ------------------------------------------------------------------------------------------------------------
    def all_reduce(self, t: torch.Tensor, avg: bool) -> torch.Tensor:
        n = t.numel()
        self.staging[:n].copy_(t.detach().reshape(-1))
        self._publish()
        out = self._sum(0, n, 1.0 / self.world if avg else 1.0)
        self._release()
        return out.to(t.dtype).reshape(t.shape)

    def reduce_scatter(self, t: torch.Tensor, avg: bool) -> torch.Tensor:
        """Dim 0 of ``t`` split into ``world`` chunks; this rank's chunk summed over the ranks."""
        n = t.numel()
        per = n // self.world
        self.staging[:n].copy_(t.detach().reshape(-1))
        self._publish()
        out = self._sum(self.rank * per, per, 1.0 / self.world if avg else 1.0)
        self._release()
        return out.to(t.dtype).reshape((t.shape[0] // self.world,) + tuple(t.shape[1:]))

    def reduce_scatter_list(self, ts: Sequence[torch.Tensor], avg: bool) -> torch.Tensor:
        """``ts[r]`` is this rank's contribution to rank r's result."""
        n = ts[0].numel()
        pad = self._pad4(n)
        for r, x in enumerate(ts):
            self.staging[r * pad:r * pad + n].copy_(x.detach().reshape(-1))
        self._publish()
        out = self._sum(self.rank * pad, n, 1.0 / self.world if avg else 1.0)
        self._release()
        return out.to(ts[0].dtype).reshape(ts[0].shape)

    def _gather(self, t: torch.Tensor) -> torch.Tensor:
        n = t.numel()
        pad = self._pad4(n)
        self.staging[:n].copy_(t.detach().reshape(-1))
        self._publish()
        out = torch.empty(self.world * pad, dtype=torch.float32, device=self.device)
        check(kernels().tyr_peer_gather(self._table, self.world, 0, ctypes.c_void_p(out.data_ptr()), pad,
                                        cur_stream(self.device)), "peer_gather")
        self._release()
        return out.reshape(self.world, pad)[:, :n]

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        """Concatenation of every rank's tensor along dim 0."""
        inp = t.reshape(1) if t.dim() == 0 else t
        g = self._gather(inp)
        return g.to(t.dtype).reshape((inp.shape[0] * self.world,) + tuple(inp.shape[1:]))

    def all_gather_list(self, t: torch.Tensor) -> List[torch.Tensor]:
        g = self._gather(t).to(t.dtype)
        return [g[r].reshape(t.shape).clone() for r in range(self.world)]

    def close(self):
        self.heap.close()
