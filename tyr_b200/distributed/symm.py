"""Symmetric heap over NVLink peer memory.

Every rank allocates one device buffer of the same size with ``cudaMalloc``, exports it with
CUDA IPC, and maps every peer's buffer (``cudaIpcOpenMemHandle``).  Tensors are bump-allocated
from the buffer in the same order on every rank, so an element offset is valid on every rank and
kernels receive a table of peer base pointers plus one offset.  Signal flags live in the same
heap.  This is what the fused compute+collective kernels (csrc/comm_fused.cu) read and write
with plain P2P loads and stores; NCCL is only used to exchange the 64-byte IPC handles.

The reference has no counterpart (its collectives are c10d calls on private clones,
Tyr/Distributed.lean:43-78); the nearest notion is ``ShardedTensor``'s gather cache.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch

from .._native import kernels, register_signatures
from ..ops._common import check, cur_stream


@register_signatures
def _sigs(lib):
    P, I, L, F, U = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_ulonglong
    PP = ctypes.POINTER(ctypes.c_void_p)
    table = {
        "tyr_symm_alloc": [PP, L], "tyr_symm_free": [P], "tyr_ipc_export": [P, P],
        "tyr_ipc_open": [P, PP], "tyr_ipc_close": [P],
        "tyr_signal": [PP, I, I, I, U, P], "tyr_wait_all": [P, I, I, U, P, P], "tyr_wait_all_budget": [P, I, I, U, P, L, P], "tyr_barrier_dev": [PP, P, I, I, I, P, P, P],
        "tyr_dp_adam_shard": [PP, PP, I, L, L, P, P, P, L] + [F] * 8 + [P, I, U, P, I, P],
        "tyr_dp_muon_gather": [PP, I, P, P, P, P, L, I, F, F, P, I, U, P, I, P],
        "tyr_dp_muon_apply_push": [PP, I, P, P, P, L, I, F, F, I, P],
        "tyr_peer_sum": [PP, I, L, P, L, F, P],
    }
    for name, args in table.items():
        fn = getattr(lib, name, None)
        if fn is not None:
            fn.argtypes = args
            fn.restype = ctypes.c_int


class _DevMem:
    """Minimal __cuda_array_interface__ holder so torch can view raw device memory."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2, "strides": None}


class SymmetricHeap:
    ALIGN = 256

    def __init__(self, nbytes: int, rank: int, world_size: int, device, group=None):
        self.rank, self.world_size = rank, world_size
        self.device = torch.device(device)
        self.nbytes = (nbytes + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        lib = kernels()
        cur_stream(self.device)  # binds the device inside the kernel library
        p = ctypes.c_void_p()
        check(lib.tyr_symm_alloc(ctypes.byref(p), self.nbytes), "symm_alloc")
        self.local_ptr = p.value
        self._bytes = torch.as_tensor(_DevMem(self.local_ptr, self.nbytes), device=self.device)
        self.peer_ptrs: List[int] = [0] * world_size
        self.peer_ptrs[rank] = self.local_ptr
        self._cursor = 0
        self._opened: List[int] = []
        if world_size > 1:
            self._rendezvous(group)

    def _rendezvous(self, group):
        import torch.distributed as dist
        lib = kernels()
        handle = (ctypes.c_ubyte * 64)()
        check(lib.tyr_ipc_export(ctypes.c_void_p(self.local_ptr), handle), "ipc_export")
        mine = bytes(handle)
        gathered: List[Optional[bytes]] = [None] * self.world_size
        dist.all_gather_object(gathered, mine, group=group)
        for r, h in enumerate(gathered):
            if r == self.rank:
                continue
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
            out = ctypes.c_void_p()
            check(lib.tyr_ipc_open(buf, ctypes.byref(out)), f"ipc_open(rank {r})")
            self.peer_ptrs[r] = out.value
            self._opened.append(out.value)
        dist.barrier(group=group)

    # -- allocation ---------------------------------------------------------------------------
    def alloc(self, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        start = (self._cursor + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        if start + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: need {start + nbytes} of {self.nbytes} bytes")
        self._cursor = start + nbytes
        t = self._bytes[start:start + nbytes].view(dtype).reshape(tuple(shape))
        t._symm_offset_bytes = start
        return t

    def offset_bytes(self, t: torch.Tensor) -> int:
        """Byte offset of (a view of) a heap tensor from the heap base (same on every rank)."""
        off = t.data_ptr() - self.local_ptr
        if off < 0 or off >= self.nbytes:
            raise ValueError("tensor does not live in this symmetric heap")
        return off

    def peer_table(self):
        arr = (ctypes.c_void_p * self.world_size)(*self.peer_ptrs)
        return arr

    def peer_table_at(self, byte_offset: int):
        return (ctypes.c_void_p * self.world_size)(*[p + byte_offset for p in self.peer_ptrs])

    def close(self):
        lib = kernels()
        for p in self._opened:
            lib.tyr_ipc_close(ctypes.c_void_p(p))
        self._opened = []
        if self.local_ptr:
            self._bytes = None
            lib.tyr_symm_free(ctypes.c_void_p(self.local_ptr))
            self.local_ptr = 0


class FlagBarrier:
    """Monotonic flag barrier in symmetric memory: ``signal(slot, v)`` writes v into slot
    ``[slot*world + my_rank]`` of every rank; ``wait(slot, v)`` enqueues a kernel that waits (with a
    cycle budget) until all ``world`` entries of the local array reached v."""

    def __init__(self, heap: SymmetricHeap, n_slots: int = 16):
        self.heap = heap
        self.n_slots = n_slots
        # the heap was zero-filled before its handles were exchanged; zeroing again here would be an asynchronous fill that
        # can run after a fast peer's first signal has already landed and erase it
        self.flags = heap.alloc((n_slots * heap.world_size,), torch.int64)
        self._off = heap.offset_bytes(self.flags)
        self._table = heap.peer_table_at(self._off)

    def signal(self, slot: int, value: int, stream=None):
        h = self.heap
        check(kernels().tyr_signal(self._table, h.world_size, h.rank, slot * h.world_size, value,
                                   stream or cur_stream(h.device)), "signal")

    def wait(self, slot: int, value: int, err_ptr, stream=None):
        h = self.heap
        check(kernels().tyr_wait_all(ctypes.c_void_p(self.flags.data_ptr()), h.world_size,
                                     slot * h.world_size, value, err_ptr,
                                     stream or cur_stream(h.device)), "wait_all")

    def local_ptr(self):
        return ctypes.c_void_p(self.flags.data_ptr())

    def barrier_device_seq(self, slot: int, err_ptr, stream=None):
        """Signal and wait in one launch, the sequence number kept in device memory (one counter per slot): nothing in
        the launch depends on the host, so it can sit inside a CUDA graph.  A slot must not mix this with
        ``signal`` / ``wait``."""
        h = self.heap
        if getattr(self, "_seq_dev", None) is None:
            self._seq_dev = torch.zeros(self.n_slots, dtype=torch.int64, device=h.device)
        check(kernels().tyr_barrier_dev(self._table, ctypes.c_void_p(self.flags.data_ptr()), h.world_size, h.rank, slot * h.world_size,
                                        ctypes.c_void_p(self._seq_dev.data_ptr() + 8 * slot), err_ptr, stream or cur_stream(h.device)), "barrier_dev")


def wait_flags_bounded(flags: torch.Tensor, world: int, slot_base: int, value: int, err_ptr, budget_cycles: int, stream=None) -> None:
    """Enqueue the flag wait on a plain local int64 tensor with an explicit cycle budget.  When the budget runs out the
    kernel writes {2 = peer flag timeout, slot} into the device error record and returns."""
    check(kernels().tyr_wait_all_budget(ctypes.c_void_p(flags.data_ptr()), world, slot_base, value, err_ptr, budget_cycles,
                                        stream or cur_stream(flags.device)), "wait_all_budget")
