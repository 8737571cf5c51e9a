"""Expert parallelism: sigmoid/softmax-routed MoE with the experts split over the ranks of one NVLink
domain.  Dispatch and combine are pulls over peer memory (csrc/ep_fused.cu): each row crosses NVLink once,
in each direction, and the expert FFN runs on the owner with the single-GPU fused op
(``ops.moe.moe_fp4_forward`` for NVFP4 banks, ``moe_dense_forward`` for bf16 banks).

On CPU / gloo (tests) the same exchange is an ``all_to_all`` of padded row blocks.
"""
from __future__ import annotations

import ctypes
from typing import Callable, Optional

import torch
import torch.distributed as dist

from .._native import kernels
from ..distributed.symm import FlagBarrier, SymmetricHeap
from ..ops import moe as moe_ops
from ..ops._common import check, cur_stream, err_word, ptr


def _declare(lib):
    if getattr(lib, "_ep_declared", False):
        return
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.tyr_ep_pull.argtypes = [P, P, I, I, I, I, P, P, P, P, P, P, P, P, I, I, P, P]
    lib.tyr_ep_pull.restype = I
    lib.tyr_ep_combine.argtypes = [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, P, P]
    lib.tyr_ep_combine.restype = I
    lib._ep_declared = True


ExpertFn = Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor]
"""(rows [R, h], expert_ids int32 [R, 1] (local ids), ones fp32 [R, 1]) -> [R, h]"""


class ExpertParallel:
    def __init__(self, rank: int, world: int, device, num_experts: int, hidden: int, max_tokens: int, top_k: int,
                 group=None, capacity_factor: Optional[float] = None):
        if num_experts % world:
            raise ValueError(f"{num_experts} experts do not split evenly over {world} ranks")
        self.rank, self.world, self.group = rank, world, group
        self.device = torch.device(device)
        self.E, self.E_local, self.h, self.k = num_experts, num_experts // world, hidden, top_k
        self.max_pairs = max_tokens * top_k
        self.capacity = world * self.max_pairs if capacity_factor is None else int(capacity_factor * self.max_pairs)
        self.fused = self.device.type == "cuda" and world > 1
        self._seq = 0
        if not self.fused:
            return
        _declare(kernels())
        nseg = self.E_local * world
        nbytes = (self.max_pairs * hidden * 2 + self.capacity * hidden * 2 + (num_experts + 1) * 4 + nseg * 4 + 4096) * 2 + 65536
        self.heap = SymmetricHeap(nbytes, rank, world, self.device, group)
        mk = self.heap.alloc
        # double-buffered so that a rank may start the next layer while a peer still reads this one
        self._xs = [mk((self.max_pairs, hidden), torch.bfloat16) for _ in range(2)]
        self._y = [mk((self.capacity, hidden), torch.bfloat16) for _ in range(2)]
        self._offsets = [mk((num_experts + 1,), torch.int32) for _ in range(2)]
        self._dest_base = [mk((nseg,), torch.int32) for _ in range(2)]
        self.barrier = FlagBarrier(self.heap, n_slots=2)
        self._parity = 0
        i32 = lambda n: torch.empty(n, dtype=torch.int32, device=self.device)
        self._seg_rows, self._seg_src = i32(nseg), i32(nseg)
        self._exp_off, self._exp_tiles, self._total = i32(self.E_local + 1), i32(self.E_local + 1), i32(1)
        self._rows = torch.empty((self.capacity, hidden), dtype=torch.bfloat16, device=self.device)
        self._row_expert = i32(self.capacity)

    def close(self):
        if self.fused:
            self.heap.close()

    def _sync(self, slot):
        # signal + wait in one launch with the sequence number in device memory: replayable from a CUDA graph
        self.barrier.barrier_device_seq(slot, ptr(err_word(self.device)))

    def _table(self, t):
        off = self.heap.offset_bytes(t)
        return (ctypes.c_void_p * self.world)(*[p + off for p in self.heap.peer_ptrs])

    def forward(self, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, expert_fn: ExpertFn,
                add: Optional[torch.Tensor] = None, counts: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x: [T, h]; ids int32 [T, k] global expert ids; weights fp32 [T, k].  ``expert_fn`` evaluates this
        rank's experts on expert-sorted rows.  Returns ``sum_s w[t, s] * expert(x[t]) (+ add)`` as [T, h]."""
        T, h = x.shape
        k = ids.shape[1]
        if self.world == 1:
            y = expert_fn(x.repeat_interleave(k, 0), ids.reshape(-1, 1).to(torch.int32), torch.ones(T * k, 1, device=x.device))
            out = (y.float().reshape(T, k, h) * weights.float().unsqueeze(-1)).sum(1)
            return (out if add is None else out + add.float()).to(x.dtype)
        if not self.fused:
            return self._forward_collective(x, ids, weights, expert_fn, add)
        if T * k > self.max_pairs:
            raise ValueError("expert parallel: more (token, slot) pairs than the buffers were sized for")
        st = cur_stream(x.device)
        lib = kernels()
        par = self._parity
        self._parity ^= 1
        if counts is None:
            counts = moe_ops.count_experts(ids, self.E)
        ids32 = ids.to(torch.int32).contiguous()
        offsets, order, pos = moe_ops.layout(ids32, counts)
        self._offsets[par].copy_(offsets)
        xs = self._xs[par]
        check(lib.tyr_moe_gather_rows(ptr(x.contiguous()), ptr(order), ptr(xs), T * k, k, h, st), "moe_gather_rows")
        R = min(self.capacity, self.world * T * k)     # host-known upper bound of the rows this rank can receive
        self._row_expert[:R].fill_(self.E_local)       # rows the pull does not fill stay marked as padding
        self._sync(0)
        check(lib.tyr_ep_pull(self._table(self._offsets[par]), self._table(xs), self.world, self.rank, self.E_local, h,
                              ptr(self._seg_rows), ptr(self._seg_src), ptr(self._dest_base[par]), ptr(self._exp_off),
                              ptr(self._exp_tiles), ptr(self._total), ptr(self._rows), ptr(self._row_expert), self.capacity,
                              self.max_pairs, ptr(err_word(x.device)), st), "ep_pull")
        # the owner evaluates its experts on that upper bound at every batch size (no host read of the received total): rows
        # past the device-side total keep the padding id, take no slot in the expert layout, cost no tensor-core tile (the
        # grouped GEMM walks the device-side tile table) and are never read back
        rows = self._rows[:R]
        row_e = self._row_expert[:R].reshape(R, 1)
        y_local = expert_fn(rows, row_e, torch.ones(R, 1, device=x.device))
        self._y[par][:R].copy_(y_local)
        self._sync(1)
        out = torch.empty_like(x)
        check(lib.tyr_ep_combine(self._table(self._y[par]), self._table(self._dest_base[par]), ptr(ids32),
                                 ptr(weights.float().contiguous()), ptr(pos), ptr(self._offsets[par]),
                                 ptr(add.contiguous() if add is not None else None), ptr(out), T, k, h, self.E_local, self.world,
                                 self.rank, self.capacity, ptr(err_word(x.device)), st), "ep_combine")
        return out

    # -- collective fallback (gloo / unsupported shapes) ----------------------------------------------------
    def _forward_collective(self, x, ids, weights, expert_fn, add):
        T, h = x.shape
        k, W, El = ids.shape[1], self.world, self.E_local
        flat = ids.reshape(-1).long()
        owner = flat // El
        order = torch.argsort(owner * self.E + flat, stable=True)          # owner-major, expert-minor
        send_counts = torch.bincount(owner, minlength=W)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        rows = x[order // k].contiguous()
        eids = (flat[order] % El).to(torch.int32)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        recv_rows = torch.empty((sum(rc), h), dtype=x.dtype, device=x.device)
        recv_e = torch.empty(sum(rc), dtype=torch.int32, device=x.device)
        dist.all_to_all_single(recv_rows, rows, rc, sc, group=self.group)
        dist.all_to_all_single(recv_e, eids, rc, sc, group=self.group)
        if recv_rows.shape[0] > 0:
            y = expert_fn(recv_rows, recv_e.reshape(-1, 1), torch.ones(recv_rows.shape[0], 1, device=x.device)).to(x.dtype)
        else:
            y = recv_rows
        back = torch.empty_like(rows)
        dist.all_to_all_single(back, y.contiguous(), sc, rc, group=self.group)
        per_pair = torch.empty((T * k, h), dtype=torch.float32, device=x.device)
        per_pair[order] = back.float()
        out = (per_pair.reshape(T, k, h) * weights.float().unsqueeze(-1)).sum(1)
        return (out if add is None else out + add.float()).to(x.dtype)


def local_expert_fn(experts, local_ids_offset: int = 0) -> ExpertFn:
    """Expert evaluation for ``ExpertParallel.forward`` from this rank's banks: a ``PackedExperts`` (NVFP4) or a
    ``(gate_up [E_local, 2*mi, h], down [E_local, h, mi])`` pair of bf16 banks."""
    if isinstance(experts, moe_ops.PackedExperts):
        return lambda rows, eids, ones: moe_ops.moe_fp4_forward(rows, eids, ones, experts)
    gate_up, down = experts
    return lambda rows, eids, ones: moe_ops.moe_dense_forward(rows, eids, ones, gate_up, down)
