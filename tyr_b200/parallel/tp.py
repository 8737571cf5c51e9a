"""Tensor parallelism with the collectives fused into the tcgen05 GEMM (one process per GPU, one
NVLink domain, symmetric heap over CUDA IPC).

* ``gemm_reduce_scatter``: row-parallel linear.  Every rank multiplies its K-slice; the GEMM epilogue
  stores each bf16 partial tile straight into the slot buffer of the rank that owns those rows
  (plain peer stores, remote owners first so the traffic overlaps the remaining tiles); after one
  flag barrier the owner sums its ``world`` slots in fp32.
* ``allgather_gemm``: column-parallel linear over row-sharded activations.  Shards are staged in
  symmetric memory; inside the GEMM kernel two gather warps per CTA pull the peers' rows over NVLink
  (plain peer loads, each row once, in the order the row tiles are consumed) into a local landing buffer
  and publish per-tile counters, while the MMA pipeline starts on the rank's own rows and picks up each
  remote tile as soon as it has landed (bounded waits, no cluster multicast).

Without CUDA (tests on gloo) or for world size 1 the same results come from ``torch.distributed``
collectives / a plain GEMM.  The reference has no tensor parallelism; these serve the Qwen3.5 TP model.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .._native import GemmArgs, kernels
from ..distributed.symm import FlagBarrier, SymmetricHeap
from ..ops._common import check, cur_stream, err_word, ptr
from ..ops.gemm import _ACT, gemm


class TpArgs(ctypes.Structure):
    _fields_ = [("mode", ctypes.c_int), ("world", ctypes.c_int), ("rank", ctypes.c_int), ("rows_per_rank", ctypes.c_int),
                ("peers", ctypes.c_void_p * 8), ("gather_buf", ctypes.c_void_p), ("tile_ready", ctypes.c_void_p)]


def _declare(lib):
    if getattr(lib, "_tp_declared", False):
        return
    lib.tyr_gemm_bf16_tp.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.tyr_gemm_bf16_tp.restype = ctypes.c_int
    lib.tyr_slot_sum_bf16.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.tyr_slot_sum_bf16.restype = ctypes.c_int
    lib.tyr_peer_sum_bf16.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.tyr_peer_sum_bf16.restype = ctypes.c_int
    fn = getattr(lib, "tyr_peer_gather_cols_bf16", None)
    if fn is not None:
        fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
        fn.restype = ctypes.c_int
    fn = getattr(lib, "tyr_tp_allreduce_norm", None)
    if fn is not None:
        P, I = ctypes.c_void_p, ctypes.c_int
        fn.argtypes = [P, P, P, I, I, I, P, P, P, P, P, P, I, I, I, ctypes.c_float, P, P]
        fn.restype = I
    lib._tp_declared = True


class TensorParallel:
    """Buffers are sized once: ``max_rows`` total activation rows (all ranks), ``max_cols`` widest
    reduce-scatter output, ``max_k`` widest gathered input, ``gather_elems`` the largest per-rank block that
    ``all_gather_cols`` gathers through peer loads (rows x local columns, e.g. decode batch x vocabulary / world; 0: that
    call uses the transport)."""

    def __init__(self, rank: int, world: int, device, group=None, max_rows: int = 8192, max_cols: int = 8192, max_k: int = 8192,
                 gather_elems: int = 0):
        self.rank, self.world, self.group = rank, world, group
        self.device = torch.device(device)
        self.fused = self.device.type == "cuda" and world > 1
        self._seq = 0
        self._parity = 0
        if not self.fused:
            return
        if world > 8:
            raise ValueError("tensor parallel groups span at most 8 GPUs of one NVLink domain")
        _declare(kernels())
        self.max_rows, self.max_cols, self.max_k = max_rows, max_cols, max_k
        rpr = (max_rows + world - 1) // world
        slot_bytes = world * rpr * max_cols * 2
        stage_bytes = rpr * max_k * 2
        self.heap = SymmetricHeap(2 * slot_bytes + 2 * stage_bytes + 4 * gather_elems + 65536, rank, world, self.device, group)
        self._slots = [self.heap.alloc((world * rpr * max_cols,), torch.bfloat16) for _ in range(2)]
        self._stage = [self.heap.alloc((rpr * max_k,), torch.bfloat16) for _ in range(2)]
        self._gcols = [self.heap.alloc((gather_elems,), torch.bfloat16) for _ in range(2)] if gather_elems > 0 else None
        self._gparity = 0
        self.barrier = FlagBarrier(self.heap, n_slots=2)
        # landing buffer of the all-gather GEMM (peers' rows cross NVLink once) and its per-row-tile counters
        self._gather = torch.empty((world * rpr * max_k,), dtype=torch.bfloat16, device=self.device)
        self._tile_ready = torch.zeros((world * rpr + 127) // 128, dtype=torch.int32, device=self.device)

    # -- helpers ----------------------------------------------------------------------------------------
    def _sync(self, slot: int):
        self.barrier.barrier_device_seq(slot, ptr(err_word(self.device)))

    def _peers(self, t: torch.Tensor):
        off = self.heap.offset_bytes(t)
        arr = (ctypes.c_void_p * 8)()
        for r in range(self.world):
            arr[r] = self.heap.peer_ptrs[r] + off
        return arr

    def close(self):
        if self.fused:
            self.heap.close()

    # -- GEMM -> reduce-scatter ----------------------------------------------------------------------------
    def gemm_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, add: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x: [M, K_local] (all M rows, this rank's K slice); w: [N, K_local].  Returns this rank's
        ``[M / world, N]`` rows of ``sum_ranks x @ w^T`` (+ ``add``)."""
        M, N = x.shape[0], w.shape[0]
        if self.world == 1:
            y = gemm(x, w, a_layout="K", b_layout="K") if x.is_cuda else (x.float() @ w.float().T).to(x.dtype)
            return y if add is None else y + add
        if M % self.world:
            raise ValueError(f"rows ({M}) must divide evenly over {self.world} ranks")
        rpr = M // self.world
        if not self.fused or rpr % 128 or N % 8 or x.dtype != torch.bfloat16:
            y = (x.float() @ w.float().T) if not x.is_cuda else torch.matmul(x, w.T).float()
            out = torch.empty((rpr, N), dtype=torch.float32, device=x.device)
            dist.reduce_scatter_tensor(out, y.contiguous(), group=self.group)
            return (out if add is None else out + add.float()).to(x.dtype)
        if M * N > self._slots[0].numel():
            raise ValueError("gemm_reduce_scatter: product exceeds the slot buffers this group was sized for")
        slots = self._slots[self._parity]
        self._parity ^= 1
        args = GemmArgs()
        x = x.contiguous()
        args.A, args.B, args.C = x.data_ptr(), w.data_ptr(), slots.data_ptr()
        args.M, args.N, args.K, args.batch = M, N, x.shape[1], 1
        args.lda, args.ldb, args.ldc = x.stride(0), w.stride(0), N
        args.alpha, args.bn = 1.0, 0
        args.err = err_word(x.device).data_ptr()
        args.stream = cur_stream(x.device).value
        tp = TpArgs(1, self.world, self.rank, rpr, self._peers(slots), None, None)
        check(kernels().tyr_gemm_bf16_tp(ctypes.byref(args), ctypes.byref(tp)), "gemm_bf16_tp(reduce-scatter)")
        self._sync(0)
        out = torch.empty((rpr, N), dtype=torch.bfloat16, device=x.device)
        check(kernels().tyr_slot_sum_bf16(ptr(slots), self.world, rpr * N, ptr(add.contiguous() if add is not None else None),
                                          ptr(out), cur_stream(x.device)), "slot_sum_bf16")
        return out

    # -- small-M linear -> one-shot all-reduce (decode) ---------------------------------------------------------
    def linear_all_reduce(self, x: torch.Tensor, w: torch.Tensor, add: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x: [M, K_local] replicated rows with this rank's K slice; w: [N, K_local].  Every rank returns the full
        ``[M, N]`` sum (+ ``add``).  The partial product lands in this rank's symmetric buffer; after one flag barrier
        each rank sums all peers' partials with plain peer loads (one launch, no ring)."""
        M, N = x.shape[0], w.shape[0]
        if self.world == 1:
            y = torch.matmul(x, w.T)
            return y if add is None else y + add
        if not self.fused or (M * N) % 8 or x.dtype != torch.bfloat16 or M * N > self._slots[0].numel():
            y = torch.matmul(x, w.T).float()
            dist.all_reduce(y, group=self.group)
            return (y if add is None else y + add.float()).to(x.dtype)
        part = self._slots[self._parity]
        self._parity ^= 1
        torch.matmul(x, w.T, out=part[:M * N].view(M, N))
        self._sync(0)
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        check(kernels().tyr_peer_sum_bf16(self._peers(part), self.world, M * N, ptr(add.contiguous() if add is not None else None),
                                          ptr(out), cur_stream(x.device)), "peer_sum_bf16")
        return out

    def linear_all_reduce_norm(self, x: torch.Tensor, w: torch.Tensor, add: torch.Tensor, norm_w: Optional[torch.Tensor],
                               eps: float, one_plus_w: bool = True):
        """``linear_all_reduce`` followed by the next sub-layer's RMSNorm: returns ``(r, n)`` with ``r = sum_ranks x @ w^T + add``
        (the new residual stream) and ``n = rmsnorm(r) * (1 + norm_w)`` (``* norm_w`` without ``one_plus_w``; ``None`` when
        ``norm_w`` is ``None``).  On the fused path the partial product comes from the weight-streaming kernel straight into
        this rank's symmetric buffer and ONE kernel does the flag barrier, the sum over the peers' partials, the residual add
        and the norm (``tyr_tp_allreduce_norm``); otherwise it falls back to ``linear_all_reduce`` and the norm op."""
        from ..ops import decode_gemm, skinny
        from ..ops.norm import rms_norm_weighted
        M, N = x.shape[0], w.shape[0]
        fused = (self.fused and x.dtype == torch.bfloat16 and N % 8 == 0 and N <= 8192 and M * N <= self._slots[0].numel()
                 and add is not None and add.is_contiguous() and hasattr(kernels(), "tyr_tp_allreduce_norm"))
        if not fused:
            r = self.linear_all_reduce(x, w, add=add)
            return r, (None if norm_w is None else rms_norm_weighted(r, norm_w, eps, one_plus_w=one_plus_w))
        part = self._slots[self._parity]
        self._parity ^= 1
        pv = part[:M * N].view(M, N)
        if skinny.supported(x, w):
            skinny.skinny_linear(x, w, out=pv)
        elif decode_gemm.supported(x, w):
            decode_gemm.decode_linear(x, w, out=pv)
        else:
            torch.matmul(x, w.T, out=pv)
        bar = self.barrier
        if getattr(bar, "_seq_dev", None) is None:
            bar._seq_dev = torch.zeros(bar.n_slots, dtype=torch.int64, device=self.device)
        if getattr(self, "_ar_done", None) is None:
            self._ar_done = torch.zeros(1, dtype=torch.int32, device=self.device)
        nw = None
        if norm_w is not None:
            nw = norm_w if (norm_w.dtype == torch.bfloat16 and norm_w.is_contiguous()) else norm_w.to(torch.bfloat16).contiguous()
        r = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        n = torch.empty((M, N), dtype=torch.bfloat16, device=x.device) if nw is not None else None
        check(kernels().tyr_tp_allreduce_norm(self._peers(part), bar._table, ctypes.c_void_p(bar.flags.data_ptr()), self.world, self.rank,
                                              0, ctypes.c_void_p(bar._seq_dev.data_ptr()), ptr(self._ar_done), ptr(add), ptr(nw), ptr(r), ptr(n),
                                              M, N, 1 if one_plus_w else 0, eps, ptr(err_word(self.device)), cur_stream(x.device)),
              "tp_allreduce_norm")
        return r, n

    def all_gather_cols(self, y_local: torch.Tensor) -> torch.Tensor:
        """[M, N_local] per rank -> [M, N_local * world] (rank-major columns); used for vocabulary-parallel logits."""
        if self.world == 1:
            return y_local
        M, Nl = y_local.shape
        if (self.fused and self._gcols is not None and y_local.dtype == torch.bfloat16 and Nl % 8 == 0
                and M * Nl <= self._gcols[0].numel() and hasattr(kernels(), "tyr_peer_gather_cols_bf16")):
            # peer loads: the block goes into this rank's symmetric buffer (two alternate, so a rank that is already a call
            # ahead cannot overwrite what a slower peer still reads), one flag barrier, every rank pulls all blocks
            buf = self._gcols[self._gparity]
            self._gparity ^= 1
            buf[:M * Nl].view(M, Nl).copy_(y_local)
            self._sync(1)
            out = torch.empty((M, Nl * self.world), dtype=torch.bfloat16, device=y_local.device)
            check(kernels().tyr_peer_gather_cols_bf16(self._peers(buf), self.world, M, Nl, ptr(out), cur_stream(y_local.device)),
                  "peer_gather_cols_bf16")
            return out
        parts = [torch.empty_like(y_local) for _ in range(self.world)]
        dist.all_gather(parts, y_local.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)

    # -- all-gather -> GEMM ------------------------------------------------------------------------------------
    def allgather_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, act: Optional[str] = None) -> torch.Tensor:
        """x_shard: this rank's ``[M / world, K]`` rows; w: [N_local, K].  Returns ``[M, N_local]``."""
        rpr, K = x_shard.shape
        if self.world == 1:
            return gemm(x_shard, w, a_layout="K", b_layout="K", act=act) if x_shard.is_cuda else _cpu_lin(x_shard, w, act)
        if not self.fused or rpr % 128 or K % 8 or w.shape[0] % 8 or x_shard.dtype != torch.bfloat16:
            full = torch.empty((rpr * self.world, K), dtype=x_shard.dtype, device=x_shard.device)
            dist.all_gather_into_tensor(full, x_shard.contiguous(), group=self.group)
            tc = full.is_cuda and full.dtype == torch.bfloat16 and K % 8 == 0 and w.shape[0] % 8 == 0
            return gemm(full, w, a_layout="K", b_layout="K", act=act) if tc else _cpu_lin(full, w, act)
        if rpr * K > self._stage[0].numel():
            raise ValueError("allgather_gemm: shard exceeds the staging buffers this group was sized for")
        stage = self._stage[self._parity]
        self._parity ^= 1
        stage[:rpr * K].view(rpr, K).copy_(x_shard)
        self._sync(1)
        M, N = rpr * self.world, w.shape[0]
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x_shard.device)
        args = GemmArgs()
        args.A, args.B, args.C = stage.data_ptr(), w.data_ptr(), out.data_ptr()
        args.M, args.N, args.K, args.batch = M, N, K, 1
        args.lda, args.ldb, args.ldc = K, w.stride(0), N
        args.alpha, args.bn, args.act = 1.0, 0, _ACT[act]
        args.err = err_word(out.device).data_ptr()
        args.stream = cur_stream(out.device).value
        tp = TpArgs(2, self.world, self.rank, rpr, self._peers(stage), self._gather.data_ptr(), self._tile_ready.data_ptr())
        check(kernels().tyr_gemm_bf16_tp(ctypes.byref(args), ctypes.byref(tp)), "gemm_bf16_tp(all-gather)")
        return out


def _cpu_lin(x, w, act):
    if x.is_cuda and x.dtype == torch.bfloat16:      # odd widths on the GPU: the library's bf16 GEMM, not an fp32 product
        y = torch.nn.functional.linear(x, w.to(x.dtype)).float()
    else:
        y = x.float() @ w.float().T
    if act == "relu":
        y = torch.relu(y)
    elif act == "relu2":
        y = torch.relu(y).square()
    return y.to(x.dtype)
