"""Data parallelism with the optimizer step fused into the gradient collective.

``FusedDataParallel`` replaces the reference's per-tensor blocking NCCL sequence
(reduce_scatter -> ~15 elementwise kernels -> 2-3 all_gathers per parameter,
Tyr/Optim/DistAdam.lean:185-267 and Tyr/Optim/NorMuon.lean:346-425) with a handful of kernels
that read peer gradients and write peer parameters directly over NVLink
(csrc/comm_fused.cu):

* AdamW tensors (embedding, value embeddings, lm_head) are sharded flat over the ranks; one
  kernel per tensor = reduce-scatter + AdamW on the fp32 master shard + all-gather of the bf16
  working copy.  Optimizer state exists only for the owned shard (ZeRO-1/2 style), where the
  reference keeps all three state tensors replicated by gathering them every step.
* Muon matrices keep the reference's whole-matrix block-cyclic ownership (matrix ``b`` of a
  stacked group belongs to rank ``b % world``): one kernel pulls + averages the owned gradients
  and applies momentum/Nesterov, the owner runs batched Newton-Schulz on its matrices only, and
  one kernel applies the update and pushes bf16 parameters to every rank.  Momentum stays on the
  owner (the reference all-gathers it).
* Tiny tensors (scalars, smear gate) are summed from peers and updated redundantly on every
  rank, which is deterministic because every rank adds the same values in the same order.
* Ordering between ranks uses a monotonic flag barrier in symmetric memory; every device-side
  wait has a cycle budget and reports through the error record instead of hanging.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional

import torch

from .._native import kernels
from ..distributed.symm import FlagBarrier, SymmetricHeap
from ..ops import optim_kernels as ok
from ..ops import polar
from ..ops._common import check, cur_stream, err_word

SLOT_GRADS_READY = 0
SLOT_PARAMS_READY = 1


def _numel(shape):
    n = 1
    for s in shape:
        n *= int(s)
    return n


class FusedDataParallel:
    def __init__(self, rank: int, world_size: int, device, group=None, comm_ctas: int = 0):
        self.rank, self.world_size = rank, world_size
        self.device = torch.device(device)
        self.group = group
        self.comm_ctas = comm_ctas
        self.heap: Optional[SymmetricHeap] = None
        self.barrier: Optional[FlagBarrier] = None
        self.step_no = 0
        # TYR_DP_TIMING=1: CUDA events around every fused kernel of the step (read with `timings()`); adds a few
        # event records per step and no synchronisation
        import os
        self._timing = os.environ.get("TYR_DP_TIMING", "0") == "1"
        self._events: List[tuple] = []

    # -- allocation hook used by the parameter store -----------------------------------------------
    def plan_heap(self, shapes_dtypes):
        total = 4096
        for shape, dtype in shapes_dtypes:
            nb = _numel(shape) * torch.empty((), dtype=dtype).element_size()
            total += (nb + 255) // 256 * 256 + 256
        total += 64 * 1024
        self.heap = SymmetricHeap(total, self.rank, self.world_size, self.device, self.group)
        self.barrier = FlagBarrier(self.heap, n_slots=8)

    def alloc(self, shape, dtype):
        return self.heap.alloc(shape, dtype)

    # -- wiring ----------------------------------------------------------------------------------
    def attach(self, trainer):
        """Builds the sharded optimizer state for ``trainer`` (whose ``work``/``grad`` tensors were
        allocated from this object's heap)."""
        p = trainer.params
        W, r = self.world_size, self.rank
        self.err = err_word(self.device)
        self.adam: Dict[str, dict] = {}
        for name in ("embed", "value_embeds", "lm_head"):
            n = p.master[name].numel()
            if n % (4 * W) != 0:
                raise ValueError(f"{name}: {n} elements are not divisible by 4*world_size")
            shard = n // W
            lo = r * shard
            st = {
                "shard": shard, "lo": lo,
                "master": p.master[name].reshape(-1)[lo:lo + shard].clone(),
                "m": torch.zeros(shard, dtype=torch.float32, device=self.device),
                "v": torch.zeros(shard, dtype=torch.float32, device=self.device),
                "grad_off": self.heap.offset_bytes(p.grad[name]) // 4 + lo,
                "work_off": self.heap.offset_bytes(p.work[name]) // 2 + lo,
                "step": 0,
            }
            self.adam[name] = st
        self.muon: Dict[str, dict] = {}
        for name in ("attn_w", "mlp_w"):
            mast = p.master[name].reshape(-1, p.master[name].shape[-2], p.master[name].shape[-1])
            B, R, C = mast.shape
            own = [b for b in range(B) if b % W == r]
            per = R * C
            g_base = self.heap.offset_bytes(p.grad[name]) // 4
            w_base = self.heap.offset_bytes(p.work[name]) // 2
            st = {
                "own": own, "per": per, "shape": (R, C),
                "master": mast[own].clone() if own else mast[:0].clone(),
                "mom": torch.zeros((len(own), R, C), dtype=torch.float32, device=self.device),
                "u": torch.zeros((len(own), R, C), dtype=torch.bfloat16, device=self.device),
                "sumsq": torch.zeros(max(len(own), 1), dtype=torch.float32, device=self.device),
                "grad_offs": torch.tensor([g_base + b * per for b in own], dtype=torch.int64, device=self.device),
                "work_offs": torch.tensor([w_base + b * per for b in own], dtype=torch.int64, device=self.device),
            }
            self.muon[name] = st
        # tiny replicated tensors: their gradients are staged into the heap for the peer sum
        self.small_stage = {
            "scalars": self.heap.alloc(p.master["scalars"].shape, torch.float32),
            "smear_gate": self.heap.alloc(p.master["smear_gate"].shape, torch.float32),
        }
        self.small_sum = {k: torch.zeros_like(v) for k, v in self.small_stage.items()}
        self._grad_table = self.heap.peer_table()
        self._work_table = self.heap.peer_table()
        self.trainer = trainer

    def _timed(self, label: str, nbytes_in: int, nbytes_out: int):
        """Context manager recording an event pair around a kernel; bytes are what crosses NVLink into / out of this GPU."""
        dp = self

        class _T:
            def __enter__(self_inner):
                if dp._timing:
                    self_inner.e0 = torch.cuda.Event(enable_timing=True)
                    self_inner.e1 = torch.cuda.Event(enable_timing=True)
                    self_inner.e0.record()
                return self_inner

            def __exit__(self_inner, *exc):
                if dp._timing:
                    self_inner.e1.record()
                    dp._events.append((label, nbytes_in, nbytes_out, self_inner.e0, self_inner.e1))
                return False
        return _T()

    def timings(self, reset: bool = True):
        """[(label, ms, NVLink bytes in, NVLink bytes out)] of the kernels recorded since the last call (synchronises)."""
        torch.cuda.synchronize(self.device)
        out = [(lab, e0.elapsed_time(e1), bi, bo) for lab, bi, bo, e0, e1 in self._events]
        if reset:
            self._events = []
        return out

    # -- the step ----------------------------------------------------------------------------------
    def optimizer_step(self, trainer, lr_embed: float, lr_unembed: float, lr_matrix: float, mu: float):
        lib = kernels()
        hp = trainer.hp
        p = trainer.params
        W = self.world_size
        self.step_no += 1
        step = self.step_no
        stream = cur_stream(self.device)
        errp = ctypes.c_void_p(self.err.data_ptr())
        # stage the tiny gradients where peers can read them
        for k, leaf in (("scalars", p.work["scalars"]), ("smear_gate", p.work["smear_gate"])):
            if leaf.grad is not None:
                self.small_stage[k].copy_(leaf.grad)
            else:
                self.small_stage[k].zero_()
        # my gradients are complete (stream order) -> tell everyone
        self.barrier.signal(SLOT_GRADS_READY, step, stream)
        flags = self.barrier.local_ptr()
        wslot = SLOT_GRADS_READY * W

        lrs = {"embed": lr_embed, "value_embeds": lr_embed, "lm_head": lr_unembed}
        for name, st in self.adam.items():
            st["step"] += 1
            bc1 = 1.0 - hp.adam_beta1 ** st["step"]
            bc2 = 1.0 - hp.adam_beta2 ** st["step"]
            rem = (W - 1) * st["shard"]
            with self._timed(f"adam_shard.{name}", rem * 4, rem * 2):
              check(lib.tyr_dp_adam_shard(self._grad_table, self._work_table, W, st["grad_off"], st["work_off"],
                                        ctypes.c_void_p(st["master"].data_ptr()),
                                        ctypes.c_void_p(st["m"].data_ptr()), ctypes.c_void_p(st["v"].data_ptr()),
                                        st["shard"], lrs[name], hp.adam_beta1, hp.adam_beta2, 1e-10,
                                        hp.adam_weight_decay, bc1, bc2, 1.0, flags, wslot, step, errp,
                                        self.comm_ctas, stream), "dp_adam_shard")

        for name, st in self.muon.items():
            nb = len(st["own"])
            if nb == 0:
                continue
            st["sumsq"].zero_()
            with self._timed(f"muon_gather.{name}", (W - 1) * nb * st["per"] * 4, 0):
              check(lib.tyr_dp_muon_gather(self._grad_table, W, ctypes.c_void_p(st["grad_offs"].data_ptr()),
                                         ctypes.c_void_p(st["mom"].data_ptr()), ctypes.c_void_p(st["u"].data_ptr()),
                                         ctypes.c_void_p(st["sumsq"].data_ptr()), st["per"], nb, mu, 1.0,
                                         flags, wslot, step, errp, self.comm_ctas, stream), "dp_muon_gather")
            with self._timed(f"newton_schulz.{name}", 0, 0):
                ok.scale_by_inv_norm_(st["u"], st["sumsq"], 1e-7)
                o = polar.newton_schulz_(st["u"], 5).contiguous()
            R, C = st["shape"]
            eff_lr = lr_matrix * (max(1.0, R / C) ** 0.5)
            with self._timed(f"muon_apply_push.{name}", 0, (W - 1) * nb * st["per"] * 2):
              check(lib.tyr_dp_muon_apply_push(self._work_table, W, ctypes.c_void_p(st["work_offs"].data_ptr()),
                                             ctypes.c_void_p(st["master"].data_ptr()),
                                             ctypes.c_void_p(o.data_ptr()), st["per"], nb, eff_lr, 0.0,
                                             self.comm_ctas, stream), "dp_muon_apply_push")

        # tiny tensors: peer sum (waits were already satisfied by the kernels above on this stream)
        for k in ("scalars", "smear_gate"):
            off = self.heap.offset_bytes(self.small_stage[k]) // 4
            check(lib.tyr_peer_sum(self._grad_table, W, off, ctypes.c_void_p(self.small_sum[k].data_ptr()),
                                   self.small_sum[k].numel(), 1.0 / W, stream), "peer_sum")
        adam = dict(beta1=hp.adam_beta1, beta2=hp.adam_beta2, eps=1e-10, weight_decay=hp.adam_weight_decay)
        g = trainer.adam_groups["scalars"]
        g.grad_getter = lambda: self.small_sum["scalars"]
        g.step(lr_unembed, **adam)
        p.work["smear_gate"].grad = self.small_sum["smear_gate"].clone()
        trainer._smear_gate_step(lr_matrix, mu)

        # everyone has finished reading my gradients and writing my parameters once all ranks
        # signalled; the wait is enqueued on the compute stream ahead of the next forward
        self.barrier.signal(SLOT_PARAMS_READY, step, stream)
        self.barrier.wait(SLOT_PARAMS_READY, step, errp, stream)

    # -- utilities -------------------------------------------------------------------------------
    def gather_master(self, trainer):
        """Rebuild full fp32 master tensors on every rank (checkpointing): owners contribute their
        shards through an NCCL all-gather; this is off the hot path."""
        import torch.distributed as dist
        p = trainer.params
        for name, st in self.adam.items():
            full = p.master[name].reshape(-1)
            parts = [torch.empty_like(st["master"]) for _ in range(self.world_size)]
            dist.all_gather(parts, st["master"], group=self.group)
            full.copy_(torch.cat(parts))
        for name, st in self.muon.items():
            mast = p.master[name].reshape(-1, *st["shape"])
            B = mast.shape[0]
            for b in range(B):
                owner = b % self.world_size
                buf = st["master"][st["own"].index(b)].clone() if owner == self.rank else torch.empty_like(mast[b])
                dist.broadcast(buf, src=owner, group=self.group)
                mast[b].copy_(buf)

    def scatter_master(self, trainer):
        """Inverse of ``gather_master``: refresh the owned fp32 shards from the (restored) full master tensors.
        The bf16 working copies were already refreshed on every rank by ``load_named``."""
        p = trainer.params
        for name, st in self.adam.items():
            full = p.master[name].reshape(-1)
            n = st["master"].numel()
            st["master"].copy_(full[self.rank * n:(self.rank + 1) * n])
        for name, st in self.muon.items():
            mast = p.master[name].reshape(-1, *st["shape"])
            if st["own"]:
                st["master"].copy_(mast[st["own"]])

    def state_dict(self):
        """This rank's optimizer shards (Adam moments of its slice, Muon momentum of its matrices)."""
        out = {}
        for name, st in self.adam.items():
            out[f"dp.adam.{name}.m"], out[f"dp.adam.{name}.v"] = st["m"], st["v"]
            out[f"dp.adam.{name}.step"] = torch.tensor([st["step"]], dtype=torch.int64)
        for name, st in self.muon.items():
            out[f"dp.muon.{name}.mom"] = st["mom"]
        out["dp.step_no"] = torch.tensor([self.step_no], dtype=torch.int64)
        return out

    def load_state_dict(self, sd):
        for name, st in self.adam.items():
            st["m"].copy_(sd[f"dp.adam.{name}.m"].reshape(st["m"].shape))
            st["v"].copy_(sd[f"dp.adam.{name}.v"].reshape(st["v"].shape))
            st["step"] = int(sd[f"dp.adam.{name}.step"][0])
        for name, st in self.muon.items():
            if st["mom"].numel():
                st["mom"].copy_(sd[f"dp.muon.{name}.mom"].reshape(st["mom"].shape))

    def close(self):
        if self.heap is not None:
            self.heap.close()
            self.heap = None
