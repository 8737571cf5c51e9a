"""NanoChat training engine (the reference's ``ModdedTrain``:
Examples/NanoChat/ModdedTrain.lean).

One ``NanoChatTrainer.step`` = zero grads -> forward/backward over the micro-batches -> optimizer
step, with the same hyper-parameters, learning-rate / momentum schedules, parameter grouping
(AdamW for embeddings, value embeddings, lm_head and scalars; Muon for the matrices and the
smear gate) and update math as ``trainStepDistributedAccum`` (:897-1160).

Differences that are deliberate and B200-specific:

* activations and working weights are bf16, master weights / moments / gradient accumulators fp32;
* the Muon update of all matrices of one shape class runs as ONE batched launch sequence
  (momentum + Nesterov + norm kernel, 15 batched tcgen05 GEMMs, apply kernel) instead of a
  per-parameter host loop with a ``maxAll.item`` sync per matrix (NorMuon.lean:244-245);
* no host synchronisation inside a step (loss stays on the device until asked for);
* multi-GPU: gradients are reduced and the sharded update applied by the fused kernels in
  :mod:`tyr_b200.parallel.dp` over NVLink peer memory instead of one blocking NCCL collective
  per tensor after backward.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, asdict
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..models import nanochat as nc
from ..ops import optim_kernels as ok
from ..ops import polar

DEFAULT_CE_CHUNK_ROWS = 8192


@dataclass
class Hyperparameters:
    """Mirrors ``Hyperparameters`` (ModdedTrain.lean:39-76)."""
    num_iterations: int = 2050
    extension_iterations: int = 0
    device_batch_size: int = 32
    total_batch_size_tokens: int = 524288
    embedding_lr: float = 0.3
    unembedding_lr: float = 0.004
    matrix_lr: float = 0.02
    adam_beta1: float = 0.8
    adam_beta2: float = 0.95
    adam_weight_decay: float = 0.0
    warmup_frac: float = 0.0
    cooldown_frac: float = 0.4
    final_lr_frac: float = 0.0
    block_size: int = 128
    max_seq_len: int = 2048
    val_interval: int = 50
    log_interval: int = 10
    checkpoint_interval: int = 100

    def to_json(self) -> dict:
        return asdict(self)

    @staticmethod
    def from_json(j: dict) -> "Hyperparameters":
        return Hyperparameters(**{k: v for k, v in j.items() if k in Hyperparameters.__dataclass_fields__})


def get_batch_size(step: int) -> int:
    return 8 if step < 200 else (16 if step < 1000 else 24)


def get_window_sizes(step: int, block_size: int = 128) -> Tuple[int, int]:
    return (3, 3) if step < 200 else ((3, 7) if step < 1000 else (3, 11))


def get_learning_rate(step: int, hp: Hyperparameters, base_lr: float = 0.023) -> float:
    """Warmup / plateau / linear warmdown (ModdedTrain.lean:121-133)."""
    total = max(1, hp.num_iterations + hp.extension_iterations)
    warmup = int(hp.warmup_frac * total)
    warmdown = int(hp.cooldown_frac * total)
    warmdown_start = total - warmdown
    if warmup > 0 and step < warmup:
        return base_lr * (step + 1.0) / warmup
    if warmdown == 0 or step <= warmdown_start:
        return base_lr
    progress = (total - step) / warmdown
    return base_lr * (progress + (1.0 - progress) * hp.final_lr_frac)


def batch_lr_scale(hp: Hyperparameters, reference_batch: float = 524288.0) -> float:
    return 1.0 if hp.total_batch_size_tokens == 0 else math.sqrt(hp.total_batch_size_tokens / reference_batch)


def d_model_lr_scale(cfg: nc.Config) -> float:
    return (cfg.model_dim / 768.0) ** -0.5


def effective_grad_accum_steps(hp: Hyperparameters, world_size: int) -> int:
    world = max(1, world_size)
    per_micro = hp.device_batch_size * hp.max_seq_len * world
    if per_micro == 0:
        return 1
    target = max(per_micro, hp.total_batch_size_tokens)
    return max(1, target // per_micro)


def validate_grad_accum_config(hp: Hyperparameters, world_size: int):
    """total_batch_size must be divisible by per-step micro-batch tokens (ModdedTrain.lean:159-165)."""
    world = max(1, world_size)
    per_micro = hp.device_batch_size * hp.max_seq_len * world
    if per_micro == 0:
        raise ValueError("device batch size, sequence length and world size must be positive")
    if hp.total_batch_size_tokens % per_micro != 0:
        raise ValueError(
            f"total_batch_size_tokens={hp.total_batch_size_tokens} is not divisible by "
            f"device_batch_size*max_seq_len*world_size={per_micro}")


def get_muon_momentum(step: int, base: float = 0.95, warmup_steps: int = 300) -> float:
    """0.85 -> base over 300 steps, then constant (NorMuon.lean:513-523)."""
    if step < warmup_steps:
        return 0.85 + (step / warmup_steps) * (base - 0.85)
    return base


def aspect_ratio_scale(shape: Sequence[int]) -> float:
    if len(shape) >= 2 and shape[-2] > shape[-1]:
        return math.sqrt(shape[-2] / shape[-1])
    return 1.0


@dataclass
class StepResult:
    loss: torch.Tensor          # device scalar (mean over micro-batches)
    tokens_processed: int
    step: int


class MuonGroup:
    """All matrices of one shape class, stacked [B, R, C]; one batched Muon update."""

    def __init__(self, master: torch.Tensor, work: torch.Tensor, grad: torch.Tensor):
        self.master = master.reshape(-1, master.shape[-2], master.shape[-1])
        self.work = work.reshape(-1, work.shape[-2], work.shape[-1])
        self.grad = grad.reshape(-1, grad.shape[-2], grad.shape[-1])
        B = self.master.shape[0]
        self.momentum = torch.zeros_like(self.master)
        self.u = torch.zeros(self.master.shape, dtype=torch.bfloat16, device=master.device)
        self.sumsq = torch.zeros(B, dtype=torch.float32, device=master.device)

    def step(self, lr: float, momentum: float, weight_decay: float, num_iters: int, grad_scale: float = 1.0):
        if self.master.shape[0] == 0:
            return
        self.sumsq.zero_()
        ok.muon_momentum_(self.grad, self.momentum, self.u, self.sumsq, momentum, grad_scale)
        ok.scale_by_inv_norm_(self.u, self.sumsq, 1e-7)
        o = polar.newton_schulz_(self.u, num_iters)
        eff_lr = lr * aspect_ratio_scale(self.master.shape)
        ok.muon_apply_(self.master, o.contiguous(), eff_lr, weight_decay,
                       self.work if self.work.dtype == torch.bfloat16 else None)
        if self.work.dtype != torch.bfloat16:
            self.work.copy_(self.master)


class AdamGroup:
    def __init__(self, master: torch.Tensor, work: Optional[torch.Tensor], grad_getter):
        self.master = master
        self.work = work
        self.grad_getter = grad_getter
        self.exp_avg = torch.zeros_like(master)
        self.exp_avg_sq = torch.zeros_like(master)
        self.step_count = 0

    def step(self, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float,
             grad_scale: float = 1.0):
        g = self.grad_getter()
        if g is None:
            return
        self.step_count += 1
        work_bf16 = self.work if (self.work is not None and self.work.dtype == torch.bfloat16
                                  and self.work.data_ptr() != self.master.data_ptr()) else None
        ok.adamw_step_(self.master, g.contiguous(), self.exp_avg, self.exp_avg_sq, lr=lr, beta1=beta1,
                       beta2=beta2, eps=eps, weight_decay=weight_decay, step=self.step_count,
                       p_bf16=work_bf16, grad_scale=grad_scale)
        if self.work is not None and work_bf16 is None and self.work.data_ptr() != self.master.data_ptr():
            with torch.no_grad():
                self.work.copy_(self.master.to(self.work.dtype))


class NanoChatTrainer:
    """Owns parameters, optimizer state and the step function."""

    def __init__(self, cfg: nc.Config, hp: Optional[Hyperparameters] = None, device="cpu",
                 compute_dtype=torch.bfloat16, seed: Optional[int] = 0, world_size: int = 1,
                 rank: int = 0, dp=None, ce_chunk_rows: Optional[int] = None):
        self.cfg = cfg
        self.hp = hp or Hyperparameters()
        self.device = torch.device(device)
        self.world_size, self.rank = world_size, rank
        alloc = None
        if dp is not None and world_size > 1:
            plan = nc.ModdedGPTParams.storage_plan(cfg, compute_dtype)
            plan += [((cfg.n_layer * 4 + 8,), torch.float32), ((1, 12), torch.float32)]
            dp.plan_heap(plan)
            alloc = dp.alloc
        self.params = nc.ModdedGPTParams(cfg, device=device, compute_dtype=compute_dtype, seed=seed, alloc=alloc)
        self.step_index = 0
        # rows of logits alive at once in the fused lm_head + loss (bf16 [rows, vocab]); TYR_CE_CHUNK_ROWS overrides the default
        self.ce_chunk_rows = ce_chunk_rows if ce_chunk_rows is not None else int(os.environ.get("TYR_CE_CHUNK_ROWS", DEFAULT_CE_CHUNK_ROWS))
        self.dp = dp
        p = self.params
        sharded = dp is not None and world_size > 1
        self.muon_groups: Dict[str, MuonGroup] = {} if sharded else {
            "attn_w": MuonGroup(p.master["attn_w"], p.work["attn_w"], p.grad["attn_w"]),
            "mlp_w": MuonGroup(p.master["mlp_w"], p.work["mlp_w"], p.grad["mlp_w"]),
        }
        self.smear_momentum = torch.zeros_like(p.master["smear_gate"])
        self.adam_groups: Dict[str, AdamGroup] = {
            "scalars": AdamGroup(p.master["scalars"], p.work["scalars"], lambda: p.work["scalars"].grad),
        }
        if not sharded:
            self.adam_groups.update({
                "embed": AdamGroup(p.master["embed"], p.work["embed"], lambda: p.grad["embed"]),
                "value_embeds": AdamGroup(p.master["value_embeds"], p.work["value_embeds"],
                                          lambda: p.grad["value_embeds"]),
                "lm_head": AdamGroup(p.master["lm_head"], p.work["lm_head"], lambda: p.grad["lm_head"]),
            })
        if sharded:
            dp.attach(self)
        # Forward + backward of a fixed-shape single micro-batch is replayed as ONE CUDA graph after two eager steps
        # (about a thousand launches per step otherwise, and the host cannot keep the GPU fed through the short ones).
        # The optimizer step stays outside the graph: its learning rates, momentum and bias corrections change per step.
        self._graph_enabled = self.device.type == "cuda" and os.environ.get("TYR_STEP_GRAPH", "1") != "0"
        self._graph = None
        self._graph_key = None
        self._graph_eager_steps = 0

    # ------------------------------------------------------------------------------------------
    def learning_rates(self, step: int):
        hp, cfg = self.hp, self.cfg
        bs, ds = batch_lr_scale(hp), d_model_lr_scale(cfg)
        return (get_learning_rate(step, hp, hp.embedding_lr * bs * ds),
                get_learning_rate(step, hp, hp.unembedding_lr * bs * ds),
                get_learning_rate(step, hp, hp.matrix_lr * bs))

    def _forward_backward_eager(self, micro_batches) -> torch.Tensor:
        self.params.zero_grads()
        n = len(micro_batches)
        total = None
        for inp, tgt in micro_batches:
            loss = nc.loss_fused(self.params, inp, tgt, loss_scale=1.0 / n, ce_chunk_rows=self.ce_chunk_rows)
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        return total

    def _capture_step_graph(self, inp: torch.Tensor, tgt: torch.Tensor) -> bool:
        """Record zero-grads + forward + backward for this input shape.  Returns False (and stays eager for good) when the
        capture fails, e.g. because an operator on the path needs the host."""
        self._static_inp, self._static_tgt = inp.clone(), tgt.clone()
        graph = torch.cuda.CUDAGraph()
        try:
            torch.cuda.synchronize(self.device)
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                self.params.zero_grads()
                loss = nc.loss_fused(self.params, self._static_inp, self._static_tgt, loss_scale=1.0,
                                     ce_chunk_rows=self.ce_chunk_rows)
                loss.backward()
                self._static_loss = loss.detach()
        except Exception as e:       # leave no half-recorded state behind
            self._graph_enabled = False
            self._graph = None
            torch.cuda.synchronize(self.device)
            import warnings
            warnings.warn(f"NanoChat step graph capture failed, staying eager: {type(e).__name__}: {e}")
            return False
        self._graph = graph
        return True

    def forward_backward(self, micro_batches: Sequence[Tuple[torch.Tensor, torch.Tensor]]) -> torch.Tensor:
        if not (self._graph_enabled and len(micro_batches) == 1 and micro_batches[0][0].is_cuda):
            return self._forward_backward_eager(micro_batches)
        inp, tgt = micro_batches[0]
        key = (tuple(inp.shape), inp.dtype, tuple(tgt.shape), tgt.dtype)
        if self._graph is not None and key == self._graph_key:
            self._static_inp.copy_(inp)
            self._static_tgt.copy_(tgt)
            self._graph.replay()
            from ..ops import _common as opc
            opc.LAUNCH_COUNT[0] += self._graph_launches
            return self._static_loss
        if key != self._graph_key:
            self._graph_key, self._graph_eager_steps, self._graph = key, 0, None
        if self._graph_eager_steps < 2:          # warm-up: lazily built buffers, module loading, autograd threads
            self._graph_eager_steps += 1
            return self._forward_backward_eager(micro_batches)
        from ..ops import _common as opc
        before = opc.LAUNCH_COUNT[0]
        if not self._capture_step_graph(inp, tgt):
            return self._forward_backward_eager(micro_batches)
        self._graph_launches = opc.LAUNCH_COUNT[0] - before
        self._graph.replay()
        opc.LAUNCH_COUNT[0] += self._graph_launches
        return self._static_loss

    def _smear_gate_step(self, lr: float, momentum: float):
        """Muon on the [1, 12] smear gate (tiny: plain torch ops; same math as the batched path)."""
        p = self.params
        g = p.work["smear_gate"].grad
        if g is None:
            return
        g = g.detach().float()
        self.smear_momentum.mul_(momentum).add_(g, alpha=1 - momentum)
        u = (1 - momentum) * g + momentum * self.smear_momentum
        o = polar.muon_orthogonalize(u, 5).float()
        eff_lr = lr * aspect_ratio_scale(u.shape)
        with torch.no_grad():
            p.master["smear_gate"].sub_((o * eff_lr).to(torch.bfloat16).float())
            p.work["smear_gate"].copy_(p.master["smear_gate"])

    def optimizer_step(self):
        hp = self.hp
        step = self.step_index
        lr_embed, lr_unembed, lr_matrix = self.learning_rates(step)
        mu = get_muon_momentum(step)
        if self.dp is not None and self.dp.world_size > 1:
            self.dp.optimizer_step(self, lr_embed, lr_unembed, lr_matrix, mu)
        else:
            adam = dict(beta1=hp.adam_beta1, beta2=hp.adam_beta2, eps=1e-10, weight_decay=hp.adam_weight_decay)
            self.adam_groups["embed"].step(lr_embed, **adam)
            self.adam_groups["value_embeds"].step(lr_embed, **adam)
            self.adam_groups["lm_head"].step(lr_unembed, **adam)
            self.adam_groups["scalars"].step(lr_unembed, **adam)
            self._smear_gate_step(lr_matrix, mu)
            for g in self.muon_groups.values():
                g.step(lr_matrix, mu, 0.0, 5)
        self.step_index += 1

    def step(self, micro_batches: Sequence[Tuple[torch.Tensor, torch.Tensor]]) -> StepResult:
        loss = self.forward_backward(micro_batches)
        self.optimizer_step()
        tokens = sum(int(i.numel()) for i, _ in micro_batches)
        return StepResult(loss=loss, tokens_processed=tokens, step=self.step_index)

    # -- end-to-end entry: pinned host tokens in, python float loss out ---------------------------
    def train_step_from_host(self, tokens_host: torch.Tensor) -> float:
        """``tokens_host``: pinned int64 [B, T+1] on the host.  Copies it to the device, runs one
        full step and returns the loss as a Python float (device -> host read)."""
        tok = tokens_host.to(self.device, non_blocking=True)
        inp, tgt = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
        res = self.step([(inp, tgt)])
        return float(res.loss.item())

    # -- state dict (optimizer layout sidecar of ModdedTrain.lean:420-836) --------------------------
    def optimizer_state_dict(self) -> Dict[str, torch.Tensor]:
        out = {}
        for k, g in self.adam_groups.items():
            out[f"adam.{k}.exp_avg"] = g.exp_avg
            out[f"adam.{k}.exp_avg_sq"] = g.exp_avg_sq
            out[f"adam.{k}.step"] = torch.tensor([g.step_count], dtype=torch.int64)
        for k, g in self.muon_groups.items():
            out[f"muon.{k}.momentum"] = g.momentum
        out["muon.smear_gate.momentum"] = self.smear_momentum
        if self.dp is not None and self.world_size > 1:
            out.update(self.dp.state_dict())
        return out

    def load_optimizer_state_dict(self, sd: Dict[str, torch.Tensor]):
        for k, g in self.adam_groups.items():
            g.exp_avg.copy_(sd[f"adam.{k}.exp_avg"])
            g.exp_avg_sq.copy_(sd[f"adam.{k}.exp_avg_sq"])
            g.step_count = int(sd[f"adam.{k}.step"][0])
        for k, g in self.muon_groups.items():
            g.momentum.copy_(sd[f"muon.{k}.momentum"].reshape(g.momentum.shape))
        self.smear_momentum.copy_(sd["muon.smear_gate.momentum"])
        if self.dp is not None and self.world_size > 1:
            self.dp.load_state_dict(sd)
