"""A plain-PyTorch restatement of the reference's NanoChat training step, used only as a comparison arm of
``bench.py --impl restated`` when the reference itself (a Lean 4 program) cannot be installed.

It restates what the reference computes with the libraries the reference calls on a CUDA box: libtorch ops
(cuBLAS GEMMs, SDPA, elementwise kernels) for the model (Examples/NanoChat/ModdedGPT.lean:552-650), per-parameter
NCCL all-reduce of gradients, Muon by five Newton-Schulz ``torch.matmul`` iterations per matrix
(cc/src/tyr_polar.cpp:267-317) and per-tensor AdamW.  None of this repository's kernels are on that path.
bf16 autocast is used for the matmuls (the reference trains in fp32; this is the generous reading).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F

from tyr_b200.models import nanochat as nc
from tyr_b200.train import nanochat_engine as eng


@dataclass
class _Res:
    loss: torch.Tensor
    tokens_processed: int
    step: int


def _rms(x):
    return x * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6).to(x.dtype)


def _rot(x, cos, sin):
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    c, s = cos[None, :, None, :].to(x.dtype), sin[None, :, None, :].to(x.dtype)
    return torch.cat([x1 * c + x2 * s, -x1 * s + x2 * c], -1)


class RestatedTrainer:
    def __init__(self, cfg: nc.Config, hp: eng.Hyperparameters, device="cuda", world_size: int = 1, rank: int = 0, seed: int = 1234):
        self.cfg, self.hp, self.device, self.world_size, self.rank = cfg, hp, torch.device(device), world_size, rank
        base = nc.ModdedGPTParams(cfg, device="cpu", compute_dtype=torch.float32, seed=seed)
        self.p: Dict[str, torch.Tensor] = {k: v.detach().clone().to(self.device).requires_grad_(True)
                                           for k, v in base.named_parameters("master").items()}
        self.cos, self.sin = (t.to(self.device) for t in base.rotary()) if hasattr(base, "rotary") else self._rope()
        self.step_index = 0
        self.adam_state = {k: (torch.zeros_like(v), torch.zeros_like(v)) for k, v in self.p.items() if not self._is_matrix(k)}
        self.muon_state = {k: torch.zeros_like(v) for k, v in self.p.items() if self._is_matrix(k)}

    def _rope(self):
        from tyr_b200.ops import rope
        return rope.rotary_freqs(self.cfg.max_seq_len, self.cfg.head_dim, self.cfg.rope_base, self.device)

    @staticmethod
    def _is_matrix(name: str) -> bool:
        return name.startswith("blocks.")

    def forward_loss(self, ids, targets):
        p, cfg = self.p, self.cfg
        B, T = ids.shape
        H, D, L = cfg.n_head, cfg.head_dim, cfg.n_layer
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=self.device.type == "cuda"):
            tok = F.embedding(ids, p["embed"])
            gate = torch.sigmoid(F.linear(tok[..., :12], p["smearGate.weight"]))
            x0 = _rms(tok + tok * gate)
            ves = [F.embedding(ids, p[f"valueEmbeds.{i}"]) for i in range(cfg.num_value_embeds)]
            sc = torch.sigmoid(p["scalars.values"].float())
            vmix, smix, fscale = sc[4 * L], sc[4 * L + 1], sc[4 * L + 2]
            x, skip = x0, None
            for i in range(L):
                lx, l0, la, lm = sc[4 * i], sc[4 * i + 1], sc[4 * i + 2], sc[4 * i + 3]
                x_in = x * lx + x0 * l0
                if i == nc.SKIP_SOURCE_LAYER:
                    skip = x_in
                if f"blocks.{i}.attn.wQ" in p:
                    xn = _rms(x_in)
                    q, k, v = (F.linear(xn, p[f"blocks.{i}.attn.{n}"]) for n in ("wQ", "wK", "wV"))
                    vi = nc.layer_value_embed_index(cfg, i)
                    if vi is not None:
                        v = v * (1 - vmix) + ves[vi] * vmix
                    q = _rms(_rot(q.reshape(B, T, H, D), self.cos[:T], self.sin[:T])).transpose(1, 2)
                    k = _rms(_rot(k.reshape(B, T, H, D), self.cos[:T], self.sin[:T])).transpose(1, 2)
                    v = v.reshape(B, T, H, D).transpose(1, 2)
                    w = nc.get_window_size_for_layer(cfg.window_pattern, i, L, T)
                    if w is None:
                        o = F.scaled_dot_product_attention(q, k, v.to(q.dtype), is_causal=True)
                    else:
                        idx = torch.arange(T, device=ids.device)
                        m = (idx[None, :] <= idx[:, None]) & (idx[None, :] > idx[:, None] - w)
                        o = F.scaled_dot_product_attention(q, k, v.to(q.dtype), attn_mask=m)
                    x1 = x_in + F.linear(o.transpose(1, 2).reshape(B, T, H * D), p[f"blocks.{i}.attn.wO"]) * la
                    h = torch.relu(F.linear(_rms(x1), p[f"blocks.{i}.mlp.cFc"]))
                    x = x1 + ((h * h) @ p[f"blocks.{i}.mlp.cProj"].to(h.dtype)) * lm
                else:
                    x = x_in + skip * smix if skip is not None else x_in
                    h = torch.relu(F.linear(_rms(x), p[f"blocks.{i}.mlp.cFc"]))
                    x = x + ((h * h) @ p[f"blocks.{i}.mlp.cProj"].to(h.dtype)) * lm
            logits = F.linear(_rms(x * fscale), p["lmHead.weight"]).float()
        logits = torch.tanh(logits / cfg.softcap_value) * cfg.softcap_value
        return F.cross_entropy(logits.reshape(-1, cfg.vocab_size), targets.reshape(-1))

    @torch.no_grad()
    def _newton_schulz(self, g: torch.Tensor, iters: int = 5) -> torch.Tensor:
        a, b, c = 3.4445, -4.7750, 2.0315
        x = g.bfloat16()
        x = x / (x.norm() + 1e-7)
        tall = x.shape[0] > x.shape[1]
        if tall:
            x = x.T
        for _ in range(iters):
            A = x @ x.T
            Bm = b * A + c * (A @ A)
            x = a * x + Bm @ x
        return (x.T if tall else x).float()

    def step(self, micro_batches: Sequence[Tuple[torch.Tensor, torch.Tensor]]):
        for v in self.p.values():
            v.grad = None
        total = 0.0
        for ids, tgt in micro_batches:
            loss = self.forward_loss(ids, tgt) / len(micro_batches)
            loss.backward()
            total = total + loss.detach()
        if self.world_size > 1:
            for v in self.p.values():                      # one NCCL all-reduce per parameter, as the reference does
                if v.grad is not None:
                    dist.all_reduce(v.grad, op=dist.ReduceOp.AVG)
        hp = self.hp
        self.step_index += 1
        t = self.step_index
        lr_m, lr_e = hp.matrix_lr, hp.embedding_lr
        with torch.no_grad():
            for k, v in self.p.items():
                if v.grad is None:
                    continue
                if self._is_matrix(k):
                    m = self.muon_state[k]
                    m.mul_(0.95).add_(v.grad)
                    u = self._newton_schulz(v.grad.add(m, alpha=0.95))
                    v.add_(u, alpha=-lr_m * max(1.0, v.shape[0] / v.shape[1]) ** 0.5)
                else:
                    m, s = self.adam_state[k]
                    m.mul_(hp.adam_beta1).add_(v.grad, alpha=1 - hp.adam_beta1)
                    s.mul_(hp.adam_beta2).addcmul_(v.grad, v.grad, value=1 - hp.adam_beta2)
                    bc1, bc2 = 1 - hp.adam_beta1 ** t, 1 - hp.adam_beta2 ** t
                    lr = hp.unembedding_lr if k == "lmHead.weight" else lr_e
                    v.addcdiv_(m / bc1, (s / bc2).sqrt_().add_(1e-10), value=-lr)
        toks = sum(int(i.numel()) for i, _ in micro_batches)
        return _Res(total, toks, self.step_index)

    def train_step_from_host(self, tokens_host: torch.Tensor) -> float:
        tok = tokens_host.to(self.device, non_blocking=True)
        return float(self.step([(tok[:, :-1].contiguous(), tok[:, 1:].contiguous())]).loss.item())
