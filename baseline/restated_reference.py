"""A plain-PyTorch restatement of the reference's NanoChat training step, used only as a comparison arm of
``bench.py --impl restated`` when the reference itself (a Lean 4 program) cannot be installed.

It restates what the reference computes with the libraries the reference calls on a CUDA box: libtorch ops
(cuBLAS GEMMs, SDPA, elementwise kernels) for the model (Examples/NanoChat/ModdedGPT.lean:552-650), Muon by five
Newton-Schulz ``torch.matmul`` iterations per matrix (cc/src/tyr_polar.cpp:267-317) and per-tensor AdamW.  None of this
repository's kernels are on that path.

Precision: ``fp32`` (the default) is what the reference trains in: fp32 parameters, activations and products, TF32 off as
in libtorch's default.  ``bf16`` wraps the model in bf16 autocast, the generous reading that an earlier comparison used.

Distributed step, as the reference sequences it (blocking c10d calls on the default stream):
  * AdamW tensors (Tyr/Optim/DistAdam.lean:226-259): reduce_scatter(avg) of the gradient over dim 0, AdamW on the owned rows,
    all_gather of the parameter rows and of both moment tensors; tensors whose dim 0 does not divide by the world all_reduce.
  * Muon matrices (Tyr/Optim/NorMuon.lean:379-404): parameters in blocks of ``world``, rank r owns ``base + r``:
    reduce_scatter over the per-rank gradient list (zero tensors pad the last block), the owner steps, all_gather of the
    parameters and of the momentum buffers.
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
    def __init__(self, cfg: nc.Config, hp: eng.Hyperparameters, device="cuda", world_size: int = 1, rank: int = 0, seed: int = 1234,
                 precision: str = "fp32"):
        if precision not in ("fp32", "bf16"):
            raise ValueError("precision must be 'fp32' or 'bf16'")
        self.cfg, self.hp, self.device, self.world_size, self.rank = cfg, hp, torch.device(device), world_size, rank
        self.precision = precision
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
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=self.device.type == "cuda" and self.precision == "bf16"):
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
        x = g.bfloat16() if self.precision == "bf16" else g.float()
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
        hp = self.hp
        self.step_index += 1
        with torch.no_grad():
            if self.world_size > 1:
                self._distributed_update()
            else:
                for k, v in self.p.items():
                    if v.grad is None:
                        continue
                    if self._is_matrix(k):
                        self.muon_state[k] = self._muon(v, v.grad, self.muon_state[k])
                    else:
                        self._adam(k, v, v.grad, *self.adam_state[k])
        toks = sum(int(i.numel()) for i, _ in micro_batches)
        return _Res(total, toks, self.step_index)

    # -- optimizer pieces ------------------------------------------------------------------------------------
    def _muon(self, v: torch.Tensor, grad: torch.Tensor, m: torch.Tensor) -> torch.Tensor:
        """In-place Muon step on ``v``; returns the new momentum buffer."""
        m = m.mul(0.95).add_(grad)
        u = self._newton_schulz(grad.add(m, alpha=0.95))
        v.add_(u.to(v.dtype), alpha=-self.hp.matrix_lr * max(1.0, v.shape[0] / v.shape[1]) ** 0.5)
        return m

    def _adam(self, k: str, v: torch.Tensor, grad: torch.Tensor, m: torch.Tensor, s: torch.Tensor) -> None:
        hp, t = self.hp, self.step_index
        m.mul_(hp.adam_beta1).add_(grad, alpha=1 - hp.adam_beta1)
        s.mul_(hp.adam_beta2).addcmul_(grad, grad, value=1 - hp.adam_beta2)
        bc1, bc2 = 1 - hp.adam_beta1 ** t, 1 - hp.adam_beta2 ** t
        lr = hp.unembedding_lr if k == "lmHead.weight" else hp.embedding_lr
        v.addcdiv_(m / bc1, (s / bc2).sqrt_().add_(1e-10), value=-lr)

    def _distributed_update(self) -> None:
        W, rank = self.world_size, self.rank
        # AdamW tensors: reduce_scatter -> step on the owned rows -> all_gather of parameter, exp_avg and exp_avg_sq
        for k, v in self.p.items():
            if v.grad is None or self._is_matrix(k):
                continue
            m, s = self.adam_state[k]
            if v.dim() == 0 or v.shape[0] % W != 0:
                dist.all_reduce(v.grad, op=dist.ReduceOp.AVG)
                self._adam(k, v, v.grad, m, s)
                continue
            rows = v.shape[0] // W
            sl = slice(rank * rows, (rank + 1) * rows)
            g_shard = torch.empty_like(v.grad[sl])
            dist.reduce_scatter_tensor(g_shard, v.grad.contiguous(), op=dist.ReduceOp.AVG)
            p_shard, m_shard, s_shard = v.data[sl].clone(), m[sl].clone(), s[sl].clone()
            self._adam(k, p_shard, g_shard, m_shard, s_shard)
            for full, shard in ((v.data, p_shard), (m, m_shard), (s, s_shard)):
                dist.all_gather_into_tensor(full, shard)
        # Muon matrices of one shape form a group; blocks of `world` parameters, rank r owns base + r
        groups: Dict[tuple, list] = {}
        for k, v in self.p.items():
            if v.grad is not None and self._is_matrix(k):
                groups.setdefault(tuple(v.shape), []).append(k)
        for names in groups.values():
            proto = self.p[names[0]]
            for base in range(0, len(names), W):
                g_list = [self.p[names[base + r]].grad.contiguous() if base + r < len(names) else torch.zeros_like(proto)
                          for r in range(W)]
                g_own = torch.empty_like(proto)
                dist.reduce_scatter(g_own, g_list, op=dist.ReduceOp.AVG)
                mine = base + rank
                if mine < len(names):
                    v = self.p[names[mine]]
                    self.muon_state[names[mine]] = self._muon(v.data, g_own, self.muon_state[names[mine]])
                    p_send, m_send = v.data, self.muon_state[names[mine]]
                else:
                    p_send, m_send = torch.zeros_like(proto), torch.zeros_like(proto)
                p_all = [torch.empty_like(proto) for _ in range(W)]
                m_all = [torch.empty_like(proto) for _ in range(W)]
                dist.all_gather(p_all, p_send.contiguous())
                dist.all_gather(m_all, m_send.contiguous())
                for r in range(W):
                    if base + r < len(names):
                        self.p[names[base + r]].data.copy_(p_all[r])
                        self.muon_state[names[base + r]] = m_all[r]

    def train_step_from_host(self, tokens_host: torch.Tensor) -> float:
        tok = tokens_host.to(self.device, non_blocking=True)
        return float(self.step([(tok[:, :-1].contiguous(), tok[:, 1:].contiguous())]).loss.item())
