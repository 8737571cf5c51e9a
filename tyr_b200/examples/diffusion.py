"""Masked discrete diffusion on ASCII text: a bidirectional transformer with timestep embeddings, parameter-free RMSNorm,
ReLU^2 MLP and rotary positions, a linear masking schedule, confidence / top-k parallel decoding, an AdamW training loop
with snapshot checkpoints and a small CLI (Examples/Diffusion/{Diffusion,DiffusionSchedule,DiffusionTrain,DiffusionCheckpoint}.lean,
Examples/TrainDiffusion.lean).

    python -m tyr_b200.examples.diffusion --data input.txt --config small --iterations 2000 --checkpoint-dir ckpt
    python -m tyr_b200.examples.diffusion --sample --checkpoint-dir ckpt --method confidence
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
from dataclasses import asdict, dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

from ..io import checkpoint as snap
from ..io import safetensors as st
from ..ops.rope import apply_rotary, rotary_freqs


@dataclass
class Config:
    seq_len: int = 256
    vocab_size: int = 128          # ASCII, 0 = [MASK]
    mask_token_id: int = 0
    n_layer: int = 4
    n_head: int = 4
    half_head_dim: int = 32
    diffusion_steps: int = 64
    context_len: int = 16          # prefix tokens that are never masked

    def __post_init__(self):
        if (self.n_head <= 0 or self.half_head_dim <= 0 or self.seq_len <= 0 or self.diffusion_steps <= 0 or self.vocab_size <= 0
                or self.context_len > self.seq_len or self.mask_token_id >= self.vocab_size):
            raise ValueError("Invalid diffusion dimensions, rotary head width, context, or mask token")

    @property
    def head_dim(self): return 2 * self.half_head_dim
    @property
    def n_embd(self): return self.n_head * self.head_dim

    @staticmethod
    def tiny(): return Config(seq_len=64, n_layer=2, n_head=2, half_head_dim=16, diffusion_steps=16)
    @staticmethod
    def small(): return Config(seq_len=128, n_layer=4, n_head=4, half_head_dim=32, diffusion_steps=64, context_len=0)
    @staticmethod
    def full(): return Config(seq_len=256, n_layer=6, n_head=6, half_head_dim=32, diffusion_steps=128)


def init(cfg: Config, device="cpu", seed: int = 0) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    C = cfg.n_embd
    rn = lambda *s: torch.randn(*s, generator=g)
    p = {"token_emb": rn(cfg.vocab_size, C) / math.sqrt(C), "time_emb": rn(cfg.diffusion_steps, C), "output_head": torch.zeros(cfg.vocab_size, C)}
    bound = math.sqrt(3.0) * 0.5 / math.sqrt(C)
    for i in range(cfg.n_layer):
        for n in ("c_q", "c_k", "c_v"):
            p[f"blocks.{i}.attn.{n}"] = (torch.rand(C, C, generator=g) * 2 - 1) * bound
        p[f"blocks.{i}.attn.c_proj"] = torch.zeros(C, C)
        p[f"blocks.{i}.mlp.c_fc"] = (torch.rand(4 * C, C, generator=g) * 2 - 1) * bound
        p[f"blocks.{i}.mlp.c_proj"] = torch.zeros(C, 4 * C)
    return {k: v.to(device).requires_grad_(True) for k, v in p.items()}


def norm(x):
    return F.rms_norm(x, (x.shape[-1],))


def forward(p: Dict[str, torch.Tensor], cfg: Config, x_t: torch.Tensor, t: torch.Tensor, rotary=None) -> torch.Tensor:
    """x_t: [B, S] tokens with masks, t: [B] timestep indices -> logits [B, S, V].  Attention is bidirectional."""
    B, S = x_t.shape
    H, D = cfg.n_head, cfg.head_dim
    cos, sin = rotary if rotary is not None else rotary_freqs(S, D, 10000.0, x_t.device)
    x = norm(F.embedding(x_t, p["token_emb"]) + F.embedding(t, p["time_emb"]).unsqueeze(1))
    for i in range(cfg.n_layer):
        h = norm(x)
        q, k, v = (F.linear(h, p[f"blocks.{i}.attn.{n}"]).reshape(B, S, H, D) for n in ("c_q", "c_k", "c_v"))
        q, k = norm(apply_rotary(q, cos[:S], sin[:S])), norm(apply_rotary(k, cos[:S], sin[:S]))
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=False)
        x = x + F.linear(a.transpose(1, 2).reshape(B, S, H * D), p[f"blocks.{i}.attn.c_proj"])
        x = x + F.linear(F.relu(F.linear(norm(x), p[f"blocks.{i}.mlp.c_fc"])).square(), p[f"blocks.{i}.mlp.c_proj"])
    return F.linear(norm(x), p["output_head"])


# ---- schedule ---------------------------------------------------------------------------------------------------------
@dataclass
class MaskedDiffusionSchedule:
    mask_token_id: int
    context_len: int
    mask_probs: torch.Tensor            # [T]: probability of masking at timestep t, linear from 1/T to 1

    @staticmethod
    def init(num_timesteps: int, mask_token_id: int, context_len: int, device="cpu") -> "MaskedDiffusionSchedule":
        return MaskedDiffusionSchedule(mask_token_id, context_len, torch.linspace(1.0 / num_timesteps, 1.0, num_timesteps, device=device))

    def add_masks(self, x0: torch.Tensor, t: torch.Tensor, generator=None) -> torch.Tensor:
        B, S = x0.shape
        prob = self.mask_probs[t].unsqueeze(1)
        should = torch.rand(B, S, generator=generator, device=x0.device if generator is None else generator.device).to(x0.device) < prob
        should &= torch.arange(S, device=x0.device)[None, :] >= self.context_len
        return torch.where(should, torch.full_like(x0, self.mask_token_id), x0)


def masked_cross_entropy_loss(logits, targets, x_t, mask_token_id: int) -> torch.Tensor:
    """Mean CE over the positions that are masked in ``x_t``."""
    per = F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), targets.reshape(-1), reduction="none")
    m = (x_t.reshape(-1) == mask_token_id).float()
    return (per * m).sum() / (m.sum() + 1e-8)


# ---- sampling -----------------------------------------------------------------------------------------------------------
def _start(cfg: Config, batch: int, context: Optional[torch.Tensor], device):
    x = torch.full((batch, cfg.seq_len), cfg.mask_token_id, dtype=torch.int64, device=device)
    prefix = 0
    if context is not None:
        if context.shape != (batch, cfg.context_len):
            raise ValueError("context tokens must be [batch, context_len]")
        x[:, :cfg.context_len] = context
        prefix = cfg.context_len
    return x, prefix


def _masked(x, cfg: Config, prefix: int):
    return (x == cfg.mask_token_id) & (torch.arange(x.shape[1], device=x.device)[None, :] >= prefix)


def _confidences(p, cfg: Config, x, t, rotary, temperature: float):
    """Top probability and its token per position; the mask token itself is never a prediction, so every decoding
    step makes progress."""
    probs = torch.softmax(forward(p, cfg, x, t, rotary).float() / temperature, -1)
    probs[..., cfg.mask_token_id] = 0.0
    return probs.max(-1)


def _validate(batch: int, temperature: float):
    if batch <= 0 or not (temperature > 0 and math.isfinite(temperature)):
        raise ValueError("Diffusion sampling requires a nonempty batch and finite positive temperature")


@torch.no_grad()
def sample_confidence(p, cfg: Config, batch: int = 1, threshold: float = 0.5, temperature: float = 1.0, max_steps: int = 256,
                      context: Optional[torch.Tensor] = None, device="cpu") -> torch.Tensor:
    """Each step decodes every masked position whose top probability reaches ``threshold``; when none does, the single
    most confident position of each row."""
    _validate(batch, temperature)
    x, prefix = _start(cfg, batch, context, device)
    rotary = rotary_freqs(cfg.seq_len, cfg.head_dim, 10000.0, device)
    for step in range(max_steps):
        masked = _masked(x, cfg, prefix)
        if not bool(masked.any()):
            break
        t = torch.full((batch,), max(cfg.diffusion_steps - 1 - step, 0), dtype=torch.int64, device=device)
        conf, pred = _confidences(p, cfg, x, t, rotary, temperature)
        pick = (conf >= threshold) & masked
        if not bool(pick.any()):
            best = torch.where(masked, conf, torch.full_like(conf, -1e10)).argmax(-1, keepdim=True)
            pick = torch.zeros_like(masked).scatter_(1, best, True) & masked
        x = torch.where(pick, pred, x)
    return x


@torch.no_grad()
def sample_top_k(p, cfg: Config, k: int, batch: int = 1, temperature: float = 1.0, max_steps: int = 256,
                 context: Optional[torch.Tensor] = None, device="cpu") -> torch.Tensor:
    """Each step decodes exactly the ``k`` most confident masked positions of every row."""
    _validate(batch, temperature)
    if not 0 < k <= cfg.seq_len:
        raise ValueError("Diffusion top-k must lie between 1 and sequence length")
    x, prefix = _start(cfg, batch, context, device)
    rotary = rotary_freqs(cfg.seq_len, cfg.head_dim, 10000.0, device)
    for step in range(max_steps):
        masked = _masked(x, cfg, prefix)
        if not bool(masked.any()):
            break
        t = torch.full((batch,), max(cfg.diffusion_steps - 1 - step, 0), dtype=torch.int64, device=device)
        conf, pred = _confidences(p, cfg, x, t, rotary, temperature)
        idx = torch.where(masked, conf, torch.full_like(conf, -1e10)).topk(k, dim=-1).indices
        pick = torch.zeros_like(masked).scatter_(1, idx, True) & masked
        x = torch.where(pick, pred, x)
    return x


def decode_ascii(tokens: torch.Tensor, mask_token_id: int = 0) -> str:
    return "".join("_" if t == mask_token_id else (chr(t) if 32 <= t < 127 or t == 10 else "?") for t in tokens.tolist())


def encode_ascii(text: str, vocab_size: int = 128) -> torch.Tensor:
    return torch.tensor([min(ord(c), vocab_size - 1) or 32 for c in text], dtype=torch.int64)


# ---- training -------------------------------------------------------------------------------------------------------------
@dataclass
class TrainConfig:
    iterations: int = 2000
    batch_size: int = 32
    lr: float = 3e-4
    weight_decay: float = 0.01
    warmup: int = 100
    log_interval: int = 50
    checkpoint_interval: int = 500
    seed: int = 0


def lr_at(step: int, tc: TrainConfig) -> float:
    if step < tc.warmup:
        return tc.lr * (step + 1) / tc.warmup
    prog = (step - tc.warmup) / max(1, tc.iterations - tc.warmup)
    return tc.lr * (0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * min(1.0, prog))))


def get_batch(data: torch.Tensor, cfg: Config, batch: int, generator) -> torch.Tensor:
    starts = torch.randint(0, data.numel() - cfg.seq_len, (batch,), generator=generator)
    return torch.stack([data[s:s + cfg.seq_len] for s in starts.tolist()])


def save_checkpoint(root: str, p, opt: torch.optim.Optimizer, cfg: Config, step: int, loss: float) -> str:
    """Snapshot directory with weights, both AdamW moments and a meta file; published atomically."""
    s = snap.begin_snapshot(root)
    st.save_file({k: v.detach().cpu().contiguous() for k, v in p.items()}, os.path.join(s, "model.safetensors"))
    names = list(p.keys())
    osd = {}
    for n in names:
        state = opt.state.get(p[n], {})
        if state:
            osd[f"{n}.exp_avg"], osd[f"{n}.exp_avg_sq"] = state["exp_avg"].cpu().contiguous(), state["exp_avg_sq"].cpu().contiguous()
            osd[f"{n}.step"] = torch.as_tensor(state["step"]).float().reshape(1).cpu()
    st.save_file(osd, os.path.join(s, "optimizer.safetensors"))
    with open(os.path.join(s, "meta.json"), "w") as f:
        json.dump({"step": step, "loss": loss, "config": asdict(cfg)}, f)
    snap.publish_snapshot(root, s)
    return s


def load_checkpoint(root: str, device="cpu", opt_factory=None):
    """Returns (params, config, step, optimizer or None)."""
    s = snap.resolve_snapshot(root)
    meta = json.load(open(os.path.join(s, "meta.json")))
    cfg = Config(**meta["config"])
    src = st.Source.open(os.path.join(s, "model.safetensors"))
    expect = init(cfg, "cpu")
    if sorted(src.names()) != sorted(expect.keys()):
        raise snap.CheckpointError("diffusion checkpoint does not hold this model's parameter set")
    p = {}
    for n in expect:
        tns = src.load(n)
        if tuple(tns.shape) != tuple(expect[n].shape):
            raise snap.CheckpointError(f"diffusion checkpoint: {n} has shape {tuple(tns.shape)}, expected {tuple(expect[n].shape)}")
        p[n] = tns.to(device).requires_grad_(True)
    opt = None
    if opt_factory is not None:
        opt = opt_factory(list(p.values()))
        osrc = st.Source.open(os.path.join(s, "optimizer.safetensors"))
        have = set(osrc.names())
        for n, t in p.items():
            if f"{n}.exp_avg" in have:
                opt.state[t] = {"exp_avg": osrc.load(f"{n}.exp_avg").to(device), "exp_avg_sq": osrc.load(f"{n}.exp_avg_sq").to(device),
                                "step": osrc.load(f"{n}.step").reshape(()).to(torch.float32)}
    return p, cfg, int(meta["step"]), opt


def train(cfg: Config, data: torch.Tensor, tc: TrainConfig, device="cpu", checkpoint_dir: Optional[str] = None, resume: bool = False, log=print,
          stop_at: Optional[int] = None):
    """``stop_at`` ends the run early (after a checkpoint) with the schedules of the full run, as an interrupted job would."""
    gen = torch.Generator().manual_seed(tc.seed)
    mk_opt = lambda params: torch.optim.AdamW(params, lr=tc.lr, betas=(0.9, 0.95), weight_decay=tc.weight_decay)
    step0 = 0
    if resume and checkpoint_dir and os.path.exists(os.path.join(checkpoint_dir, "CURRENT")):
        p, cfg, step0, opt = load_checkpoint(checkpoint_dir, device, mk_opt)
        for _ in range(step0):                                  # replay the data and noise streams up to the saved step
            get_batch(data, cfg, tc.batch_size, gen)
            torch.randint(0, cfg.diffusion_steps, (tc.batch_size,), generator=gen)
            torch.rand(tc.batch_size, cfg.seq_len, generator=gen)
        log(f"resumed at step {step0}")
    else:
        p = init(cfg, device, tc.seed)
        opt = mk_opt(list(p.values()))
    sched = MaskedDiffusionSchedule.init(cfg.diffusion_steps, cfg.mask_token_id, cfg.context_len, device)
    rotary = rotary_freqs(cfg.seq_len, cfg.head_dim, 10000.0, device)
    loss_val = float("nan")
    last = tc.iterations if stop_at is None else min(tc.iterations, stop_at)
    for step in range(step0, last):
        x0 = get_batch(data, cfg, tc.batch_size, gen).to(device)
        t = torch.randint(0, cfg.diffusion_steps, (tc.batch_size,), generator=gen).to(device)
        x_t = sched.add_masks(x0, t, generator=gen)
        for gparam in opt.param_groups:
            gparam["lr"] = lr_at(step, tc)
        loss = masked_cross_entropy_loss(forward(p, cfg, x_t, t, rotary), x0, x_t, cfg.mask_token_id)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(list(p.values()), 1.0)
        opt.step()
        loss_val = float(loss.detach())
        if tc.log_interval and (step + 1) % tc.log_interval == 0:
            log(f"step {step + 1}/{tc.iterations} loss {loss_val:.4f} lr {lr_at(step, tc):.2e}")
        if checkpoint_dir and ((tc.checkpoint_interval and (step + 1) % tc.checkpoint_interval == 0) or step + 1 == last):
            save_checkpoint(checkpoint_dir, p, opt, cfg, step + 1, loss_val)
    return p, loss_val


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="train_diffusion")
    ap.add_argument("--data", default=None, help="text file (ASCII); synthetic text when absent")
    ap.add_argument("--config", default="small", choices=["tiny", "small", "full"])
    ap.add_argument("--iterations", type=int, default=2000)
    ap.add_argument("--batch-size", type=int, default=32)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--checkpoint-dir", default=None)
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--sample", action="store_true")
    ap.add_argument("--method", default="confidence", choices=["confidence", "topk"])
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(sys.argv[1:] if argv is None else argv)
    cfg = getattr(Config, a.config)()
    if a.sample:
        if not a.checkpoint_dir:
            print("--sample needs --checkpoint-dir", file=sys.stderr)
            return 2
        p, cfg, step, _ = load_checkpoint(a.checkpoint_dir, a.device)
        x = sample_confidence(p, cfg, 1, temperature=a.temperature, device=a.device) if a.method == "confidence" else \
            sample_top_k(p, cfg, a.top_k, 1, temperature=a.temperature, device=a.device)
        print(decode_ascii(x[0], cfg.mask_token_id))
        return 0
    if a.data:
        text = open(a.data, encoding="utf-8", errors="replace").read()
    else:
        text = "the quick brown fox jumps over the lazy dog. " * 400
    data = encode_ascii(text, cfg.vocab_size)
    if data.numel() <= cfg.seq_len:
        print("training text is shorter than one sequence", file=sys.stderr)
        return 2
    train(cfg, data, TrainConfig(a.iterations, a.batch_size, a.lr), a.device, a.checkpoint_dir, a.resume)
    return 0


if __name__ == "__main__":
    sys.exit(main())
