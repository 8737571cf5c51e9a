"""KV-cached inference for the NanoChat (modded-nanogpt) model: prefill + single-token steps that reproduce
``forward_reference`` logits position by position (Examples/NanoChat/Generator/KVCache.lean, ModdedGPT.lean:552-635)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from ..models import nanochat as nc
from ..models.common import KVCache, cached_attention
from ..ops import rope as rope_ops
from ..ops.norm import rms_norm_ref


class NanoChatSession:
    """Owns one KV cache per attention layer.  ``params`` uses the reference parameter names."""

    def __init__(self, params: Dict[str, torch.Tensor], cfg: nc.Config, batch: int, max_len: int):
        self.p, self.cfg, self.batch, self.max_len, self.pos = params, cfg, batch, max_len, 0
        dev, dt = params["embed"].device, params["embed"].dtype
        self.cos, self.sin = rope_ops.rotary_freqs(max_len, cfg.head_dim, cfg.rope_base if hasattr(cfg, "rope_base") else 500000.0, dev)
        self.caches: List[Optional[KVCache]] = [
            KVCache.allocate(batch, cfg.n_head, max_len, cfg.head_dim, dev, dt) if f"blocks.{i}.attn.wQ" in params else None
            for i in range(cfg.n_layer)]

    @torch.no_grad()
    def run(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [B, S] appended at the current position; returns soft-capped logits of the last position [B, V]."""
        p, cfg = self.p, self.cfg
        B, S = ids.shape
        if self.pos + S > self.max_len:
            raise ValueError("NanoChat session overflow")
        d, H, D, L = cfg.model_dim, cfg.n_head, cfg.head_dim, cfg.n_layer
        dt = p["embed"].dtype
        norm = lambda x: rms_norm_ref(x).to(dt)
        cos, sin = self.cos[self.pos:self.pos + S], self.sin[self.pos:self.pos + S]
        tok = F.embedding(ids, p["embed"])
        gate = torch.sigmoid(F.linear(tok[..., :12], p["smearGate.weight"].to(dt)))
        x0 = norm(tok + tok * gate)
        ves = [F.embedding(ids, p[f"valueEmbeds.{i}"]) for i in range(cfg.num_value_embeds)]
        sc = p["scalars.values"].float()
        sg = lambda i: torch.sigmoid(sc[i]).to(dt)
        value_mix, skip_mix, final_scale = sg(L * 4), sg(L * 4 + 1), sg(L * 4 + 2)
        x, skip = x0, None
        total = self.pos + S
        for i in range(L):
            lam_x, lam_x0, lam_attn, lam_mlp = sg(4 * i), sg(4 * i + 1), sg(4 * i + 2), sg(4 * i + 3)
            x_in = x * lam_x + x0 * lam_x0
            if i == nc.SKIP_SOURCE_LAYER:
                skip = x_in
            if self.caches[i] is not None:
                window = nc.get_window_size_for_layer(cfg.window_pattern, i, L, cfg.max_seq_len)
                xn = norm(x_in)
                q = F.linear(xn, p[f"blocks.{i}.attn.wQ"])
                k = F.linear(xn, p[f"blocks.{i}.attn.wK"])
                v = F.linear(xn, p[f"blocks.{i}.attn.wV"])
                vi = nc.layer_value_embed_index(cfg, i)
                if vi is not None:
                    v = v * (1 - value_mix) + ves[vi] * value_mix
                q = norm(rope_ops.apply_rotary(q.reshape(B, S, H, D), cos, sin)).transpose(1, 2)
                k = norm(rope_ops.apply_rotary(k.reshape(B, S, H, D), cos, sin)).transpose(1, 2)
                v = v.reshape(B, S, H, D).transpose(1, 2)
                w = window
                o = cached_attention(q, k, v, self.caches[i], w).transpose(1, 2).reshape(B, S, H * D)
                x1 = x_in + F.linear(o, p[f"blocks.{i}.attn.wO"]) * lam_attn
                h = torch.relu(F.linear(norm(x1), p[f"blocks.{i}.mlp.cFc"]))
                x = x1 + ((h * h) @ p[f"blocks.{i}.mlp.cProj"]) * lam_mlp
            else:
                x = x_in + skip * skip_mix if skip is not None else x_in
                h = torch.relu(F.linear(norm(x), p[f"blocks.{i}.mlp.cFc"]))
                x = x + ((h * h) @ p[f"blocks.{i}.mlp.cProj"]) * lam_mlp
        self.pos = total
        logits = F.linear(norm(x[:, -1] * final_scale), p["lmHead.weight"]).float()
        return torch.tanh(logits / cfg.softcap_value) * cfg.softcap_value

    def prefill(self, ids):
        return self.run(ids)

    def step(self, tok):
        return self.run(tok.reshape(self.batch, 1))
