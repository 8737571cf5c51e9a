"""Laguna (poolside Laguna-S-2.1 family): hybrid full / sliding-window attention with per-head
softplus output gates, sigmoid-routed NVFP4 mixture of experts plus a shared expert.

Behavioural contract: Tyr/Model/Laguna/{Config,ConfigIO,Rope,MoE,Model,Weights}.lean.
The expert path runs on the kernels in csrc/moe_nvfp4.cu and the grouped tcgen05 GEMM; sliding
layers keep a ring KV cache of one window.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..io import safetensors as st
from ..ops import moe as moe_ops
from ..ops import decode_attention as da
from ..ops.decode_attention import decode_attention
from ..ops.rope import rope_norm
from .common import (KVCache, apply_rotary_partial, cached_attention, cos_sin_tables, head_norm, lin, norm_w,
                     plain_inv_freq, swiglu_mlp, yarn_inv_freq)
from .generation import SamplingStrategy, StreamCallback, generate_cached

FULL, SLIDING = "full_attention", "sliding_attention"


def default_layer_types(n: int) -> List[str]:
    return [FULL if i % 4 == 0 else SLIDING for i in range(n)]


@dataclass
class LagunaConfig:
    """Defaults match ``poolside/Laguna-S-2.1-NVFP4`` (Config.lean:54-94)."""
    vocab_size: int = 100352
    hidden_size: int = 3072
    intermediate_size: int = 12288
    num_hidden_layers: int = 48
    num_attention_heads: int = 48
    num_attention_heads_sliding: int = 72
    num_key_value_heads: int = 8
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    sliding_window: int = 512
    rope_theta_sliding: float = 10000.0
    half_rotary_dim_sliding: int = 64
    rope_theta_full: float = 500000.0
    half_rotary_dim_full: int = 32
    yarn_factor: float = 32.0
    yarn_original_max_position_embeddings: int = 8192
    yarn_beta_fast: float = 32.0
    yarn_beta_slow: float = 1.0
    yarn_attention_factor: float = 1.3465735902799727
    num_experts: int = 256
    num_experts_per_tok: int = 10
    moe_intermediate_size: int = 1024
    shared_expert_intermediate_size: int = 1024
    norm_topk_prob: bool = True
    moe_routed_scaling_factor: float = 2.5
    moe_router_logit_softcapping: float = 0.0
    mlp_only_layers: Tuple[int, ...] = (0,)
    layer_types: Optional[List[str]] = None
    eos_token_ids: Tuple[int, ...] = (2, 24)

    def __post_init__(self):
        if self.layer_types is None:
            self.layer_types = default_layer_types(self.num_hidden_layers)
        self.validate()

    def validate(self):
        err = lambda m: ValueError(f"Invalid Laguna config: {m}")
        if self.sliding_window <= 0:
            raise err("sliding_window must be positive")
        if min(self.num_attention_heads, self.num_attention_heads_sliding, self.num_key_value_heads) <= 0:
            raise err(f"head counts ({self.num_attention_heads}, {self.num_attention_heads_sliding}, "
                      f"kv {self.num_key_value_heads}) must be positive")
        if self.num_attention_heads % self.num_key_value_heads:
            raise err(f"num_attention_heads ({self.num_attention_heads}) must be divisible by "
                      f"num_key_value_heads ({self.num_key_value_heads})")
        if self.num_attention_heads_sliding % self.num_key_value_heads:
            raise err(f"sliding-layer heads ({self.num_attention_heads_sliding}) must be divisible by "
                      f"num_key_value_heads ({self.num_key_value_heads})")
        for half in (self.half_rotary_dim_full, self.half_rotary_dim_sliding):
            if half <= 0 or 2 * half > self.head_dim:
                raise err(f"rotary dims ({2 * self.half_rotary_dim_full}, {2 * self.half_rotary_dim_sliding}) must be "
                          f"positive, even and at most head_dim={self.head_dim}")
        if len(self.layer_types) != self.num_hidden_layers:
            raise err(f"layer_types has {len(self.layer_types)} entries for num_hidden_layers={self.num_hidden_layers}")
        for t in self.layer_types:
            if t not in (FULL, SLIDING):
                raise err(f'unknown layer type "{t}"; expected full_attention or sliding_attention')
        if any(i >= self.num_hidden_layers for i in self.mlp_only_layers):
            raise err(f"mlp_only_layers {list(self.mlp_only_layers)} must name layers below {self.num_hidden_layers}")
        if self.num_experts > 0 and not (0 < self.num_experts_per_tok <= self.num_experts):
            raise err(f"num_experts_per_tok={self.num_experts_per_tok} must be between 1 and num_experts={self.num_experts}")
        if self.yarn_original_max_position_embeddings <= 0:
            raise err("original_max_position_embeddings must be positive")
        if min(self.rms_norm_eps, self.rope_theta_sliding, self.rope_theta_full, self.yarn_factor) <= 0:
            raise err(f"rms_norm_eps={self.rms_norm_eps}, rope thetas ({self.rope_theta_sliding}, {self.rope_theta_full}) "
                      f"and yarn factor={self.yarn_factor} must be positive")
        if any(e >= self.vocab_size for e in self.eos_token_ids):
            raise err(f"eos_token_id must be below vocab_size={self.vocab_size}")

    # -- per-layer selectors ---------------------------------------------------------------------
    def is_full(self, i: int) -> bool:
        return self.layer_types[i] == FULL

    def heads(self, i: int) -> int:
        return self.num_attention_heads if self.is_full(i) else self.num_attention_heads_sliding

    def is_moe_layer(self, i: int) -> bool:
        return self.num_experts > 0 and i not in self.mlp_only_layers

    def rotary_half(self, i: int) -> int:
        return self.half_rotary_dim_full if self.is_full(i) else self.half_rotary_dim_sliding

    @staticmethod
    def from_json(j: dict) -> "LagunaConfig":
        """HF ``config.json`` (ConfigIO.lean:30-147)."""
        d = LagunaConfig()
        if j.get("hidden_act", "silu") != "silu":
            raise ValueError(f"Invalid Laguna config: hidden_act must be one of ['silu']")
        if j.get("attention_bias", False):
            raise ValueError("Invalid Laguna config: attention_bias must be false")
        n = j.get("num_hidden_layers", d.num_hidden_layers)
        lt = j.get("layer_types") or default_layer_types(n)
        heads_full = j.get("num_attention_heads", d.num_attention_heads)
        heads_sliding = j.get("num_attention_heads_sliding", heads_full if "num_attention_heads" in j else d.num_attention_heads_sliding)
        per_layer = j.get("num_attention_heads_per_layer")
        if per_layer is not None:
            if len(per_layer) != n:
                raise ValueError(f"Invalid Laguna config: num_attention_heads_per_layer has {len(per_layer)} entries for {n} layers")
            for kind in (FULL, SLIDING):
                vals = {h for h, t in zip(per_layer, lt) if t == kind}
                if len(vals) > 1:
                    raise ValueError(f"Invalid Laguna config: num_attention_heads_per_layer varies within {kind} layers")
                if vals:
                    if kind == FULL:
                        heads_full = vals.pop()
                    else:
                        heads_sliding = vals.pop()
        head_dim = j.get("head_dim", d.head_dim)
        rope = j.get("rope_parameters") or {}

        def rf(kind, key, default):
            return (rope.get(kind) or {}).get(key, default)

        def rotary_half(kind, default_half):
            factor = rf(kind, "partial_rotary_factor", None)
            if factor is None:
                return default_half if head_dim == d.head_dim else head_dim // 2
            dim = head_dim * factor
            if abs(dim - round(dim)) > 1e-9 or round(dim) % 2:
                raise ValueError(f"Invalid Laguna config: {kind} partial_rotary_factor={factor} does not select a whole "
                                 f"number of the {head_dim} head channels")
            return int(round(dim)) // 2
        eos = j.get("eos_token_id", list(d.eos_token_ids))
        eos = tuple(eos) if isinstance(eos, list) else (int(eos),)
        simple = {k: j[k] for k in ("vocab_size", "hidden_size", "intermediate_size", "num_key_value_heads", "rms_norm_eps",
                                    "sliding_window", "num_experts", "num_experts_per_tok", "moe_intermediate_size",
                                    "shared_expert_intermediate_size", "norm_topk_prob", "moe_routed_scaling_factor",
                                    "moe_router_logit_softcapping") if k in j}
        return LagunaConfig(
            num_hidden_layers=n, layer_types=list(lt), num_attention_heads=heads_full,
            num_attention_heads_sliding=heads_sliding, head_dim=head_dim,
            half_rotary_dim_full=rotary_half(FULL, d.half_rotary_dim_full),
            half_rotary_dim_sliding=rotary_half(SLIDING, d.half_rotary_dim_sliding),
            rope_theta_sliding=rf(SLIDING, "rope_theta", d.rope_theta_sliding),
            rope_theta_full=rf(FULL, "rope_theta", j.get("rope_theta", d.rope_theta_full)),
            yarn_factor=rf(FULL, "factor", d.yarn_factor),
            yarn_original_max_position_embeddings=rf(FULL, "original_max_position_embeddings", d.yarn_original_max_position_embeddings),
            yarn_beta_fast=rf(FULL, "beta_fast", d.yarn_beta_fast), yarn_beta_slow=rf(FULL, "beta_slow", d.yarn_beta_slow),
            yarn_attention_factor=rf(FULL, "attention_factor", d.yarn_attention_factor),
            mlp_only_layers=tuple(j.get("mlp_only_layers", [i for i in d.mlp_only_layers if i < n])),
            eos_token_ids=eos, **simple)

    def to_json(self) -> dict:
        """The HF ``config.json`` form that ``from_json`` reads back to an equal config (fixture generators, export)."""
        rope = {
            FULL: {"rope_theta": self.rope_theta_full, "partial_rotary_factor": 2 * self.half_rotary_dim_full / self.head_dim,
                   "factor": self.yarn_factor, "original_max_position_embeddings": self.yarn_original_max_position_embeddings,
                   "beta_fast": self.yarn_beta_fast, "beta_slow": self.yarn_beta_slow, "attention_factor": self.yarn_attention_factor},
            SLIDING: {"rope_theta": self.rope_theta_sliding, "partial_rotary_factor": 2 * self.half_rotary_dim_sliding / self.head_dim},
        }
        return {"model_type": "laguna", "hidden_act": "silu", "attention_bias": False, "vocab_size": self.vocab_size,
                "hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
                "num_hidden_layers": self.num_hidden_layers, "layer_types": list(self.layer_types),
                "num_attention_heads": self.num_attention_heads, "num_attention_heads_sliding": self.num_attention_heads_sliding,
                "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim, "rms_norm_eps": self.rms_norm_eps,
                "sliding_window": self.sliding_window, "num_experts": self.num_experts,
                "num_experts_per_tok": self.num_experts_per_tok, "moe_intermediate_size": self.moe_intermediate_size,
                "shared_expert_intermediate_size": self.shared_expert_intermediate_size, "norm_topk_prob": self.norm_topk_prob,
                "moe_routed_scaling_factor": self.moe_routed_scaling_factor,
                "moe_router_logit_softcapping": self.moe_router_logit_softcapping, "mlp_only_layers": list(self.mlp_only_layers),
                "eos_token_id": list(self.eos_token_ids), "rope_parameters": rope}

    @staticmethod
    def load_from_pretrained_dir(model_dir: str) -> "LagunaConfig":
        with open(os.path.join(model_dir, "config.json")) as f:
            return LagunaConfig.from_json(json.load(f))


# ---- rotary tables -------------------------------------------------------------------------------------
@dataclass
class RotaryTables:
    sliding_cos: torch.Tensor
    sliding_sin: torch.Tensor
    full_cos: torch.Tensor
    full_sin: torch.Tensor

    def rows(self, full: bool, start: int, n: int):
        c, s = (self.full_cos, self.full_sin) if full else (self.sliding_cos, self.sliding_sin)
        if start + n > c.shape[0]:
            raise ValueError("Laguna cache rotary tables do not cover the requested positions")
        return c[start:start + n], s[start:start + n]


def precompute_rotary_tables(cfg: LagunaConfig, max_len: int, device="cpu") -> RotaryTables:
    sc, ss = cos_sin_tables(plain_inv_freq(cfg.half_rotary_dim_sliding, cfg.rope_theta_sliding), max_len, 1.0, device)
    fc, fs = cos_sin_tables(yarn_inv_freq(cfg.half_rotary_dim_full, cfg.rope_theta_full, cfg.yarn_factor,
                                          cfg.yarn_original_max_position_embeddings, cfg.yarn_beta_fast, cfg.yarn_beta_slow),
                            max_len, cfg.yarn_attention_factor, device)
    return RotaryTables(sc, ss, fc, fs)


# ---- parameters --------------------------------------------------------------------------------------------
@dataclass
class Attention:
    q_proj: torch.Tensor
    k_proj: torch.Tensor
    v_proj: torch.Tensor
    o_proj: torch.Tensor
    g_proj: torch.Tensor
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    _qkvg: Optional[torch.Tensor] = None      # fused [q;k;v;g] projection, built lazily for inference

    def fused(self) -> torch.Tensor:
        if self._qkvg is None:
            pad = (-self.g_proj.shape[0]) % 8
            g = F.pad(self.g_proj, (0, 0, 0, pad)) if pad else self.g_proj
            self._qkvg = torch.cat([self.q_proj, self.k_proj, self.v_proj, g], 0).contiguous()
        return self._qkvg


@dataclass
class DenseMLP:
    gate_proj: torch.Tensor
    up_proj: torch.Tensor
    down_proj: torch.Tensor


@dataclass
class Router:
    weight: torch.Tensor                           # [E, hidden]
    e_score_correction_bias: Optional[torch.Tensor] = None


@dataclass
class DenseExperts:
    gate_proj: torch.Tensor   # [E, mi, h]
    up_proj: torch.Tensor
    down_proj: torch.Tensor   # [E, h, mi]


@dataclass
class SparseMoeBlock:
    router: Router
    experts: Optional[moe_ops.PackedExperts]
    shared_gate_proj: torch.Tensor
    shared_up_proj: torch.Tensor
    shared_down_proj: torch.Tensor
    dense_experts: Optional[DenseExperts] = None


@dataclass
class Layer:
    input_layernorm: torch.Tensor
    attn: Attention
    post_attention_layernorm: torch.Tensor
    ffn: object                                   # DenseMLP | SparseMoeBlock


@dataclass
class LagunaForCausalLM:
    cfg: LagunaConfig
    embed_tokens: torch.Tensor
    layers: List[Layer]
    norm: torch.Tensor
    lm_head: torch.Tensor
    tie_word_embeddings: bool = False
    ep: Optional[object] = None      # parallel.ep.ExpertParallel: experts split over the ranks, banks hold the local slice

    @property
    def device(self):
        return self.embed_tokens.device

    @property
    def dtype(self):
        return self.embed_tokens.dtype


def _w(shape, fan_in, device, dtype, gen):
    return (torch.randn(shape, generator=gen, dtype=torch.float32) * (fan_in ** -0.5)).to(device=device, dtype=dtype)


def random_packed_experts(cfg: LagunaConfig, device, gen, dense_std: Optional[float] = None,
                          num_local: Optional[int] = None) -> moe_ops.PackedExperts:
    """Synthetic NVFP4 banks: quantised gaussian weights, real U8 / e4m3 tensors (the fused op needs
    those, Tyr/Model/Laguna/MoE.lean:209-216).  ``num_local`` builds only that many experts (one EP rank's slice)."""
    E, mi, h = num_local or cfg.num_experts, cfg.moe_intermediate_size, cfg.hidden_size

    def bank(rows, cols):
        packed = torch.empty((E, rows, cols // 2), dtype=torch.uint8, device=device)
        scales = torch.empty((E, rows, cols // 16), dtype=torch.float8_e4m3fn, device=device)
        glob = torch.empty(E, dtype=torch.float32, device=device)
        step = max(1, min(E, (1 << 28) // (rows * cols)))
        for e0 in range(0, E, step):
            n = min(step, E - e0)
            w = torch.randn((n, rows, cols), generator=gen, dtype=torch.float32) * (dense_std or cols ** -0.5)
            p, s, g = moe_ops.nvfp4_quantize(w.to(device))
            packed[e0:e0 + n], scales[e0:e0 + n], glob[e0:e0 + n] = p, s, g
        return packed, scales, glob
    gp, gs, gg = bank(mi, h)
    up, us, ug = bank(mi, h)
    dp, ds, dg = bank(h, mi)
    return moe_ops.PackedExperts(gp, gs, gg, up, us, ug, dp, ds, dg)


def init(cfg: LagunaConfig, device="cpu", dtype=torch.float32, tie_word_embeddings: bool = False, seed: int = 0,
         dense_experts: bool = False, ep=None) -> LagunaForCausalLM:
    """Random-init model.  With ``ep`` (an ``ExpertParallel`` group) every rank draws the same dense weights and
    only its own slice of each expert bank."""
    gen = torch.Generator().manual_seed(seed)
    egen = torch.Generator().manual_seed(seed + 7919 * (1 + (ep.rank if ep is not None else 0)))
    h, D = cfg.hidden_size, cfg.head_dim
    mk = lambda shape, fan: _w(shape, fan, device, dtype, gen)
    ones = lambda n: torch.ones(n, device=device, dtype=dtype)
    layers = []
    for i in range(cfg.num_hidden_layers):
        H = cfg.heads(i)
        attn = Attention(mk((H * D, h), h), mk((cfg.num_key_value_heads * D, h), h), mk((cfg.num_key_value_heads * D, h), h),
                         mk((h, H * D), H * D), mk((H, h), h), ones(D), ones(D))
        if cfg.is_moe_layer(i):
            E, mi, si = cfg.num_experts, cfg.moe_intermediate_size, cfg.shared_expert_intermediate_size
            router = Router(_w((E, h), h, device, torch.float32, gen))
            if dense_experts:
                de = DenseExperts(mk((E, mi, h), h), mk((E, mi, h), h), mk((E, h, mi), mi))
                ffn = SparseMoeBlock(router, None, mk((si, h), h), mk((si, h), h), mk((h, si), si), de)
            else:
                n_loc = ep.E_local if ep is not None else None
                ffn = SparseMoeBlock(router, random_packed_experts(cfg, device, egen if ep is not None else gen, num_local=n_loc),
                                     mk((si, h), h), mk((si, h), h), mk((h, si), si))
        else:
            ffn = DenseMLP(mk((cfg.intermediate_size, h), h), mk((cfg.intermediate_size, h), h), mk((h, cfg.intermediate_size), cfg.intermediate_size))
        layers.append(Layer(ones(h), attn, ones(h), ffn))
    emb = (torch.randn((cfg.vocab_size, h), generator=gen) * 0.02).to(device=device, dtype=dtype)
    head = emb if tie_word_embeddings else mk((cfg.vocab_size, h), h)
    return LagunaForCausalLM(cfg, emb, layers, ones(h), head, tie_word_embeddings, ep)


# ---- blocks ------------------------------------------------------------------------------------------------------
def route(cfg: LagunaConfig, r: Router, x2: torch.Tensor):
    """fp32 router logits -> (ids int32 [T,k], weights fp32 [T,k] including the routed scale, counts)."""
    if moe_ops.route_fused_supported(x2, r.weight):
        return moe_ops.route_fused(x2, r.weight, cfg.num_experts_per_tok, softmax=False, bias=r.e_score_correction_bias, renorm=cfg.norm_topk_prob,
                                   softcap=cfg.moe_router_logit_softcapping, scale=cfg.moe_routed_scaling_factor)
    logits = F.linear(x2.float(), r.weight.float())
    return moe_ops.route(logits, cfg.num_experts_per_tok, softmax=False, bias=r.e_score_correction_bias,
                         renorm=cfg.norm_topk_prob, softcap=cfg.moe_router_logit_softcapping,
                         scale=cfg.moe_routed_scaling_factor)


def moe_forward(cfg: LagunaConfig, m: SparseMoeBlock, x2: torch.Tensor, use_fused: bool = True, ep=None) -> torch.Tensor:
    """``scale * sum_k w_k expert_k(x) + shared(x)`` over [tokens, hidden] (MoE.lean:267-356).  With ``ep`` the
    routed part runs expert-parallel: rows are pulled by the rank that owns the expert and the results pulled back."""
    ids, w, counts = route(cfg, m.router, x2)
    shared = swiglu_mlp(x2, m.shared_gate_proj, m.shared_up_proj, m.shared_down_proj)
    if ep is not None:
        from ..parallel.ep import local_expert_fn
        banks = m.experts if m.dense_experts is None else (
            torch.cat([m.dense_experts.gate_proj, m.dense_experts.up_proj], 1), m.dense_experts.down_proj)
        return ep.forward(x2, ids, w, local_expert_fn(banks), add=shared, counts=counts)
    if m.dense_experts is not None:
        de = m.dense_experts
        return (moe_ops.moe_eager(x2, ids, w, de.gate_proj, de.up_proj, de.down_proj).float() + shared.float()).to(x2.dtype)
    fused_ok = use_fused and x2.is_cuda and x2.dtype == torch.bfloat16
    if fused_ok:
        return moe_ops.moe_fp4_forward(x2, ids, w, m.experts, counts=counts, add=shared)
    # eager path on the dequantised banks: model-dtype arithmetic in the reference's op order
    g, u, d = m.experts.dense()
    sc = cfg.moe_routed_scaling_factor
    return moe_ops.moe_eager_model_dtype(x2, ids, w / sc, g, u, d, scale=sc) + shared


def attention_forward(cfg: LagunaConfig, i: int, a: Attention, x: torch.Tensor, cos, sin,
                      cache: Optional[KVCache]) -> torch.Tensor:
    B, S, _ = x.shape
    H, Hkv, D = cfg.heads(i), cfg.num_key_value_heads, cfg.head_dim
    y = lin(x, a.fused())
    q, k, v, g = torch.split(y, [H * D, Hkv * D, Hkv * D, y.shape[-1] - (H + 2 * Hkv) * D], dim=-1)
    q = head_norm(q.reshape(B, S, H, D), a.q_norm, cfg.rms_norm_eps)
    k = head_norm(k.reshape(B, S, Hkv, D), a.k_norm, cfg.rms_norm_eps)
    q = apply_rotary_partial(q, cos, sin).transpose(1, 2)
    k = apply_rotary_partial(k, cos, sin).transpose(1, 2)
    v = v.reshape(B, S, Hkv, D).transpose(1, 2)
    window = None if cfg.is_full(i) else cfg.sliding_window
    o = cached_attention(q, k, v, cache, window)                      # [B, H, S, D]
    gate = F.softplus(g[..., :H].float()).to(x.dtype)                 # [B, S, H]
    gated = (o.transpose(1, 2) * gate.unsqueeze(-1)).reshape(B, S, H * D)
    return lin(gated, a.o_proj)


def attention_decode(cfg: LagunaConfig, i: int, a: Attention, x: torch.Tensor, tables: RotaryTables, pos_t: torch.Tensor,
                     cache: KVCache) -> torch.Tensor:
    """One new token per row with the position on the device: fused q/k/v/g projection, RMSNorm+RoPE kernel on the q and k
    slices, split-KV attention kernel that also appends to the store.  x: [B, 1, hidden]."""
    B = x.shape[0]
    H, Hkv, D = cfg.heads(i), cfg.num_key_value_heads, cfg.head_dim
    y = lin(x, a.fused()).reshape(B, -1)
    q, k, v = y[:, :H * D].view(B, H, D), y[:, H * D:(H + Hkv) * D].view(B, Hkv, D), y[:, (H + Hkv) * D:(H + 2 * Hkv) * D].view(B, Hkv, D)
    g = y[:, (H + 2 * Hkv) * D:(H + 2 * Hkv) * D + H]
    cos, sin = (tables.full_cos, tables.full_sin) if cfg.is_full(i) else (tables.sliding_cos, tables.sliding_sin)
    positions = pos_t.expand(B)
    rot = 2 * cos.shape[1]
    q = rope_norm(q, cos, sin, weight=a.q_norm, positions=positions, rot=rot, eps=cfg.rms_norm_eps)
    k = rope_norm(k, cos, sin, weight=a.k_norm, positions=positions, rot=rot, eps=cfg.rms_norm_eps)
    # the per-head softplus gate is applied inside the attention kernel's final write
    o = decode_attention(q, k, v, cache.k, cache.v, pos_t, ring=cache.ring, window=None if cfg.is_full(i) else cfg.sliding_window,
                         head_gate=g)
    return lin(o.reshape(B, 1, H * D), a.o_proj)


def layer_decode(cfg: LagunaConfig, i: int, layer: Layer, x: torch.Tensor, h1: torch.Tensor, next_norm: torch.Tensor,
                 tables: RotaryTables, pos_t: torch.Tensor, cache: KVCache, use_fused: bool = True, ep=None):
    """One decode layer on the residual stream ``x`` whose input norm ``h1`` is already taken.  Returns the new residual
    stream and its norm under ``next_norm`` (the next layer's input norm or the final norm): each residual add runs inside
    the norm kernel that follows it."""
    B, S, h = x.shape
    eps = cfg.rms_norm_eps
    h3, h2 = norm_w(attention_decode(cfg, i, layer.attn, h1, tables, pos_t, cache), layer.post_attention_layernorm, eps,
                    residual=x, return_residual=True)
    if isinstance(layer.ffn, DenseMLP):
        f = swiglu_mlp(h3, layer.ffn.gate_proj, layer.ffn.up_proj, layer.ffn.down_proj)
    else:
        f = moe_forward(cfg, layer.ffn, h3.reshape(B * S, h), use_fused, ep).reshape(B, S, h)
    h_next, x_new = norm_w(f, next_norm, eps, residual=h2, return_residual=True)
    return x_new, h_next


def layer_forward(cfg: LagunaConfig, i: int, layer: Layer, x: torch.Tensor, tables: RotaryTables, position: int,
                  cache: Optional[KVCache], use_fused: bool = True, ep=None) -> torch.Tensor:
    B, S, h = x.shape
    cos, sin = tables.rows(cfg.is_full(i), position, S)
    h1 = norm_w(x, layer.input_layernorm, cfg.rms_norm_eps)
    h2 = x + attention_forward(cfg, i, layer.attn, h1, cos, sin, cache)
    h3 = norm_w(h2, layer.post_attention_layernorm, cfg.rms_norm_eps)
    if isinstance(layer.ffn, DenseMLP):
        f = swiglu_mlp(h3, layer.ffn.gate_proj, layer.ffn.up_proj, layer.ffn.down_proj)
    else:
        f = moe_forward(cfg, layer.ffn, h3.reshape(B * S, h), use_fused, ep).reshape(B, S, h)
    return h2 + f


def forward_hidden(m: LagunaForCausalLM, input_ids: torch.Tensor, use_fused: bool = True) -> torch.Tensor:
    """Uncached full-sequence forward to final hidden states (Model.lean LagunaModel.forward)."""
    cfg = m.cfg
    x = F.embedding(input_ids, m.embed_tokens)
    tables = precompute_rotary_tables(cfg, input_ids.shape[1], x.device)
    for i, layer in enumerate(m.layers):
        x = layer_forward(cfg, i, layer, x, tables, 0, None, use_fused, m.ep)
    return norm_w(x, m.norm, cfg.rms_norm_eps)


def forward(m: LagunaForCausalLM, input_ids: torch.Tensor, use_fused: bool = True) -> torch.Tensor:
    return lin(forward_hidden(m, input_ids, use_fused), m.lm_head)


# ---- inference session --------------------------------------------------------------------------------------------------
class CacheSession:
    """Owned per-layer caches: full layers reserve ``max_len``, sliding layers ``min(max_len, window)``
    as ring stores (Model.lean:729-752).  ``fork`` copies the stores so an earlier state stays intact."""

    def __init__(self, m: LagunaForCausalLM, batch: int, max_len: int, tables: Optional[RotaryTables] = None):
        cfg = m.cfg
        if max_len <= 0:
            raise ValueError("Laguna cache capacity must be positive")
        if cfg.num_hidden_layers == 0:
            raise ValueError("Laguna cache session requires at least one layer")
        self.m, self.batch, self.max_len, self.pos = m, batch, max_len, 0
        self.pos_t, self._graph, self._pos_t_host = None, None, -1
        self.tables = tables or precompute_rotary_tables(cfg, max_len, m.device)
        self.caches = [KVCache.allocate(batch, cfg.num_key_value_heads,
                                        max_len if cfg.is_full(i) else min(max_len, cfg.sliding_window),
                                        cfg.head_dim, m.device, m.dtype, ring=not cfg.is_full(i))
                       for i in range(cfg.num_hidden_layers)]

    def capacities(self) -> List[int]:
        return [c.cap for c in self.caches]

    def fork(self) -> "CacheSession":
        other = object.__new__(CacheSession)
        other.m, other.batch, other.max_len, other.pos, other.tables = self.m, self.batch, self.max_len, self.pos, self.tables
        other.caches = [c.clone() for c in self.caches]
        other.pos_t, other._graph, other._pos_t_host = None, None, -1
        return other

    @torch.no_grad()
    def _run(self, x: torch.Tensor, use_fused: bool) -> torch.Tensor:
        cfg, S = self.m.cfg, x.shape[1]
        if tuple(x.shape) != (self.batch, S, cfg.hidden_size):
            raise ValueError("Laguna cache input shape mismatch")
        if S == 0 or self.pos + S > self.max_len:
            raise ValueError("Laguna cache overflow")
        if self.pos > 0 and S != 1:
            raise ValueError("chunked prefill is not supported; prefill a fresh session")
        for i, layer in enumerate(self.m.layers):
            x = layer_forward(cfg, i, layer, x, self.tables, self.pos, self.caches[i], use_fused, self.m.ep)
        self.pos += S
        return norm_w(x, self.m.norm, cfg.rms_norm_eps)

    def prefill(self, input_ids: torch.Tensor, use_fused: bool = True) -> torch.Tensor:
        """Returns last-position logits [B, V]."""
        h = self._run(F.embedding(input_ids, self.m.embed_tokens), use_fused)
        return lin(h[:, -1], self.m.lm_head)

    # -- decode with the position on the device --------------------------------------------------------------------
    def device_step_supported(self) -> bool:
        cfg, m = self.m.cfg, self.m
        if not m.embed_tokens.is_cuda or m.dtype != torch.bfloat16 or os.environ.get("TYR_DECODE_GRAPH", "1") == "0":
            return False
        if m.ep is not None and not m.ep.fused:
            return False          # the collective fallback runs host-side collectives
        return all(da.geometry_supported(cfg.heads(i), cfg.num_key_value_heads, cfg.head_dim) for i in range(cfg.num_hidden_layers))

    def _device_step(self, tokens: torch.Tensor, use_fused: bool = True) -> torch.Tensor:
        """One decode step whose only position input is ``self.pos_t``; advances ``pos_t`` (graph body)."""
        cfg = self.m.cfg
        x = F.embedding(tokens.reshape(self.batch, 1), self.m.embed_tokens)
        if self.m.ep is not None and len(self.m.layers) % 2:
            self.m.ep._sync(0)    # odd depth: the first layer of a replay reuses the exchange buffers of the last layer before it
        layers = self.m.layers
        h1 = norm_w(x, layers[0].input_layernorm, cfg.rms_norm_eps)
        for i, layer in enumerate(layers):
            next_norm = layers[i + 1].input_layernorm if i + 1 < len(layers) else self.m.norm
            x, h1 = layer_decode(cfg, i, layer, x, h1, next_norm, self.tables, self.pos_t, self.caches[i], use_fused, self.m.ep)
        logits = lin(h1[:, -1], self.m.lm_head)
        self.pos_t += 1
        return logits

    def _advance_host(self):
        self.pos += 1
        for c in self.caches:
            c.length += 1

    def step(self, tokens: torch.Tensor, use_fused: bool = True) -> torch.Tensor:
        if self.pos == 0 or not use_fused or not self.device_step_supported():
            h = self._run(F.embedding(tokens.reshape(self.batch, 1), self.m.embed_tokens), use_fused)
            return lin(h[:, -1], self.m.lm_head)
        if self.pos + 1 > self.max_len:
            raise ValueError("Laguna cache overflow")
        if getattr(self, "pos_t", None) is None:
            self.pos_t = torch.zeros(1, dtype=torch.int32, device=self.m.device)
            self._graph = None
        if self._graph is None:
            from ..utils.graph import GraphedStep
            self.pos_t.fill_(self.pos)
            self._graph = GraphedStep(self._device_step, (tokens.reshape(self.batch).clone(),), advancing_state=(self.pos_t,))
        elif self._pos_t_host != self.pos:
            self.pos_t.fill_(self.pos)
        out = self._graph(tokens.reshape(self.batch))
        self._advance_host()
        self._pos_t_host = self.pos
        return out


def generate(m: LagunaForCausalLM, input_ids: torch.Tensor, max_new_tokens: int = 256,
             strategy: SamplingStrategy = SamplingStrategy(), eos_token_ids: Optional[Sequence[int]] = None,
             on_step: Optional[StreamCallback] = None, use_fused: bool = True, generator=None) -> torch.Tensor:
    if input_ids.shape[1] == 0:
        raise ValueError("generate requires non-empty prompt sequence")
    if max_new_tokens == 0:
        return input_ids
    eos = m.cfg.eos_token_ids if eos_token_ids is None else eos_token_ids
    sess = CacheSession(m, input_ids.shape[0], input_ids.shape[1] + max_new_tokens)
    return generate_cached(lambda ids: sess.prefill(ids, use_fused), lambda t: sess.step(t, use_fused), input_ids,
                           max_new_tokens, strategy, eos, on_step, generator)


def generate_stream(m, input_ids, on_step, max_new_tokens=256, strategy=SamplingStrategy(), eos_token_ids=None):
    return generate(m, input_ids, max_new_tokens, strategy, eos_token_ids, on_step)


def generate_greedy(m, input_ids, max_new_tokens=256, eos_token_ids=None):
    return generate(m, input_ids, max_new_tokens, SamplingStrategy.greedy(), eos_token_ids)


# ---- weights -------------------------------------------------------------------------------------------------------------
def name_candidates(name: str) -> List[str]:
    """Accepted spellings of a checkpoint key (plain, ``language_model.`` and ``model.language_model.`` prefixes)."""
    out = [name, f"language_model.{name}", f"model.language_model.{name}"]
    if name.startswith("model."):
        suffix = name[len("model."):]
        out += [f"model.language_model.{suffix}", f"language_model.{suffix}"]
    seen, uniq = set(), []
    for n in out:
        if n not in seen:
            seen.add(n)
            uniq.append(n)
    return uniq


def load(cfg: LagunaConfig, source, device="cpu", dtype=torch.bfloat16, log=None) -> LagunaForCausalLM:
    """Load from a safetensors ``Source`` (file, sharded directory): Weights.lean:80-321."""
    src = source if isinstance(source, st.Source) else st.Source.open(source)
    info = log or (lambda s: None)

    def get(name, shape=None, dt=dtype):
        t = src.load(src.resolve(*name_candidates(name)))
        if shape is not None and tuple(t.shape) != tuple(shape):
            raise st.SafeTensorsError(f"{name}: expected shape {list(shape)}, got {list(t.shape)}")
        return t.to(device=device, dtype=dt) if dt is not None else t.to(device)

    def find(name):
        for c in name_candidates(name):
            if src.find(c) is not None:
                return c
        return None
    h, D, Hkv = cfg.hidden_size, cfg.head_dim, cfg.num_key_value_heads
    info("Loading LagunaForCausalLM...")
    emb = get("model.embed_tokens.weight", (cfg.vocab_size, h))
    layers = []
    for i in range(cfg.num_hidden_layers):
        p, H = f"model.layers.{i}.self_attn", cfg.heads(i)
        attn = Attention(get(f"{p}.q_proj.weight", (H * D, h)), get(f"{p}.k_proj.weight", (Hkv * D, h)),
                         get(f"{p}.v_proj.weight", (Hkv * D, h)), get(f"{p}.o_proj.weight", (h, H * D)),
                         get(f"{p}.g_proj.weight", (H, h)), get(f"{p}.q_norm.weight", (D,)), get(f"{p}.k_norm.weight", (D,)))
        p = f"model.layers.{i}.mlp"
        if cfg.is_moe_layer(i):
            E, mi, si = cfg.num_experts, cfg.moe_intermediate_size, cfg.shared_expert_intermediate_size
            bias_name = find(f"{p}.gate.e_score_correction_bias") or find(f"{p}.experts.e_score_correction_bias")
            router = Router(get(f"{p}.gate.weight", (E, h), torch.float32),
                            src.load(bias_name).to(device=device, dtype=torch.float32) if bias_name else None)
            shared = [get(f"{p}.shared_expert.gate_proj.weight", (si, h)), get(f"{p}.shared_expert.up_proj.weight", (si, h)),
                      get(f"{p}.shared_expert.down_proj.weight", (h, si))]
            gu_name = find(f"{p}.experts.gate_up_proj")
            if gu_name is not None:
                gu = src.load(gu_name).to(device=device, dtype=dtype)        # [E, 2*mi, h]
                down = get(f"{p}.experts.down_proj", (E, h, mi))
                de = DenseExperts(gu[:, :mi].contiguous(), gu[:, mi:].contiguous(), down)
                ffn = SparseMoeBlock(router, None, *shared, dense_experts=de)
            else:
                banks = {}
                for proj, rows, cols in (("gate", mi, h), ("up", mi, h), ("down", h, mi)):
                    pk = torch.empty((E, rows, cols // 2), dtype=torch.uint8, device=device)
                    sc = torch.empty((E, rows, cols // 16), dtype=torch.float8_e4m3fn, device=device)
                    gl = torch.empty(E, dtype=torch.float32, device=device)
                    for e in range(E):
                        ep = f"{p}.experts.{e}.{proj}_proj"
                        pk[e] = get(f"{ep}.weight_packed", (rows, cols // 2), None)
                        sc[e] = get(f"{ep}.weight_scale", (rows, cols // 16), None)
                        gl[e] = get(f"{ep}.weight_global_scale", (), torch.float32)
                    banks[proj] = (pk, sc, gl)
                ex = moe_ops.PackedExperts(*banks["gate"], *banks["up"], *banks["down"])
                ex.validate()
                ffn = SparseMoeBlock(router, ex, *shared)
        else:
            I = cfg.intermediate_size
            ffn = DenseMLP(get(f"{p}.gate_proj.weight", (I, h)), get(f"{p}.up_proj.weight", (I, h)), get(f"{p}.down_proj.weight", (h, I)))
        lp = f"model.layers.{i}"
        layers.append(Layer(get(f"{lp}.input_layernorm.weight", (h,)), attn, get(f"{lp}.post_attention_layernorm.weight", (h,)), ffn))
        info(f"  loaded layers {i + 1}/{cfg.num_hidden_layers}")
    norm = get("model.norm.weight", (h,))
    head_name = find("lm_head.weight")
    if head_name is None:
        info("  lm_head.weight not found; tying to embeddings.")
        return LagunaForCausalLM(cfg, emb, layers, norm, emb, True)
    return LagunaForCausalLM(cfg, emb, layers, norm, src.load(head_name).to(device=device, dtype=dtype), False)


def load_pretrained(model_dir: str, device="cpu", dtype=torch.bfloat16, log=None) -> LagunaForCausalLM:
    return load(LagunaConfig.load_from_pretrained_dir(model_dir), model_dir, device, dtype, log)


def state_dict(m: LagunaForCausalLM) -> Dict[str, torch.Tensor]:
    """Checkpoint-format names (inverse of ``load``); used by fixtures and export."""
    out = {"model.embed_tokens.weight": m.embed_tokens, "model.norm.weight": m.norm}
    if not m.tie_word_embeddings:
        out["lm_head.weight"] = m.lm_head
    for i, l in enumerate(m.layers):
        p = f"model.layers.{i}"
        out[f"{p}.input_layernorm.weight"] = l.input_layernorm
        out[f"{p}.post_attention_layernorm.weight"] = l.post_attention_layernorm
        for n in ("q_proj", "k_proj", "v_proj", "o_proj", "g_proj"):
            out[f"{p}.self_attn.{n}.weight"] = getattr(l.attn, n)
        out[f"{p}.self_attn.q_norm.weight"], out[f"{p}.self_attn.k_norm.weight"] = l.attn.q_norm, l.attn.k_norm
        f = l.ffn
        if isinstance(f, DenseMLP):
            for n in ("gate_proj", "up_proj", "down_proj"):
                out[f"{p}.mlp.{n}.weight"] = getattr(f, n)
            continue
        out[f"{p}.mlp.gate.weight"] = f.router.weight
        if f.router.e_score_correction_bias is not None:
            out[f"{p}.mlp.gate.e_score_correction_bias"] = f.router.e_score_correction_bias
        for n in ("gate", "up", "down"):
            out[f"{p}.mlp.shared_expert.{n}_proj.weight"] = getattr(f, f"shared_{n}_proj")
        if f.dense_experts is not None:
            out[f"{p}.mlp.experts.gate_up_proj"] = torch.cat([f.dense_experts.gate_proj, f.dense_experts.up_proj], 1)
            out[f"{p}.mlp.experts.down_proj"] = f.dense_experts.down_proj
        else:
            ex = f.experts
            for e in range(ex.num_experts):
                for n in ("gate", "up", "down"):
                    ep = f"{p}.mlp.experts.{e}.{n}_proj"
                    out[f"{ep}.weight_packed"] = getattr(ex, f"{n}_packed")[e]
                    out[f"{ep}.weight_scale"] = getattr(ex, f"{n}_scale")[e]
                    out[f"{ep}.weight_global_scale"] = getattr(ex, f"{n}_global")[e]
    return out
