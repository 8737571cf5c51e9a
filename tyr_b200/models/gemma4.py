"""Gemma 4 text model: sliding / full attention hybrid with different head geometry per kind, Q/K RMSNorm with
weights and V RMSNorm without, attention scale 1, K/V sharing for the last layers, per-layer input embeddings,
GELU-tanh MLP (optionally double-wide on shared layers), optional routed-experts branch, layer scalars and a
logit soft-cap (Tyr/Model/Gemma4/{Config,ConfigIO,Model,Weights}.lean)."""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..io import safetensors as st
from ..ops.attention import attention
from ..ops.norm import rms_norm_weighted
from .common import KVCache, apply_rotary_partial, cos_sin_tables, lin, plain_inv_freq
from .generation import SamplingStrategy, generate_cached

SLIDING, FULL = "sliding_attention", "full_attention"


def default_layer_types(n: int, interval: int = 6) -> List[str]:
    return [FULL if ((i + 1) % interval == 0 or i + 1 == n) else SLIDING for i in range(n)]


@dataclass
class Gemma4Config:
    vocab_size: int = 262144
    hidden_size: int = 2560
    intermediate_size: int = 10240
    num_hidden_layers: int = 42
    num_attention_heads: int = 8
    num_key_value_heads: int = 2
    num_global_key_value_heads: Optional[int] = None     # None: same as sliding layers
    half_head_dim: int = 128
    global_half_head_dim: Optional[int] = 256
    sliding_window: int = 512
    sliding_rope_theta: float = 10000.0
    full_rope_theta: float = 1000000.0
    half_full_rotary_dim: int = 64
    rms_norm_eps: float = 1e-6
    hidden_activation: str = "gelu_pytorch_tanh"
    attention_k_eq_v: bool = False
    use_bidirectional_attention: str = ""
    layer_types: Optional[List[str]] = None
    num_kv_shared_layers: int = 0
    use_double_wide_mlp: bool = False
    hidden_size_per_layer_input: int = 0
    vocab_size_per_layer_input: int = 262144
    enable_moe_block: bool = False
    num_experts: int = 0
    top_k_experts: int = 0
    moe_intermediate_size: int = 0
    tie_word_embeddings: bool = True
    final_logit_softcapping: Optional[float] = 30.0
    pad_token_id: Optional[int] = 0
    eos_token_id: Tuple[int, ...] = (1,)

    def __post_init__(self):
        if self.layer_types is None:
            self.layer_types = default_layer_types(self.num_hidden_layers)
        e = lambda m: ValueError(f"Invalid Gemma4 config: {m}")
        if self.num_attention_heads % self.num_key_value_heads or self.num_attention_heads % self.full_num_kv_heads:
            raise e("query heads must be whole multiples of the K/V heads of both layer kinds")
        if not (0 < self.half_full_rotary_dim <= self.full_half_head_dim):
            raise e("full layers must rotate a nonzero prefix of each head")
        if len(self.layer_types) != self.num_hidden_layers or (self.num_hidden_layers and self.layer_types[-1] != FULL):
            raise e("one attention kind per layer and the last layer must be full attention")
        if self.num_kv_shared_layers:
            first = self.first_kv_shared_layer
            if not (self.num_kv_shared_layers < self.num_hidden_layers and
                    all(self.layer_types[i] in self.layer_types[:first] for i in range(first, self.num_hidden_layers))):
                raise e("every KV-shared layer needs an earlier layer of its attention kind")
        if self.top_k_experts > self.num_experts or (self.enable_moe_block and not (self.top_k_experts > 0 and self.moe_intermediate_size > 0)):
            raise e("the router picks top_k_experts of num_experts and needs a nonzero expert MLP")
        if self.hidden_size_per_layer_input > 0 and self.vocab_size > self.vocab_size_per_layer_input:
            raise e("per-layer inputs must embed the same ids as the main embedding")
        if self.use_bidirectional_attention not in ("", "vision"):
            raise e("only vision tokens may attend bidirectionally")

    @property
    def head_dim(self): return 2 * self.half_head_dim
    @property
    def full_half_head_dim(self): return self.global_half_head_dim or self.half_head_dim
    @property
    def full_head_dim(self): return 2 * self.full_half_head_dim
    @property
    def full_num_kv_heads(self): return self.num_global_key_value_heads or self.num_key_value_heads
    @property
    def first_kv_shared_layer(self):
        return 0 if self.num_kv_shared_layers == 0 or self.num_kv_shared_layers >= self.num_hidden_layers else self.num_hidden_layers - self.num_kv_shared_layers

    def is_full(self, i): return self.layer_types[i] == FULL
    def is_kv_shared_layer(self, i): return self.num_kv_shared_layers > 0 and self.first_kv_shared_layer > 0 and i >= self.first_kv_shared_layer
    def layer_intermediate_size(self, i): return 2 * self.intermediate_size if self.use_double_wide_mlp and self.is_kv_shared_layer(i) else self.intermediate_size

    def shared_source_layer(self, i) -> Optional[int]:
        """The last non-shared layer of the same attention kind."""
        if not self.is_kv_shared_layer(i):
            return None
        src = None
        for j in range(self.first_kv_shared_layer):
            if self.layer_types[j] == self.layer_types[i]:
                src = j
        return src

    def geometry(self, i) -> Tuple[int, int]:
        """(kv heads, head dim) of layer ``i``."""
        return (self.full_num_kv_heads, self.full_head_dim) if self.is_full(i) else (self.num_key_value_heads, self.head_dim)

    @staticmethod
    def gemma4_e2b():
        return Gemma4Config(hidden_size=1536, intermediate_size=6144, num_hidden_layers=35, num_key_value_heads=1, layer_types=default_layer_types(35, 5),
                            num_kv_shared_layers=20, use_double_wide_mlp=True, hidden_size_per_layer_input=256)

    @staticmethod
    def from_json(j: dict) -> "Gemma4Config":
        j = j.get("text_config", j)
        d = Gemma4Config()
        n = j.get("num_hidden_layers", d.num_hidden_layers)
        head_dim = j.get("head_dim", d.head_dim)
        ghd = j.get("global_head_dim", None)
        rope = j.get("rope_parameters") or {}
        full = rope.get(FULL) or {}
        frac = full.get("partial_rotary_factor", j.get("partial_rotary_factor"))
        fhd = ghd or head_dim
        eos = j.get("eos_token_id", list(d.eos_token_id))
        g = lambda k: j.get(k, getattr(d, k))
        return Gemma4Config(g("vocab_size"), g("hidden_size"), g("intermediate_size"), n, g("num_attention_heads"), g("num_key_value_heads"),
                            j.get("num_global_key_value_heads"), head_dim // 2, (ghd // 2) if ghd else None, g("sliding_window"),
                            float((rope.get(SLIDING) or {}).get("rope_theta", j.get("rope_local_base_freq", d.sliding_rope_theta))),
                            float(full.get("rope_theta", j.get("rope_theta", d.full_rope_theta))),
                            int(round(fhd * frac)) // 2 if frac is not None else min(d.half_full_rotary_dim, fhd // 2), float(g("rms_norm_eps")),
                            g("hidden_activation"), bool(g("attention_k_eq_v")), j.get("use_bidirectional_attention") or "",
                            list(j.get("layer_types") or default_layer_types(n)), g("num_kv_shared_layers"), bool(g("use_double_wide_mlp")),
                            g("hidden_size_per_layer_input"), g("vocab_size_per_layer_input"), bool(g("enable_moe_block")), g("num_experts"),
                            g("top_k_experts"), g("moe_intermediate_size"), bool(g("tie_word_embeddings")), j.get("final_logit_softcapping", d.final_logit_softcapping),
                            j.get("pad_token_id", d.pad_token_id), tuple(eos) if isinstance(eos, list) else (int(eos),))

    @staticmethod
    def load_from_pretrained_dir(d: str) -> "Gemma4Config":
        with open(os.path.join(d, "config.json")) as f:
            return Gemma4Config.from_json(json.load(f))


@dataclass
class Attention:
    q_proj: torch.Tensor
    k_proj: torch.Tensor
    v_proj: Optional[torch.Tensor]
    o_proj: torch.Tensor
    q_norm: torch.Tensor
    k_norm: torch.Tensor


@dataclass
class MLP:
    gate_proj: torch.Tensor
    up_proj: torch.Tensor
    down_proj: torch.Tensor


@dataclass
class MoeBranch:
    router_proj: torch.Tensor           # [E, hidden] fp32
    router_scale: torch.Tensor          # [hidden]
    per_expert_scale: torch.Tensor      # [E]
    gate_up_proj: torch.Tensor          # [E, 2*mi, hidden]
    down_proj: torch.Tensor             # [E, hidden, mi]
    post_feedforward_layernorm_1: torch.Tensor
    post_feedforward_layernorm_2: torch.Tensor
    pre_feedforward_layernorm_2: torch.Tensor


@dataclass
class PerLayerInputBlock:
    per_layer_input_gate: torch.Tensor
    per_layer_projection: torch.Tensor
    post_per_layer_input_norm: torch.Tensor


@dataclass
class Layer:
    input_layernorm: torch.Tensor
    self_attn: Attention
    post_attention_layernorm: torch.Tensor
    pre_feedforward_layernorm: torch.Tensor
    mlp: MLP
    post_feedforward_layernorm: torch.Tensor
    layer_scalar: torch.Tensor
    moe: Optional[MoeBranch] = None
    per_layer_input: Optional[PerLayerInputBlock] = None


@dataclass
class Gemma4ForCausalLM:
    cfg: Gemma4Config
    embed_tokens: torch.Tensor
    layers: List[Layer]
    norm: torch.Tensor
    lm_head: torch.Tensor
    embed_tokens_per_layer: Optional[torch.Tensor] = None
    per_layer_model_projection: Optional[torch.Tensor] = None
    per_layer_projection_norm: Optional[torch.Tensor] = None

    @property
    def device(self): return self.embed_tokens.device
    @property
    def dtype(self): return self.embed_tokens.dtype


def rms(x, w, eps):
    return rms_norm_weighted(x, w, eps)


def rms_no_scale(x, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)


def gelu_tanh(x):
    return F.gelu(x, approximate="tanh")


def rotary_tables(cfg: Gemma4Config, max_len: int, device):
    sc, ss = cos_sin_tables(plain_inv_freq(cfg.half_head_dim, cfg.sliding_rope_theta), max_len, 1.0, device)
    fc, fs = cos_sin_tables(plain_inv_freq(cfg.full_half_head_dim, cfg.full_rope_theta), max_len, 1.0, device)
    r = cfg.half_full_rotary_dim
    fc = torch.cat([fc[:, :r], torch.ones_like(fc[:, r:])], 1)      # channels past the rotary prefix pass through
    fs = torch.cat([fs[:, :r], torch.zeros_like(fs[:, r:])], 1)
    return (sc, ss), (fc, fs)


def route(cfg: Gemma4Config, m: MoeBranch, hidden2: torch.Tensor):
    normed = rms_no_scale(hidden2, cfg.rms_norm_eps).float() * m.router_scale.float() * (cfg.hidden_size ** -0.5)
    probs = torch.softmax(F.linear(normed, m.router_proj.float()), -1)
    top, idx = torch.topk(probs, cfg.top_k_experts, dim=-1)
    w = top / top.sum(-1, keepdim=True) * m.per_expert_scale.float()[idx]
    return idx, w


def experts_forward(m: MoeBranch, x2: torch.Tensor, idx: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """GELU-gated routed experts: per unique expert, ``down(gelu_tanh(gate x) * up x)`` weighted into the token rows
    (the reference's fused expert loop, cc/src/tyr.cpp:1468-1546)."""
    if x2.is_cuda and x2.dtype == torch.bfloat16 and m.gate_up_proj.dtype == torch.bfloat16 and x2.shape[1] % 8 == 0 and (m.gate_up_proj.shape[1] // 2) % 8 == 0:
        # grouped tcgen05 GEMMs with the GELU gate in the epilogue; no host read of the expert ids
        from ..ops import moe as moe_ops
        return moe_ops.moe_dense_forward(x2, idx.to(torch.int32), w.float(), m.gate_up_proj, m.down_proj, act="geglu")
    out = torch.zeros_like(x2, dtype=torch.float32)
    mi = m.gate_up_proj.shape[1] // 2
    for e in torch.unique(idx).tolist():
        tok, slot = torch.nonzero(idx == e, as_tuple=True)
        xe = x2[tok]
        gu = lin(xe, m.gate_up_proj[e])
        h = gelu_tanh(gu[:, :mi]) * gu[:, mi:]
        out.index_add_(0, tok, lin(h, m.down_proj[e]).float() * w[tok, slot].unsqueeze(-1))
    return out.to(x2.dtype)


def attention_forward(cfg: Gemma4Config, i: int, a: Attention, x, rot, cache: Optional[KVCache], shared: Optional[KVCache],
                      edge_mask: Optional[torch.Tensor] = None):
    B, S, _ = x.shape
    H = cfg.num_attention_heads
    Hkv, D = cfg.geometry(i)
    cos, sin = rot
    q = rms(lin(x, a.q_proj[:H * D]).reshape(B, S, H, D), a.q_norm[:D], cfg.rms_norm_eps)
    q = apply_rotary_partial(q, cos, sin).transpose(1, 2) * math.sqrt(D)      # cancels the 1/sqrt(D) of SDPA: scale 1
    if shared is not None:
        k, v = shared.view()                                                   # K/V of the source layer, already written this step
    else:
        kr = lin(x, a.k_proj[:Hkv * D]).reshape(B, S, Hkv, D)
        vr = kr if (cfg.attention_k_eq_v and cfg.is_full(i)) or a.v_proj is None else lin(x, a.v_proj[:Hkv * D]).reshape(B, S, Hkv, D)
        k = apply_rotary_partial(rms(kr, a.k_norm[:D], cfg.rms_norm_eps), cos, sin).transpose(1, 2)
        v = rms_no_scale(vr, cfg.rms_norm_eps).transpose(1, 2)
        if cache is not None:
            cache.write(k, v)
            k, v = cache.view()
    window = None if cfg.is_full(i) else cfg.sliding_window
    Tk = k.shape[2]
    if edge_mask is not None:
        o = attention(q, k, v, causal=False, edge_mask=edge_mask)
    elif S == 1 and Tk > 1:
        if window is not None and Tk > window:
            k, v = k[:, :, -window:], v[:, :, -window:]
        o = attention(q, k, v, causal=False)
    else:
        o = attention(q, k, v, causal=True, window=window)
    return lin(o.transpose(1, 2).reshape(B, S, H * D), a.o_proj[:, :H * D])


def layer_forward(cfg, i, l: Layer, x, rot, cache, shared, per_layer_input=None, edge_mask=None):
    """``edge_mask``: one [B, S, S] mask for every layer, or a ``(sliding, full)`` pair chosen by the layer's kind."""
    B, S, h = x.shape
    if isinstance(edge_mask, (tuple, list)):
        edge_mask = edge_mask[1] if cfg.is_full(i) else edge_mask[0]
    eps = cfg.rms_norm_eps
    h2 = x + rms(attention_forward(cfg, i, l.self_attn, rms(x, l.input_layernorm, eps), rot, cache, shared, edge_mask), l.post_attention_layernorm, eps)
    h3 = rms(h2, l.pre_feedforward_layernorm, eps)
    I = cfg.layer_intermediate_size(i)
    mlp = lin(gelu_tanh(lin(h3, l.mlp.gate_proj[:I])) * lin(h3, l.mlp.up_proj[:I]), l.mlp.down_proj[:, :I])
    if l.moe is not None:
        dense = rms(mlp, l.moe.post_feedforward_layernorm_1, eps)
        r2 = h2.reshape(B * S, h)
        idx, w = route(cfg, l.moe, r2)
        ex = experts_forward(l.moe, rms(r2, l.moe.pre_feedforward_layernorm_2, eps), idx, w).reshape(B, S, h)
        mlp = dense + rms(ex, l.moe.post_feedforward_layernorm_2, eps)
    h4 = h2 + rms(mlp, l.post_feedforward_layernorm, eps)
    if l.per_layer_input is not None and per_layer_input is not None:
        blk = l.per_layer_input
        mixed = gelu_tanh(lin(h4, blk.per_layer_input_gate)) * per_layer_input
        h4 = h4 + rms(lin(mixed, blk.per_layer_projection), blk.post_per_layer_input_norm, eps)
    return h4 * l.layer_scalar.to(h4.dtype)


def embed_tokens(m: Gemma4ForCausalLM, ids):
    return F.embedding(ids, m.embed_tokens) * math.sqrt(m.cfg.hidden_size)


def compute_per_layer_inputs(m: Gemma4ForCausalLM, ids, embeds) -> Optional[torch.Tensor]:
    cfg = m.cfg
    if m.embed_tokens_per_layer is None or m.per_layer_model_projection is None:
        return None
    B, S = ids.shape
    P, L = cfg.hidden_size_per_layer_input, cfg.num_hidden_layers
    tok = (F.embedding(ids, m.embed_tokens_per_layer) * math.sqrt(P)).reshape(B, S, L, P)
    proj = (lin(embeds, m.per_layer_model_projection) * cfg.hidden_size ** -0.5).reshape(B, S, L, P)
    proj = rms(proj, m.per_layer_projection_norm, cfg.rms_norm_eps)
    return (proj + tok) * math.sqrt(0.5)


def cap_logits(cfg, logits):
    c = cfg.final_logit_softcapping
    return logits if c is None else torch.tanh(logits.float() / c) * c


class Gemma4Cache:
    """One KV cache per non-shared layer; shared layers read their source layer's cache (Model.lean:827, 1134-1148)."""

    def __init__(self, m: Gemma4ForCausalLM, batch: int, max_len: int):
        cfg = m.cfg
        self.m, self.pos, self.max_len = m, 0, max_len
        self.rot = rotary_tables(cfg, max_len, m.device)
        self.caches: List[Optional[KVCache]] = []
        for i in range(cfg.num_hidden_layers):
            if cfg.shared_source_layer(i) is not None:
                self.caches.append(None)
            else:
                Hkv, D = cfg.geometry(i)
                self.caches.append(KVCache.allocate(batch, Hkv, max_len, D, m.device, m.dtype))

    @torch.no_grad()
    def run(self, ids: torch.Tensor, embeds: Optional[torch.Tensor] = None, per_layer=None, edge_mask=None) -> torch.Tensor:
        """``edge_mask`` (prefill of an empty cache only) replaces the causal / window masks, e.g. to let the tokens of one
        image attend to each other in both directions."""
        m, cfg = self.m, self.m.cfg
        if edge_mask is not None and self.pos != 0:
            raise ValueError("edge masks apply to the prefill of an empty cache")
        x = embed_tokens(m, ids) if embeds is None else embeds
        S = x.shape[1]
        if self.pos + S > self.max_len:
            raise ValueError("Gemma4 cache overflow")
        pli = per_layer if per_layer is not None else (compute_per_layer_inputs(m, ids, x) if ids is not None else None)
        (sc, ss), (fc, fs) = self.rot
        sl = slice(self.pos, self.pos + S)
        for i, l in enumerate(m.layers):
            rot = (fc[sl], fs[sl]) if cfg.is_full(i) else (sc[sl], ss[sl])
            src = cfg.shared_source_layer(i)
            x = layer_forward(cfg, i, l, x, rot, self.caches[i], self.caches[src] if src is not None else None,
                              pli[:, :, i] if pli is not None else None, edge_mask)
        self.pos += S
        return cap_logits(cfg, lin(rms(x[:, -1], m.norm, cfg.rms_norm_eps), m.lm_head))

    def prefill(self, ids): return self.run(ids)
    def step(self, tok): return self.run(tok.reshape(-1, 1))


def forward(m: Gemma4ForCausalLM, ids: Optional[torch.Tensor] = None, embeds=None, per_layer_inputs=None, edge_mask=None) -> torch.Tensor:
    """Uncached logits [B, S, V].  ``edge_mask`` [B, S, S] (True = may attend) replaces the causal / window masks
    (bidirectional vision spans)."""
    cfg = m.cfg
    x = embed_tokens(m, ids) if embeds is None else embeds
    S = x.shape[1]
    pli = per_layer_inputs if per_layer_inputs is not None else (compute_per_layer_inputs(m, ids, x) if ids is not None else None)
    (sc, ss), (fc, fs) = rotary_tables(cfg, S, x.device)
    kv: Dict[int, KVCache] = {}
    for i, l in enumerate(m.layers):
        src = cfg.shared_source_layer(i)
        Hkv, D = cfg.geometry(i)
        c = None
        if src is None and any(cfg.shared_source_layer(j) == i for j in range(i + 1, cfg.num_hidden_layers)):
            c = kv[i] = KVCache.allocate(x.shape[0], Hkv, S, D, x.device, x.dtype)
        x = layer_forward(cfg, i, l, x, (fc, fs) if cfg.is_full(i) else (sc, ss), c, kv.get(src) if src is not None else None,
                          pli[:, :, i] if pli is not None else None, edge_mask)
    return cap_logits(cfg, lin(rms(x, m.norm, cfg.rms_norm_eps), m.lm_head))


def generate(m, input_ids, max_new_tokens=64, strategy=SamplingStrategy(), eos_token_ids=None, on_step=None):
    c = Gemma4Cache(m, input_ids.shape[0], input_ids.shape[1] + max_new_tokens)
    return generate_cached(c.prefill, c.step, input_ids, max_new_tokens, strategy, m.cfg.eos_token_id if eos_token_ids is None else eos_token_ids, on_step)


def generate_greedy(m, input_ids, max_new_tokens=64, eos_token_ids=None):
    return generate(m, input_ids, max_new_tokens, SamplingStrategy.greedy(), eos_token_ids)


def init(cfg: Gemma4Config, device="cpu", dtype=torch.float32, seed=0) -> Gemma4ForCausalLM:
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: (torch.randn(*s, generator=g) * s[-1] ** -0.5).to(device=device, dtype=dtype)
    ones = lambda n: torch.ones(n, device=device, dtype=dtype)
    h, H = cfg.hidden_size, cfg.num_attention_heads
    maxD = max(cfg.head_dim, cfg.full_head_dim)
    maxKV = max(cfg.num_key_value_heads, cfg.full_num_kv_heads) * maxD
    maxI = 2 * cfg.intermediate_size if cfg.use_double_wide_mlp else cfg.intermediate_size
    layers = []
    for i in range(cfg.num_hidden_layers):
        a = Attention(mk(H * maxD, h), mk(maxKV, h), None if cfg.attention_k_eq_v and cfg.is_full(i) else mk(maxKV, h), mk(h, H * maxD), ones(maxD), ones(maxD))
        moe = None
        if cfg.enable_moe_block:
            E, mi = cfg.num_experts, cfg.moe_intermediate_size
            moe = MoeBranch(mk(E, h).float(), torch.ones(h, device=device), torch.ones(E, device=device), mk(E, 2 * mi, h), mk(E, h, mi), ones(h), ones(h), ones(h))
        pli = PerLayerInputBlock(mk(cfg.hidden_size_per_layer_input, h), mk(h, cfg.hidden_size_per_layer_input), ones(h)) if cfg.hidden_size_per_layer_input else None
        layers.append(Layer(ones(h), a, ones(h), ones(h), MLP(mk(maxI, h), mk(maxI, h), mk(h, maxI)), ones(h), ones(1), moe, pli))
    emb = (torch.randn(cfg.vocab_size, h, generator=g) * 0.02).to(device=device, dtype=dtype)
    P, L = cfg.hidden_size_per_layer_input, cfg.num_hidden_layers
    return Gemma4ForCausalLM(cfg, emb, layers, ones(h), emb if cfg.tie_word_embeddings else mk(cfg.vocab_size, h),
                             (torch.randn(cfg.vocab_size_per_layer_input, L * P, generator=g) * 0.02).to(device=device, dtype=dtype) if P else None,
                             mk(L * P, h) if P else None, ones(P) if P else None)


def _pad_rows(t: torch.Tensor, rows: int) -> torch.Tensor:
    if t.shape[0] > rows:
        raise st.SafeTensorsError(f"Gemma4 weight of size {t.shape[0]} does not fit its padded size {rows}")
    return F.pad(t, (0, 0) * (t.dim() - 1) + (0, rows - t.shape[0])) if t.shape[0] < rows else t


def load(cfg: Gemma4Config, source, device="cpu", dtype=torch.bfloat16, log=None) -> Gemma4ForCausalLM:
    """Checkpoint names live under ``model.language_model.`` (also accepted: ``model.`` and ``language_model.``).  Layers of the
    smaller geometry are zero-padded to the larger one so that every layer has the same parameter shapes
    (Weights.lean:60-100); the forward slices the live part back out."""
    src = source if isinstance(source, st.Source) else st.Source.open(source)

    def find(suffix):
        for pre in ("model.language_model.", "model.", "language_model.", ""):
            if src.find(pre + suffix) is not None:
                return pre + suffix
        return None

    def get(suffix, required=True, dt=dtype):
        n = find(suffix)
        if n is None:
            if required:
                raise st.SafeTensorsError(f"missing tensor {suffix}")
            return None
        return src.load(n).to(device=device, dtype=dt)
    h, H = cfg.hidden_size, cfg.num_attention_heads
    maxD = max(cfg.head_dim, cfg.full_head_dim)
    maxKV = max(cfg.num_key_value_heads, cfg.full_num_kv_heads) * maxD
    maxI = 2 * cfg.intermediate_size if cfg.use_double_wide_mlp else cfg.intermediate_size
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"layers.{i}"
        v = get(f"{p}.self_attn.v_proj.weight", required=False)
        o = get(f"{p}.self_attn.o_proj.weight")
        a = Attention(_pad_rows(get(f"{p}.self_attn.q_proj.weight"), H * maxD), _pad_rows(get(f"{p}.self_attn.k_proj.weight"), maxKV),
                      _pad_rows(v, maxKV) if v is not None else None, F.pad(o, (0, H * maxD - o.shape[1])),
                      _pad_rows(get(f"{p}.self_attn.q_norm.weight"), maxD), _pad_rows(get(f"{p}.self_attn.k_norm.weight"), maxD))
        dn = get(f"{p}.mlp.down_proj.weight")
        mlp = MLP(_pad_rows(get(f"{p}.mlp.gate_proj.weight"), maxI), _pad_rows(get(f"{p}.mlp.up_proj.weight"), maxI), F.pad(dn, (0, maxI - dn.shape[1])))
        moe = None
        if cfg.enable_moe_block and find(f"{p}.router.proj.weight") is not None:
            moe = MoeBranch(get(f"{p}.router.proj.weight", dt=torch.float32), get(f"{p}.router.scale", dt=torch.float32),
                            get(f"{p}.router.per_expert_scale", dt=torch.float32), get(f"{p}.experts.gate_up_proj"), get(f"{p}.experts.down_proj"),
                            get(f"{p}.post_feedforward_layernorm_1.weight"), get(f"{p}.post_feedforward_layernorm_2.weight"),
                            get(f"{p}.pre_feedforward_layernorm_2.weight"))
        pli = None
        if cfg.hidden_size_per_layer_input and find(f"{p}.per_layer_input_gate.weight") is not None:
            pli = PerLayerInputBlock(get(f"{p}.per_layer_input_gate.weight"), get(f"{p}.per_layer_projection.weight"), get(f"{p}.post_per_layer_input_norm.weight"))
        sc = get(f"{p}.layer_scalar", required=False)
        layers.append(Layer(get(f"{p}.input_layernorm.weight"), a, get(f"{p}.post_attention_layernorm.weight"), get(f"{p}.pre_feedforward_layernorm.weight"),
                            mlp, get(f"{p}.post_feedforward_layernorm.weight"), sc.reshape(1) if sc is not None else torch.ones(1, device=device, dtype=dtype), moe, pli))
        if log:
            log(f"  loaded layers {i + 1}/{cfg.num_hidden_layers}")
    emb = get("embed_tokens.weight")
    head = get("lm_head.weight", required=False)
    return Gemma4ForCausalLM(cfg, emb, layers, get("norm.weight"), head if head is not None else emb, get("embed_tokens_per_layer.weight", required=False),
                             get("per_layer_model_projection.weight", required=False), get("per_layer_projection_norm.weight", required=False))


def state_dict(m: Gemma4ForCausalLM) -> Dict[str, torch.Tensor]:
    cfg, P = m.cfg, "model.language_model."
    out = {P + "embed_tokens.weight": m.embed_tokens, P + "norm.weight": m.norm}
    if m.lm_head is not m.embed_tokens:
        out[P + "lm_head.weight"] = m.lm_head
    for n in ("embed_tokens_per_layer", "per_layer_model_projection", "per_layer_projection_norm"):
        if getattr(m, n) is not None:
            out[f"{P}{n}.weight"] = getattr(m, n)
    for i, l in enumerate(m.layers):
        p = f"{P}layers.{i}"
        Hkv, D = cfg.geometry(i)
        H, I = cfg.num_attention_heads, cfg.layer_intermediate_size(i)
        a = l.self_attn
        out[f"{p}.self_attn.q_proj.weight"], out[f"{p}.self_attn.k_proj.weight"] = a.q_proj[:H * D], a.k_proj[:Hkv * D]
        if a.v_proj is not None:
            out[f"{p}.self_attn.v_proj.weight"] = a.v_proj[:Hkv * D]
        out[f"{p}.self_attn.o_proj.weight"] = a.o_proj[:, :H * D]
        out[f"{p}.self_attn.q_norm.weight"], out[f"{p}.self_attn.k_norm.weight"] = a.q_norm[:D], a.k_norm[:D]
        out[f"{p}.mlp.gate_proj.weight"], out[f"{p}.mlp.up_proj.weight"], out[f"{p}.mlp.down_proj.weight"] = l.mlp.gate_proj[:I], l.mlp.up_proj[:I], l.mlp.down_proj[:, :I]
        for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
            out[f"{p}.{n}.weight"] = getattr(l, n)
        out[f"{p}.layer_scalar"] = l.layer_scalar
        if l.moe is not None:
            mo = l.moe
            out[f"{p}.router.proj.weight"], out[f"{p}.router.scale"], out[f"{p}.router.per_expert_scale"] = mo.router_proj, mo.router_scale, mo.per_expert_scale
            out[f"{p}.experts.gate_up_proj"], out[f"{p}.experts.down_proj"] = mo.gate_up_proj, mo.down_proj
            for n in ("post_feedforward_layernorm_1", "post_feedforward_layernorm_2", "pre_feedforward_layernorm_2"):
                out[f"{p}.{n}.weight"] = getattr(mo, n)
        if l.per_layer_input is not None:
            b = l.per_layer_input
            out[f"{p}.per_layer_input_gate.weight"], out[f"{p}.per_layer_projection.weight"], out[f"{p}.post_per_layer_input_norm.weight"] = \
                b.per_layer_input_gate, b.per_layer_projection, b.post_per_layer_input_norm
    return out
