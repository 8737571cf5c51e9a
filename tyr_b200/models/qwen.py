"""Qwen3 blocks, base model, causal LM, Flux text embedder and the Qwen2.5-Omni thinker mapping.

Contract: Tyr/Model/Qwen/{Config,Attention,MLP,Layer,RoPE,Model,Embedder,Weights}.lean,
Tyr/Model/Qwen3/{Config,ConfigIO,Model,Weights}.lean, Tyr/Model/Qwen25Omni/{Weights,Pretrained}.lean.
GQA attention with optional per-head q/k RMSNorm, full-width HF rotate-half RoPE, SwiGLU MLP.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from ..io import safetensors as st
from ..ops.attention import attention
from .common import KVCache, apply_rotary_partial, cached_attention, cos_sin_tables, head_norm, lin, norm_w, plain_inv_freq, swiglu_mlp
from .generation import SamplingStrategy, generate_cached


@dataclass
class QwenConfig:
    """Defaults are Qwen3-4B (Qwen/Config.lean:14-45)."""
    vocab_size: int = 151936
    hidden_size: int = 2560
    intermediate_size: int = 6912
    num_hidden_layers: int = 28
    num_attention_heads: int = 20
    num_key_value_heads: int = 4
    half_head_dim: int = 64
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = True
    eos_token_ids: tuple = (151645, 151643)

    def __post_init__(self):
        if not (self.num_attention_heads > 0 and self.num_key_value_heads > 0
                and self.num_attention_heads % self.num_key_value_heads == 0):
            raise ValueError("Invalid Qwen config: query heads must form whole groups over the K/V heads")
        if self.half_head_dim <= 0 or self.vocab_size <= 0 or self.rope_theta <= 0 or self.rms_norm_eps <= 0:
            raise ValueError("Invalid Qwen config: head_dim, vocab_size, rope_theta and rms_norm_eps must be positive")

    @property
    def head_dim(self) -> int:
        return 2 * self.half_head_dim

    @staticmethod
    def qwen3_4b() -> "QwenConfig":
        return QwenConfig()

    @staticmethod
    def flux_klein_text_encoder() -> "QwenConfig":
        return QwenConfig(intermediate_size=9728, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
                          rope_theta=1000000.0)

    @staticmethod
    def from_json(j: dict, defaults: Optional["QwenConfig"] = None) -> "QwenConfig":
        d = defaults or QwenConfig()
        j = j.get("text_config", j)
        heads = j.get("num_attention_heads", d.num_attention_heads)
        hidden = j.get("hidden_size", d.hidden_size)
        head_dim = j.get("head_dim", hidden // heads if "hidden_size" in j and "head_dim" not in j else d.head_dim)
        if head_dim % 2:
            raise ValueError(f"Invalid Qwen config: head_dim={head_dim} must be even")
        eos = j.get("eos_token_id", list(d.eos_token_ids))
        return QwenConfig(vocab_size=j.get("vocab_size", d.vocab_size), hidden_size=hidden,
                          intermediate_size=j.get("intermediate_size", d.intermediate_size),
                          num_hidden_layers=j.get("num_hidden_layers", d.num_hidden_layers), num_attention_heads=heads,
                          num_key_value_heads=j.get("num_key_value_heads", d.num_key_value_heads),
                          half_head_dim=head_dim // 2, rope_theta=float(j.get("rope_theta", d.rope_theta)),
                          rms_norm_eps=float(j.get("rms_norm_eps", d.rms_norm_eps)),
                          tie_word_embeddings=bool(j.get("tie_word_embeddings", d.tie_word_embeddings)),
                          eos_token_ids=tuple(eos) if isinstance(eos, list) else (int(eos),))

    @staticmethod
    def load_from_pretrained_dir(model_dir: str, defaults: Optional["QwenConfig"] = None) -> "QwenConfig":
        with open(os.path.join(model_dir, "config.json")) as f:
            return QwenConfig.from_json(json.load(f), defaults)


@dataclass
class RoPECache:
    cos: torch.Tensor   # [max_seq, half_head_dim] fp32
    sin: torch.Tensor

    @staticmethod
    def init(max_seq: int, half_head_dim: int, theta: float, device="cpu") -> "RoPECache":
        c, s = cos_sin_tables(plain_inv_freq(half_head_dim, theta), max_seq, 1.0, device)
        return RoPECache(c, s)

    def rows(self, start: int, n: int):
        if start + n > self.cos.shape[0]:
            raise ValueError("RoPE cache does not cover the requested positions")
        return self.cos[start:start + n], self.sin[start:start + n]


@dataclass
class QwenAttention:
    q_proj: torch.Tensor
    k_proj: torch.Tensor
    v_proj: torch.Tensor
    o_proj: torch.Tensor
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    q_bias: Optional[torch.Tensor] = None
    k_bias: Optional[torch.Tensor] = None
    v_bias: Optional[torch.Tensor] = None


@dataclass
class QwenMLP:
    gate_proj: torch.Tensor
    up_proj: torch.Tensor
    down_proj: torch.Tensor


@dataclass
class QwenLayer:
    input_layernorm: torch.Tensor
    self_attn: QwenAttention
    post_attention_layernorm: torch.Tensor
    mlp: QwenMLP


@dataclass
class Qwen3Model:
    cfg: QwenConfig
    embed_tokens: torch.Tensor
    layers: List[QwenLayer]
    norm: torch.Tensor


def attention_forward(cfg: QwenConfig, a: QwenAttention, x, cos, sin, cache: Optional[KVCache] = None,
                      key_padding_mask=None, causal: bool = True):
    B, S, _ = x.shape
    H, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    q = lin(x, a.q_proj, a.q_bias).reshape(B, S, H, D)
    k = lin(x, a.k_proj, a.k_bias).reshape(B, S, Hkv, D)
    v = lin(x, a.v_proj, a.v_bias).reshape(B, S, Hkv, D).transpose(1, 2)
    if a.q_norm is not None:
        q = head_norm(q, a.q_norm, cfg.rms_norm_eps)
    if a.k_norm is not None:
        k = head_norm(k, a.k_norm, cfg.rms_norm_eps)
    q = apply_rotary_partial(q, cos, sin).transpose(1, 2)
    k = apply_rotary_partial(k, cos, sin).transpose(1, 2)
    if key_padding_mask is not None:
        o = attention(q, k, v, causal=causal, key_padding_mask=key_padding_mask)
    elif not causal:
        o = attention(q, k, v, causal=False)
    else:
        o = cached_attention(q, k, v, cache, None)
    return lin(o.transpose(1, 2).reshape(B, S, H * D), a.o_proj)


def layer_forward(cfg, l: QwenLayer, x, cos, sin, cache=None, key_padding_mask=None, causal=True):
    h = x + attention_forward(cfg, l.self_attn, norm_w(x, l.input_layernorm, cfg.rms_norm_eps), cos, sin, cache,
                              key_padding_mask, causal)
    return h + swiglu_mlp(norm_w(h, l.post_attention_layernorm, cfg.rms_norm_eps), l.mlp.gate_proj, l.mlp.up_proj, l.mlp.down_proj)


def forward_with_hidden_states(m: Qwen3Model, input_ids=None, cos=None, sin=None, attn_mask=None, inputs_embeds=None,
                               causal: bool = True) -> List[torch.Tensor]:
    """One hidden state per layer output plus the final normed state (Qwen/Model.lean:63-103)."""
    cfg = m.cfg
    h = F.embedding(input_ids, m.embed_tokens) if inputs_embeds is None else inputs_embeds
    if cos is None:
        rc = RoPECache.init(h.shape[1], cfg.half_head_dim, cfg.rope_theta, h.device)
        cos, sin = rc.cos, rc.sin
    states = []
    kpm = attn_mask.bool() if attn_mask is not None else None
    for l in m.layers:
        h = layer_forward(cfg, l, h, cos, sin, None, kpm, causal)
        states.append(h)
    states.append(norm_w(h, m.norm, cfg.rms_norm_eps))
    return states


def model_forward(m: Qwen3Model, input_ids=None, cos=None, sin=None, inputs_embeds=None) -> torch.Tensor:
    return forward_with_hidden_states(m, input_ids, cos, sin, None, inputs_embeds)[-1]


def _w(shape, fan_in, device, dtype, gen):
    return (torch.randn(shape, generator=gen) * fan_in ** -0.5).to(device=device, dtype=dtype)


def init_model(cfg: QwenConfig, device="cpu", dtype=torch.float32, seed=0, qk_norm: bool = True) -> Qwen3Model:
    gen = torch.Generator().manual_seed(seed)
    h, D, H, Hkv, I = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size
    ones = lambda n: torch.ones(n, device=device, dtype=dtype)
    layers = []
    for _ in range(cfg.num_hidden_layers):
        a = QwenAttention(_w((H * D, h), h, device, dtype, gen), _w((Hkv * D, h), h, device, dtype, gen),
                          _w((Hkv * D, h), h, device, dtype, gen), _w((h, H * D), H * D, device, dtype, gen),
                          ones(D) if qk_norm else None, ones(D) if qk_norm else None)
        mlp = QwenMLP(_w((I, h), h, device, dtype, gen), _w((I, h), h, device, dtype, gen), _w((h, I), I, device, dtype, gen))
        layers.append(QwenLayer(ones(h), a, ones(h), mlp))
    emb = (torch.randn((cfg.vocab_size, h), generator=gen) * 0.02).to(device=device, dtype=dtype)
    return Qwen3Model(cfg, emb, layers, ones(h))


# ---- causal LM -------------------------------------------------------------------------------------------
@dataclass
class Qwen3ForCausalLM:
    model: Qwen3Model
    lm_head: torch.Tensor
    tie_word_embeddings: bool = True

    @property
    def cfg(self):
        return self.model.cfg

    @staticmethod
    def init(cfg: QwenConfig, tie_word_embeddings: bool = True, device="cpu", dtype=torch.float32, seed=0) -> "Qwen3ForCausalLM":
        m = init_model(cfg, device, dtype, seed)
        head = m.embed_tokens if tie_word_embeddings else _w((cfg.vocab_size, cfg.hidden_size), cfg.hidden_size, device, dtype,
                                                            torch.Generator().manual_seed(seed + 1))
        return Qwen3ForCausalLM(m, head, tie_word_embeddings)

    def embed_tokens(self, ids):
        return F.embedding(ids, self.model.embed_tokens)

    def forward_embeds(self, embeds) -> torch.Tensor:
        return lin(model_forward(self.model, inputs_embeds=embeds), self.lm_head)

    def forward(self, input_ids) -> torch.Tensor:
        return self.forward_embeds(self.embed_tokens(input_ids))

    def forward_with_hidden_states(self, input_ids):
        hs = forward_with_hidden_states(self.model, input_ids)
        return lin(hs[-1], self.lm_head), hs


class Qwen3Session:
    """Per-layer static KV caches of ``max_len`` and a RoPE cache (Qwen3/Model.lean:126-195)."""

    def __init__(self, lm: Qwen3ForCausalLM, batch: int, max_len: int):
        cfg = lm.cfg
        dev, dt = lm.model.embed_tokens.device, lm.model.embed_tokens.dtype
        self.lm, self.pos, self.max_len = lm, 0, max_len
        self.rope = RoPECache.init(max_len, cfg.half_head_dim, cfg.rope_theta, dev)
        self.caches = [KVCache.allocate(batch, cfg.num_key_value_heads, max_len, cfg.head_dim, dev, dt)
                       for _ in range(cfg.num_hidden_layers)]

    @torch.no_grad()
    def run_embeds(self, h: torch.Tensor) -> torch.Tensor:
        cfg, S = self.lm.cfg, h.shape[1]
        cos, sin = self.rope.rows(self.pos, S)
        for l, c in zip(self.lm.model.layers, self.caches):
            h = layer_forward(cfg, l, h, cos, sin, c)
        self.pos += S
        return lin(norm_w(h[:, -1], self.lm.model.norm, cfg.rms_norm_eps), self.lm.lm_head)

    def prefill(self, ids):
        return self.run_embeds(self.lm.embed_tokens(ids))

    # -- decode with the position on the device: one CUDA graph replayed per token ------------------------------------
    def device_step_supported(self) -> bool:
        from ..ops.decode_attention import geometry_supported
        cfg, e = self.lm.cfg, self.lm.model.embed_tokens
        return (e.is_cuda and e.dtype == torch.bfloat16 and os.environ.get("TYR_DECODE_GRAPH", "1") != "0"
                and geometry_supported(cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim))

    def _device_step(self, tok: torch.Tensor) -> torch.Tensor:
        """One token per row; the only position input is ``self.pos_t`` (advanced here).  Per layer: RMSNorm(+RoPE) kernel on q and
        k, split-KV attention that also appends to the store, decode-sized linears."""
        from ..ops.decode_attention import decode_attention
        from ..ops.rope import rope_norm
        cfg, m = self.lm.cfg, self.lm.model
        H, Hkv, D, eps = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps
        x = self.lm.embed_tokens(tok.reshape(-1, 1))
        B = x.shape[0]
        positions = self.pos_t.expand(B)
        rot = 2 * self.rope.cos.shape[1]
        for l, c in zip(m.layers, self.caches):
            a = l.self_attn
            h1 = norm_w(x, l.input_layernorm, eps)
            q = rope_norm(lin(h1, a.q_proj, a.q_bias).reshape(B, H, D), self.rope.cos, self.rope.sin, weight=a.q_norm, positions=positions, rot=rot, eps=eps)
            k = rope_norm(lin(h1, a.k_proj, a.k_bias).reshape(B, Hkv, D), self.rope.cos, self.rope.sin, weight=a.k_norm, positions=positions, rot=rot, eps=eps)
            v = lin(h1, a.v_proj, a.v_bias).reshape(B, Hkv, D)
            o = decode_attention(q, k, v, c.k, c.v, self.pos_t)
            h = x + lin(o.reshape(B, 1, H * D), a.o_proj)
            x = h + swiglu_mlp(norm_w(h, l.post_attention_layernorm, eps), l.mlp.gate_proj, l.mlp.up_proj, l.mlp.down_proj)
        self.pos_t += 1
        return lin(norm_w(x[:, -1], m.norm, eps), self.lm.lm_head)

    def step(self, tok):
        if self.pos == 0 or not self.device_step_supported():
            return self.run_embeds(self.lm.embed_tokens(tok.reshape(-1, 1)))
        if self.pos + 1 > self.max_len:
            raise ValueError("Qwen3 cache overflow")
        if getattr(self, "_graph", None) is None:
            from ..utils.graph import GraphedStep
            self.pos_t = torch.full((1,), self.pos, dtype=torch.int32, device=self.lm.model.embed_tokens.device)
            self._graph = GraphedStep(self._device_step, (tok.reshape(-1).clone(),), advancing_state=(self.pos_t,))
        elif self._pos_t_host != self.pos:               # a multi-token run moved the position since the last replay
            self.pos_t.fill_(self.pos)
        out = self._graph(tok.reshape(-1))
        self.pos += 1
        self._pos_t_host = self.pos
        for c in self.caches:
            c.length += 1
        return out


def generate(lm: Qwen3ForCausalLM, input_ids, max_new_tokens=64, strategy=SamplingStrategy(), eos_token_ids=None, on_step=None):
    eos = lm.cfg.eos_token_ids if eos_token_ids is None else eos_token_ids
    s = Qwen3Session(lm, input_ids.shape[0], input_ids.shape[1] + max_new_tokens)
    return generate_cached(s.prefill, s.step, input_ids, max_new_tokens, strategy, eos, on_step)


def generate_greedy(lm, input_ids, max_new_tokens=64, eos_token_ids=None):
    return generate(lm, input_ids, max_new_tokens, SamplingStrategy.greedy(), eos_token_ids)


@torch.no_grad()
def generate_greedy_uncached(lm: Qwen3ForCausalLM, input_ids, max_new_tokens=64, eos_token_ids=None):
    """Recomputes the full sequence every step: the parity oracle of the cached path (Qwen3/Model.lean:314)."""
    ids = input_ids
    prefill = lambda x: lm.forward(x)[:, -1]

    def step(tok):
        nonlocal ids
        ids = torch.cat([ids, tok.reshape(-1, 1)], 1)
        return lm.forward(ids)[:, -1]
    eos = lm.cfg.eos_token_ids if eos_token_ids is None else eos_token_ids
    return generate_cached(prefill, step, input_ids, max_new_tokens, SamplingStrategy.greedy(), eos)


# ---- Flux text embedder --------------------------------------------------------------------------------------
@dataclass
class QwenFluxEmbedder:
    """Concatenates the hidden states of chosen layers (default 8, 17, 26 -> 3 * 2560 = 7680 channels)."""
    model: Qwen3Model
    rope: RoPECache
    output_layers: Sequence[int] = (8, 17, 26)

    @staticmethod
    def from_model(model: Qwen3Model, max_seq: int = 512, output_layers: Sequence[int] = (8, 17, 26)) -> "QwenFluxEmbedder":
        cfg = model.cfg
        return QwenFluxEmbedder(model, RoPECache.init(max_seq, cfg.half_head_dim, cfg.rope_theta, model.embed_tokens.device),
                                tuple(output_layers))

    def output_dim(self) -> int:
        return len(self.output_layers) * self.model.cfg.hidden_size

    @torch.no_grad()
    def encode(self, input_ids, attn_mask=None) -> torch.Tensor:
        S = input_ids.shape[1]
        cos, sin = self.rope.rows(0, S)
        hs = forward_with_hidden_states(self.model, input_ids, cos, sin, attn_mask)
        sel = [hs[i] for i in self.output_layers if i < len(hs)]
        if len(sel) != len(self.output_layers):
            raise ValueError(f"encode: output layers {list(self.output_layers)} exceed the {len(hs)} hidden states")
        return torch.cat(sel, dim=2).float()

    encode_masked = encode


# ---- weights ------------------------------------------------------------------------------------------------------
def _load_linear(src: st.Source, name: str, out_dim: int, in_dim: int, device, dtype, prefix_map=lambda n: n):
    """Plain weight, or FP8 block-quantised weight with ``weight_scale_inv`` [out/128, in/128] (Qwen/Weights.lean:29-43)."""
    w = src.load(prefix_map(f"{name}.weight"))
    if tuple(w.shape) != (out_dim, in_dim):
        raise st.SafeTensorsError(f"{name}.weight: expected shape [{out_dim}, {in_dim}], got {list(w.shape)}")
    sname = prefix_map(f"{name}.weight_scale_inv")
    if src.find(sname) is not None:
        if out_dim % 128 or in_dim % 128:
            raise st.SafeTensorsError(f"{name}.weight_scale_inv: FP8 block scales need dims divisible by 128, got [{out_dim}, {in_dim}]")
        s = src.load(sname).float()
        w = (w.float().reshape(out_dim // 128, 128, in_dim // 128, 128) * s[:, None, :, None]).reshape(out_dim, in_dim)
    return w.to(device=device, dtype=dtype)


def load_qwen3_model(cfg: QwenConfig, source, device="cpu", dtype=torch.bfloat16, log=None, name_map=lambda n: n) -> Qwen3Model:
    src = source if isinstance(source, st.Source) else st.Source.open(source)
    info = log or (lambda s: None)
    h, D, H, Hkv, I = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size

    def vec(name, n, required=True):
        nm = name_map(name)
        if src.find(nm) is None:
            if required:
                raise st.SafeTensorsError(f"missing tensor {nm}")
            return None
        t = src.load(nm)
        if tuple(t.shape) != (n,):
            raise st.SafeTensorsError(f"{nm}: expected shape [{n}], got {list(t.shape)}")
        return t.to(device=device, dtype=dtype)
    emb = src.load(name_map("model.embed_tokens.weight")).to(device=device, dtype=dtype)
    info("  Loaded embed_tokens")
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}.self_attn"
        a = QwenAttention(_load_linear(src, f"{p}.q_proj", H * D, h, device, dtype, name_map),
                          _load_linear(src, f"{p}.k_proj", Hkv * D, h, device, dtype, name_map),
                          _load_linear(src, f"{p}.v_proj", Hkv * D, h, device, dtype, name_map),
                          _load_linear(src, f"{p}.o_proj", h, H * D, device, dtype, name_map),
                          vec(f"{p}.q_norm.weight", D, False), vec(f"{p}.k_norm.weight", D, False),
                          vec(f"{p}.q_proj.bias", H * D, False), vec(f"{p}.k_proj.bias", Hkv * D, False),
                          vec(f"{p}.v_proj.bias", Hkv * D, False))
        p = f"model.layers.{i}.mlp"
        mlp = QwenMLP(_load_linear(src, f"{p}.gate_proj", I, h, device, dtype, name_map),
                      _load_linear(src, f"{p}.up_proj", I, h, device, dtype, name_map),
                      _load_linear(src, f"{p}.down_proj", h, I, device, dtype, name_map))
        layers.append(QwenLayer(vec(f"model.layers.{i}.input_layernorm.weight", h), a,
                                vec(f"model.layers.{i}.post_attention_layernorm.weight", h), mlp))
        info(f"  Loaded {i + 1}/{cfg.num_hidden_layers} layers")
    return Qwen3Model(cfg, emb, layers, vec("model.norm.weight", h))


def load_qwen3_causal_lm(cfg: QwenConfig, source, device="cpu", dtype=torch.bfloat16, log=None, name_map=lambda n: n) -> Qwen3ForCausalLM:
    src = source if isinstance(source, st.Source) else st.Source.open(source)
    m = load_qwen3_model(cfg, src, device, dtype, log, name_map)
    hn = name_map("lm_head.weight")
    if src.find(hn) is None:
        return Qwen3ForCausalLM(m, m.embed_tokens, True)
    return Qwen3ForCausalLM(m, src.load(hn).to(device=device, dtype=dtype), False)


def load_qwen_flux_embedder(source, cfg: Optional[QwenConfig] = None, max_seq: int = 512, device="cpu", dtype=torch.bfloat16,
                            output_layers=(8, 17, 26)) -> QwenFluxEmbedder:
    cfg = cfg or QwenConfig.flux_klein_text_encoder()
    return QwenFluxEmbedder.from_model(load_qwen3_model(cfg, source, device, dtype), max_seq, output_layers)


def load_from_pretrained(model_dir: str, device="cpu", dtype=torch.bfloat16) -> Qwen3ForCausalLM:
    return load_qwen3_causal_lm(QwenConfig.load_from_pretrained_dir(model_dir), model_dir, device, dtype)


def qwen25_omni_name_map(name: str) -> str:
    """Thinker text weights live under ``thinker.`` in Qwen2.5-Omni checkpoints (Qwen25Omni/Weights.lean)."""
    if name.startswith("model."):
        return "thinker." + name
    if name == "lm_head.weight":
        return "thinker.lm_head.weight"
    return name


def load_qwen25_omni_thinker(model_dir: str, device="cpu", dtype=torch.bfloat16) -> Qwen3ForCausalLM:
    with open(os.path.join(model_dir, "config.json")) as f:
        j = json.load(f)
    tj = (j.get("thinker_config") or j).get("text_config") or j
    cfg = QwenConfig.from_json(tj, QwenConfig(tie_word_embeddings=False))
    return load_qwen3_causal_lm(cfg, model_dir, device, dtype, name_map=qwen25_omni_name_map)


def state_dict(lm: Qwen3ForCausalLM) -> Dict[str, torch.Tensor]:
    m = lm.model
    out = {"model.embed_tokens.weight": m.embed_tokens, "model.norm.weight": m.norm}
    if not lm.tie_word_embeddings:
        out["lm_head.weight"] = lm.lm_head
    for i, l in enumerate(m.layers):
        p = f"model.layers.{i}"
        out[f"{p}.input_layernorm.weight"], out[f"{p}.post_attention_layernorm.weight"] = l.input_layernorm, l.post_attention_layernorm
        a = l.self_attn
        for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
            out[f"{p}.self_attn.{n}.weight"] = getattr(a, n)
        for n in ("q_norm", "k_norm"):
            if getattr(a, n) is not None:
                out[f"{p}.self_attn.{n}.weight"] = getattr(a, n)
        for n in ("q", "k", "v"):
            if getattr(a, f"{n}_bias") is not None:
                out[f"{p}.self_attn.{n}_proj.bias"] = getattr(a, f"{n}_bias")
        for n in ("gate_proj", "up_proj", "down_proj"):
            out[f"{p}.mlp.{n}.weight"] = getattr(l.mlp, n)
    return out
