"""Qwen3.5 / Qwen3.6 text models: hybrid of gated full attention and GatedDeltaNet linear attention,
dense SwiGLU or softmax-routed MoE FFN with a gated shared expert.

Contract: Tyr/Model/Qwen35/{Config,ConfigIO,Model,Weights,Pretrained}.lean, Tyr/Model/Qwen36/*.
Decode runs the fused recurrent delta-rule kernel (csrc/delta_rule.cu); prefill the chunked form;
MoE layers the grouped tcgen05 GEMM with the SwiGLU epilogue.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..io import safetensors as st
from ..ops import delta_rule as dr
from ..ops import moe as moe_ops
from ..ops.attention import attention
from ..ops.decode_attention import decode_attention, geometry_supported
from ..ops.rope import rope_norm
from .common import KVCache, apply_rotary_partial, cached_attention, cos_sin_tables, head_norm, lin, norm_w, plain_inv_freq, swiglu_mlp
from .generation import SamplingStrategy, generate_cached
from .laguna import name_candidates

LINEAR, FULL = "linear_attention", "full_attention"


def default_layer_types(n: int, interval: int = 4) -> List[str]:
    return [FULL if (i + 1) % interval == 0 else LINEAR for i in range(n)]


@dataclass
class Qwen35Config:
    vocab_size: int = 248320
    hidden_size: int = 4096
    intermediate_size: int = 12288
    num_hidden_layers: int = 32
    num_attention_heads: int = 16
    num_key_value_heads: int = 4
    head_dim: int = 256
    rope_theta: float = 1000000.0
    half_rotary_dim: int = 32
    rms_norm_eps: float = 1e-6
    linear_conv_kernel_dim: int = 4
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 32
    layer_types: Optional[List[str]] = None
    moe_intermediate_size: int = 512
    shared_expert_intermediate_size: int = 512
    num_experts_per_tok: int = 8
    num_experts: int = 0
    tie_word_embeddings: bool = False
    eos_token_id: Optional[int] = None

    def __post_init__(self):
        if self.layer_types is None:
            self.layer_types = default_layer_types(self.num_hidden_layers)
        e = lambda m: ValueError(f"Invalid Qwen3.5 config: {m}")
        if self.linear_num_value_heads % self.linear_num_key_heads:
            raise e("linear value heads must be a whole multiple of key heads")
        if self.num_attention_heads % self.num_key_value_heads:
            raise e("query heads must be a whole multiple of K/V heads")
        if not (0 < self.half_rotary_dim and 2 * self.half_rotary_dim <= self.head_dim):
            raise e("rotary dims must be a nonzero even prefix of the head")
        if len(self.layer_types) != self.num_hidden_layers:
            raise e(f"layer_types has {len(self.layer_types)} entries for {self.num_hidden_layers} layers")
        if any(t not in (LINEAR, FULL) for t in self.layer_types):
            raise e("layer_types entries must be linear_attention or full_attention")
        if self.linear_conv_kernel_dim <= 0 or self.linear_key_head_dim <= 0:
            raise e("conv kernel and key head dim must be positive")
        if self.num_experts > 0 and not (0 < self.num_experts_per_tok <= self.num_experts):
            raise e("num_experts_per_tok must be between 1 and num_experts")
        if self.eos_token_id is not None and self.eos_token_id >= self.vocab_size:
            raise e("eos_token_id must be below vocab_size")

    # derived dims (Config.lean linearKeyDim / linearValueDim / linearConvDim)
    @property
    def linear_key_dim(self): return self.linear_num_key_heads * self.linear_key_head_dim
    @property
    def linear_value_dim(self): return self.linear_num_value_heads * self.linear_value_head_dim
    @property
    def linear_conv_dim(self): return 2 * self.linear_key_dim + self.linear_value_dim
    @property
    def is_moe(self): return self.num_experts > 0

    def is_full(self, i): return self.layer_types[i] == FULL

    @staticmethod
    def qwen35_9b(): return Qwen35Config()

    @staticmethod
    def qwen35_0_8b():
        return Qwen35Config(hidden_size=1024, intermediate_size=3584, num_hidden_layers=24, num_attention_heads=8,
                            num_key_value_heads=2, rope_theta=10000000.0, linear_num_value_heads=16, tie_word_embeddings=True)

    @staticmethod
    def qwen35_27b():
        return Qwen35Config(hidden_size=5120, intermediate_size=17408, num_hidden_layers=64, num_attention_heads=24, num_key_value_heads=4,
                            linear_num_value_heads=48)

    @staticmethod
    def qwen35_35b_a3b():
        return Qwen35Config(hidden_size=2048, intermediate_size=0, num_hidden_layers=40, num_key_value_heads=2, num_experts=256)

    @staticmethod
    def qwen36_35b_a3b():
        return Qwen35Config(hidden_size=2048, intermediate_size=0, num_hidden_layers=40, num_key_value_heads=2, num_experts=256,
                            rope_theta=10000000.0, eos_token_id=248044)

    @staticmethod
    def from_json(j: dict, defaults: Optional["Qwen35Config"] = None) -> "Qwen35Config":
        d = defaults or Qwen35Config()
        j = j.get("text_config", j)
        n = j.get("num_hidden_layers", d.num_hidden_layers)
        lt = j.get("layer_types") or default_layer_types(n, j.get("full_attention_interval", 4))
        head_dim = j.get("head_dim", d.head_dim)
        rope = j.get("rope_parameters") or j.get("rope_scaling") or {}
        prf = j.get("partial_rotary_factor", rope.get("partial_rotary_factor"))
        half = d.half_rotary_dim if prf is None else int(round(head_dim * prf)) // 2
        eos = j.get("eos_token_id", d.eos_token_id)
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        g = lambda k: j.get(k, getattr(d, k))
        return Qwen35Config(vocab_size=g("vocab_size"), hidden_size=g("hidden_size"), intermediate_size=g("intermediate_size"),
                            num_hidden_layers=n, num_attention_heads=g("num_attention_heads"), num_key_value_heads=g("num_key_value_heads"),
                            head_dim=head_dim, rope_theta=float(j.get("rope_theta", rope.get("rope_theta", d.rope_theta))),
                            half_rotary_dim=half, rms_norm_eps=float(g("rms_norm_eps")), linear_conv_kernel_dim=g("linear_conv_kernel_dim"),
                            linear_key_head_dim=g("linear_key_head_dim"), linear_value_head_dim=g("linear_value_head_dim"),
                            linear_num_key_heads=g("linear_num_key_heads"), linear_num_value_heads=g("linear_num_value_heads"),
                            layer_types=list(lt), moe_intermediate_size=g("moe_intermediate_size"),
                            shared_expert_intermediate_size=g("shared_expert_intermediate_size"),
                            num_experts_per_tok=g("num_experts_per_tok"), num_experts=g("num_experts"),
                            tie_word_embeddings=bool(g("tie_word_embeddings")), eos_token_id=eos)

    @staticmethod
    def load_from_pretrained_dir(model_dir, defaults=None):
        with open(os.path.join(model_dir, "config.json")) as f:
            return Qwen35Config.from_json(json.load(f), defaults)


PRETRAINED_REPOS = ("Qwen/Qwen3.5-0.8B", "Qwen/Qwen3.5-9B", "Qwen/Qwen3.5-27B", "Qwen/Qwen3.5-35B-A3B", "Qwen/Qwen3.6-35B-A3B")


# ---- parameters --------------------------------------------------------------------------------------------
@dataclass
class Attention:
    q_proj: torch.Tensor      # [H*D*2, hidden]: per head q (D) then gate (D)
    k_proj: torch.Tensor
    v_proj: torch.Tensor
    o_proj: torch.Tensor
    q_norm: torch.Tensor      # zero-centred: scale = 1 + w
    k_norm: torch.Tensor


@dataclass
class GatedDeltaNet:
    in_proj_qkv: torch.Tensor
    in_proj_z: torch.Tensor
    in_proj_b: torch.Tensor
    in_proj_a: torch.Tensor
    conv1d_weight: torch.Tensor   # [conv_dim, 1, K]
    conv1d_bias: Optional[torch.Tensor]
    dt_bias: torch.Tensor         # fp32 [Hv]
    a_log: torch.Tensor           # fp32 [Hv]
    norm_weight: torch.Tensor     # [dv] (plain scale)
    out_proj: torch.Tensor


@dataclass
class MLP:
    gate_proj: torch.Tensor
    up_proj: torch.Tensor
    down_proj: torch.Tensor


@dataclass
class SparseMoeBlock:
    router: torch.Tensor          # [E, hidden]
    gate_up_proj: torch.Tensor    # [E, 2*mi, hidden]
    down_proj: torch.Tensor       # [E, hidden, mi]
    shared_expert: MLP
    shared_expert_gate: torch.Tensor   # [1, hidden]


@dataclass
class Layer:
    input_layernorm: torch.Tensor
    mixer: object                 # Attention | GatedDeltaNet
    post_attention_layernorm: torch.Tensor
    ffn: object                   # MLP | SparseMoeBlock


@dataclass
class Qwen35ForCausalLM:
    cfg: Qwen35Config
    embed_tokens: torch.Tensor
    layers: List[Layer]
    norm: torch.Tensor
    lm_head: torch.Tensor
    tie_word_embeddings: bool = False

    @property
    def device(self): return self.embed_tokens.device
    @property
    def dtype(self): return self.embed_tokens.dtype


def init(cfg: Qwen35Config, device="cpu", dtype=torch.float32, seed=0) -> Qwen35ForCausalLM:
    gen = torch.Generator().manual_seed(seed)
    mk = lambda shape, fan: (torch.randn(shape, generator=gen) * fan ** -0.5).to(device=device, dtype=dtype)
    zeros = lambda n: torch.zeros(n, device=device, dtype=dtype)
    h, D, H, Hkv = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    layers = []
    for i in range(cfg.num_hidden_layers):
        if cfg.is_full(i):
            mixer = Attention(mk((H * D * 2, h), h), mk((Hkv * D, h), h), mk((Hkv * D, h), h), mk((h, H * D), H * D), zeros(D), zeros(D))
        else:
            Hv, cd, vd, K = cfg.linear_num_value_heads, cfg.linear_conv_dim, cfg.linear_value_dim, cfg.linear_conv_kernel_dim
            a = torch.rand(Hv, generator=gen) * 16.0 + 1e-6
            mixer = GatedDeltaNet(mk((cd, h), h), mk((vd, h), h), mk((Hv, h), h), mk((Hv, h), h), mk((cd, 1, K), K),
                                  (torch.rand(cd, generator=gen) * 0.2 - 0.1).to(device=device, dtype=dtype),
                                  torch.ones(Hv, device=device), torch.log(a).to(device),
                                  torch.ones(cfg.linear_value_head_dim, device=device, dtype=dtype), mk((h, vd), vd))
        if cfg.is_moe:
            E, mi, si = cfg.num_experts, cfg.moe_intermediate_size, cfg.shared_expert_intermediate_size
            ffn = SparseMoeBlock(mk((E, h), h), mk((E, 2 * mi, h), h), mk((E, h, mi), mi),
                                 MLP(mk((si, h), h), mk((si, h), h), mk((h, si), si)), mk((1, h), h))
        else:
            I = cfg.intermediate_size
            ffn = MLP(mk((I, h), h), mk((I, h), h), mk((h, I), I))
        layers.append(Layer(zeros(h), mixer, zeros(h), ffn))
    emb = (torch.randn((cfg.vocab_size, h), generator=gen) * 0.02).to(device=device, dtype=dtype)
    head = emb if cfg.tie_word_embeddings else mk((cfg.vocab_size, h), h)
    return Qwen35ForCausalLM(cfg, emb, layers, zeros(h), head, cfg.tie_word_embeddings)


# ---- blocks ------------------------------------------------------------------------------------------------------
def rms(x, w, eps):
    """Zero-centred RMSNorm: ``norm(x) * (1 + w)``."""
    return norm_w(x, w, eps, one_plus_w=True)


def attention_core(cfg: Qwen35Config, q_norm, k_norm, qg, k, v, cos, sin, cache: Optional[KVCache], attn_mask=None):
    """Everything between the input and output projections of a gated full-attention layer.  ``qg``: [B, S, H*2D]
    (per head q then gate), ``k``/``v``: [B, S, Hkv*D]; head counts come from ``cfg`` (a tensor-parallel rank passes
    its local counts).  Returns [B, S, H*D]."""
    B, S, _ = qg.shape
    H, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    qg = qg.reshape(B, S, H, 2 * D)
    q, gate = qg[..., :D], qg[..., D:].reshape(B, S, H * D)
    k = k.reshape(B, S, Hkv, D)
    v = v.reshape(B, S, Hkv, D).transpose(1, 2)
    q = head_norm(q.contiguous(), q_norm, cfg.rms_norm_eps, one_plus_w=True)
    k = head_norm(k, k_norm, cfg.rms_norm_eps, one_plus_w=True)
    q = apply_rotary_partial(q, cos, sin).transpose(1, 2)
    k = apply_rotary_partial(k, cos, sin).transpose(1, 2)
    if attn_mask is not None:
        o = attention(q, k, v, causal=True, key_padding_mask=attn_mask.bool())
    else:
        o = cached_attention(q, k, v, cache, None)
    return o.transpose(1, 2).reshape(B, S, H * D) * torch.sigmoid(gate)


def attention_core_decode(cfg: Qwen35Config, q_norm, k_norm, qg, k, v, cos_table, sin_table, pos_t, cache: KVCache):
    """``attention_core`` for one new token per row with the position in the device tensor ``pos_t``: RMSNorm+RoPE kernel,
    then the split-KV kernel that also appends to the store.  ``cos_table`` / ``sin_table`` are the whole tables."""
    B = qg.shape[0]
    H, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    qg = qg.reshape(B, H, 2 * D)
    positions = pos_t.expand(B)
    rot = 2 * cos_table.shape[1]
    q = rope_norm(qg[..., :D], cos_table, sin_table, weight=q_norm, positions=positions, rot=rot, eps=cfg.rms_norm_eps, one_plus_w=True)
    kn = rope_norm(k.reshape(B, Hkv, D), cos_table, sin_table, weight=k_norm, positions=positions, rot=rot, eps=cfg.rms_norm_eps, one_plus_w=True)
    # the element-wise sigmoid gate is applied inside the attention kernel's final write
    o = decode_attention(q, kn, v.reshape(B, Hkv, D), cache.k, cache.v, pos_t, elem_gate=qg[..., D:])
    return o.reshape(B, 1, H * D)


def attention_forward(cfg: Qwen35Config, a: Attention, x, cos, sin, cache: Optional[KVCache], attn_mask=None):
    o = attention_core(cfg, a.q_norm, a.k_norm, lin(x, a.q_proj), lin(x, a.k_proj), lin(x, a.v_proj), cos, sin, cache, attn_mask)
    return lin(o, a.o_proj)


@dataclass
class LinearState:
    conv: Optional[torch.Tensor] = None        # [B, conv_dim, K] last K pre-conv inputs
    rec: Optional[torch.Tensor] = None         # fp32 [B, Hv, dk, dv]


def rms_norm_gated(x, gate, w, eps):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return (y * F.silu(gate.float())).to(x.dtype)


def gated_delta_net_core(cfg: Qwen35Config, m, mixed, z, b, a, state: Optional[LinearState] = None):
    """Causal depthwise conv + SiLU, gated delta rule and gated RMSNorm of one GatedDeltaNet layer, between its input
    and output projections.  ``mixed``: [B, S, conv_dim] (q | k | v channels), ``z``: [B, S, Hv*dv], ``b``/``a``: [B, S, Hv];
    head counts come from ``cfg``.  ``state`` (if given) is advanced in place; a one-token call on a state that already
    holds context takes the recurrent kernel (Model.lean:642-779).  Returns [B, S, Hv*dv]."""
    B, S, _ = mixed.shape
    K, cd = cfg.linear_conv_kernel_dim, cfg.linear_conv_dim
    Hk, Hv, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    z = z.reshape(B, S, Hv, dv)
    step = state is not None and state.conv is not None and S == 1
    if step and state.rec is not None and dr.gdn_decode_fused_supported(mixed, state.conv, state.rec, dk, dv):
        return dr.gdn_decode_fused(mixed, z, b, a, state.conv, m.conv1d_weight, m.conv1d_bias, m.dt_bias, m.a_log, m.norm_weight,
                                   cfg.rms_norm_eps, state.rec, Hk, Hv, dk, dv)
    w = m.conv1d_weight.reshape(cd, K).to(mixed.dtype)
    if step:
        window = torch.cat([state.conv[:, :, 1:], mixed.transpose(1, 2)], dim=2)       # [B, cd, K]
        y = (window.float() * w.float()).sum(-1)
        if m.conv1d_bias is not None:
            y = y + m.conv1d_bias.float()
        conv_out = F.silu(y).to(mixed.dtype).unsqueeze(1)                                 # [B, 1, cd]
        state.conv.copy_(window)                                                          # in place: the step is graph-replayable
    else:
        xc = mixed.transpose(1, 2)
        conv_out = dr.causal_conv1d_silu(mixed, m.conv1d_weight.reshape(cd, K), m.conv1d_bias)
        if state is not None:
            state.conv = (xc[:, :, S - K:] if S >= K else F.pad(xc, (K - S, 0))).contiguous()
    kd = cfg.linear_key_dim
    q = conv_out[..., :kd].reshape(B, S, Hk, dk)
    k = conv_out[..., kd:2 * kd].reshape(B, S, Hk, dk)
    v = conv_out[..., 2 * kd:].reshape(B, S, Hv, dv)
    beta = torch.sigmoid(b.float())
    g = -F.softplus(a.float() + m.dt_bias.float()) * torch.exp(m.a_log.float())
    rep = Hv // Hk
    if step and state.rec is not None:
        core = dr.gdr_decode_step(q.contiguous(), k.contiguous(), v.contiguous(), g, beta, state.rec)
    else:
        core, rec = dr.chunk_gated_delta_rule(q, k, v, g, beta, state=state.rec if state is not None else None)    # keys stay grouped
        if state is not None:
            state.rec = rec.contiguous()
    core = rms_norm_gated(core.reshape(B * S * Hv, dv), z.reshape(B * S * Hv, dv), m.norm_weight, cfg.rms_norm_eps)
    return core.reshape(B, S, Hv * dv)


def gated_delta_net_forward(cfg: Qwen35Config, m: GatedDeltaNet, x, state: Optional[LinearState] = None, attn_mask=None):
    if attn_mask is not None:
        x = x * attn_mask.to(x.dtype).unsqueeze(-1)
    core = gated_delta_net_core(cfg, m, lin(x, m.in_proj_qkv), lin(x, m.in_proj_z), lin(x, m.in_proj_b), lin(x, m.in_proj_a), state)
    return lin(core, m.out_proj)


def moe_forward(cfg: Qwen35Config, m: SparseMoeBlock, x2: torch.Tensor) -> torch.Tensor:
    """softmax router over all experts, top-k renormalised; gated shared expert added (Model.lean:162-292)."""
    logits = F.linear(x2, m.router.to(x2.dtype)).float()
    ids, w, counts = moe_ops.route(logits, cfg.num_experts_per_tok, softmax=True, renorm=True)
    shared = swiglu_mlp(x2, m.shared_expert.gate_proj, m.shared_expert.up_proj, m.shared_expert.down_proj)
    shared = (torch.sigmoid(F.linear(x2, m.shared_expert_gate.to(x2.dtype)).float()) * shared.float()).to(x2.dtype)
    return moe_ops.moe_dense_forward(x2, ids, w, m.gate_up_proj, m.down_proj, counts=counts, add=shared)


def layer_forward(cfg, i, layer: Layer, x, cos, sin, kv: Optional[KVCache], lin_state: Optional[LinearState], attn_mask=None):
    B, S, h = x.shape
    h1 = rms(x, layer.input_layernorm, cfg.rms_norm_eps)
    if cfg.is_full(i):
        mixed = attention_forward(cfg, layer.mixer, h1, cos, sin, kv, attn_mask)
    else:
        mixed = gated_delta_net_forward(cfg, layer.mixer, h1, lin_state, attn_mask)
    h2 = x + mixed
    h3 = rms(h2, layer.post_attention_layernorm, cfg.rms_norm_eps)
    if isinstance(layer.ffn, MLP):
        f = swiglu_mlp(h3, layer.ffn.gate_proj, layer.ffn.up_proj, layer.ffn.down_proj)
    else:
        f = moe_forward(cfg, layer.ffn, h3.reshape(B * S, h)).reshape(B, S, h)
    return h2 + f


def rope_tables(cfg: Qwen35Config, max_len: int, device):
    return cos_sin_tables(plain_inv_freq(cfg.half_rotary_dim, cfg.rope_theta), max_len, 1.0, device)


def forward_hidden(m: Qwen35ForCausalLM, input_ids=None, attn_mask=None, inputs_embeds=None) -> torch.Tensor:
    cfg = m.cfg
    x = F.embedding(input_ids, m.embed_tokens) if inputs_embeds is None else inputs_embeds
    cos, sin = rope_tables(cfg, x.shape[1], x.device)
    for i, l in enumerate(m.layers):
        x = layer_forward(cfg, i, l, x, cos, sin, None, None, attn_mask)
    return rms(x, m.norm, cfg.rms_norm_eps)


def forward(m: Qwen35ForCausalLM, input_ids=None, attn_mask=None, inputs_embeds=None) -> torch.Tensor:
    return lin(forward_hidden(m, input_ids, attn_mask, inputs_embeds), m.lm_head)


class HybridCache:
    """KV caches for full layers, conv + recurrent states for linear layers (Model.lean:784-860)."""

    def __init__(self, m: Qwen35ForCausalLM, batch: int, max_len: int):
        cfg = m.cfg
        self.m, self.pos, self.max_len, self.batch = m, 0, max_len, batch
        self.cos, self.sin = rope_tables(cfg, max_len, m.device)
        self.kv = [KVCache.allocate(batch, cfg.num_key_value_heads, max_len, cfg.head_dim, m.device, m.dtype) if cfg.is_full(i) else None
                   for i in range(cfg.num_hidden_layers)]
        self.lin = [None if cfg.is_full(i) else LinearState() for i in range(cfg.num_hidden_layers)]

    def state_bytes(self) -> int:
        n = sum(c.nbytes() for c in self.kv if c is not None)
        for s in self.lin:
            if s is not None:
                n += sum(t.numel() * t.element_size() for t in (s.conv, s.rec) if t is not None)
        return n

    @torch.no_grad()
    def run(self, x: torch.Tensor) -> torch.Tensor:
        cfg, S = self.m.cfg, x.shape[1]
        if self.pos + S > self.max_len:
            raise ValueError("Qwen3.5 cache overflow")
        cos, sin = self.cos[self.pos:self.pos + S], self.sin[self.pos:self.pos + S]
        for i, l in enumerate(self.m.layers):
            x = layer_forward(cfg, i, l, x, cos, sin, self.kv[i], self.lin[i])
        self.pos += S
        return lin(rms(x[:, -1], self.m.norm, cfg.rms_norm_eps), self.m.lm_head)

    def prefill(self, ids): return self.run(F.embedding(ids, self.m.embed_tokens))

    # -- decode with the position on the device (CUDA-graph body) ---------------------------------------------------
    def device_step_supported(self) -> bool:
        cfg, m = self.m.cfg, self.m
        return (m.embed_tokens.is_cuda and m.dtype == torch.bfloat16 and os.environ.get("TYR_DECODE_GRAPH", "1") != "0" and not cfg.is_moe
                and geometry_supported(cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim))

    def _device_step(self, tok: torch.Tensor) -> torch.Tensor:
        m, cfg = self.m, self.m.cfg
        eps = cfg.rms_norm_eps
        x = F.embedding(tok.reshape(-1, 1), m.embed_tokens)
        n_layers = len(m.layers)
        h1 = rms(x, m.layers[0].input_layernorm, eps)
        for i, l in enumerate(m.layers):
            if cfg.is_full(i):
                a = l.mixer
                o = attention_core_decode(cfg, a.q_norm, a.k_norm, lin(h1, a.q_proj), lin(h1, a.k_proj), lin(h1, a.v_proj), self.cos, self.sin,
                                          self.pos_t, self.kv[i])
                mixed = lin(o, a.o_proj)
            else:
                mixed = gated_delta_net_forward(cfg, l.mixer, h1, self.lin[i])
            # residual add and the next norm in one kernel: (normed, new residual stream)
            h3, h2 = norm_w(mixed, l.post_attention_layernorm, eps, one_plus_w=True, residual=x, return_residual=True)
            f = swiglu_mlp(h3, l.ffn.gate_proj, l.ffn.up_proj, l.ffn.down_proj) if isinstance(l.ffn, MLP) else \
                moe_forward(cfg, l.ffn, h3.reshape(-1, cfg.hidden_size)).reshape(h3.shape)
            next_w = m.layers[i + 1].input_layernorm if i + 1 < n_layers else m.norm
            h1, x = norm_w(f, next_w, eps, one_plus_w=True, residual=h2, return_residual=True)
        self.pos_t += 1
        return lin(h1[:, -1], m.lm_head)

    def _advance_host(self):
        self.pos += 1
        for c in self.kv:
            if c is not None:
                c.length += 1

    def step(self, tok):
        if self.pos == 0 or not self.device_step_supported():
            return self.run(F.embedding(tok.reshape(-1, 1), self.m.embed_tokens))
        if self.pos + 1 > self.max_len:
            raise ValueError("Qwen3.5 cache overflow")
        if getattr(self, "_graph", None) is None:
            from ..utils.graph import GraphedStep
            self.pos_t = torch.full((1,), self.pos, dtype=torch.int32, device=self.m.device)
            state = [self.pos_t] + [t for s in self.lin if s is not None for t in (s.conv, s.rec)]
            self._graph = GraphedStep(self._device_step, (tok.reshape(-1).clone(),), advancing_state=state)
        out = self._graph(tok.reshape(-1))
        self._advance_host()
        return out


def generate(m: Qwen35ForCausalLM, input_ids, max_new_tokens=64, strategy=SamplingStrategy(), eos_token_ids=None, on_step=None):
    eos = eos_token_ids if eos_token_ids is not None else (() if m.cfg.eos_token_id is None else (m.cfg.eos_token_id,))
    c = HybridCache(m, input_ids.shape[0], input_ids.shape[1] + max_new_tokens)
    return generate_cached(c.prefill, c.step, input_ids, max_new_tokens, strategy, eos, on_step)


def generate_greedy(m, input_ids, max_new_tokens=64, eos_token_ids=None):
    return generate(m, input_ids, max_new_tokens, SamplingStrategy.greedy(), eos_token_ids)


def generate_stream(m, input_ids, on_step, max_new_tokens=64, strategy=SamplingStrategy(), eos_token_ids=None):
    return generate(m, input_ids, max_new_tokens, strategy, eos_token_ids, on_step)


@torch.no_grad()
def generate_uncached(m: Qwen35ForCausalLM, input_ids, max_new_tokens=64, eos_token_ids=None):
    """Full recomputation each step; the cached/uncached parity reference (Model.lean:1403)."""
    ids = input_ids

    def step(tok):
        nonlocal ids
        ids = torch.cat([ids, tok.reshape(-1, 1)], 1)
        return forward(m, ids)[:, -1]
    eos = eos_token_ids if eos_token_ids is not None else (() if m.cfg.eos_token_id is None else (m.cfg.eos_token_id,))
    return generate_cached(lambda x: forward(m, x)[:, -1], step, input_ids, max_new_tokens, SamplingStrategy.greedy(), eos)


# ---- weights ----------------------------------------------------------------------------------------------------------
def load(cfg: Qwen35Config, source, device="cpu", dtype=torch.bfloat16, log=None) -> Qwen35ForCausalLM:
    src = source if isinstance(source, st.Source) else st.Source.open(source)
    info = log or (lambda s: None)

    def find(name):
        for c in name_candidates(name):
            if src.find(c) is not None:
                return c
        return None

    def linear_w(base, out_dim, in_dim, suffix=".weight"):
        n = find(base + suffix)
        if n is None:
            raise st.SafeTensorsError(f"Failed to load linear weight: {base}")
        w = src.load(n)
        sname = n[:-len(".weight")] + ".weight_scale_inv" if n.endswith(".weight") else n + "_scale_inv"
        if src.find(sname) is not None:
            s = src.load(sname).float()
            w = w.float()
            shp = w.shape
            w = (w.reshape(*shp[:-2], shp[-2] // 128, 128, shp[-1] // 128, 128) * s[..., :, None, :, None]).reshape(shp)
        if tuple(w.shape[-2:]) != (out_dim, in_dim):
            raise st.SafeTensorsError(f"{n}: expected trailing shape [{out_dim}, {in_dim}], got {list(w.shape)}")
        return w.to(device=device, dtype=dtype)

    def vec(base, n, dt=dtype, required=True):
        nm = find(base)
        if nm is None:
            if required:
                raise st.SafeTensorsError(f"missing tensor {base}")
            return None
        t = src.load(nm)
        if t.numel() != n and n is not None:
            raise st.SafeTensorsError(f"{nm}: expected {n} elements, got {list(t.shape)}")
        return t.to(device=device, dtype=dt)
    h, D, H, Hkv = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    emb = vec("model.embed_tokens.weight", cfg.vocab_size * h)
    layers = []
    for i in range(cfg.num_hidden_layers):
        lp = f"model.layers.{i}"
        if cfg.is_full(i):
            p = f"{lp}.self_attn"
            mixer = Attention(linear_w(f"{p}.q_proj", H * D * 2, h), linear_w(f"{p}.k_proj", Hkv * D, h), linear_w(f"{p}.v_proj", Hkv * D, h),
                              linear_w(f"{p}.o_proj", h, H * D), vec(f"{p}.q_norm.weight", D), vec(f"{p}.k_norm.weight", D))
        else:
            p = f"{lp}.linear_attn"
            Hv, cd, vd, K = cfg.linear_num_value_heads, cfg.linear_conv_dim, cfg.linear_value_dim, cfg.linear_conv_kernel_dim
            mixer = GatedDeltaNet(linear_w(f"{p}.in_proj_qkv", cd, h), linear_w(f"{p}.in_proj_z", vd, h), linear_w(f"{p}.in_proj_b", Hv, h),
                                  linear_w(f"{p}.in_proj_a", Hv, h), vec(f"{p}.conv1d.weight", cd * K).reshape(cd, 1, K),
                                  vec(f"{p}.conv1d.bias", cd, required=False), vec(f"{p}.dt_bias", Hv, torch.float32),
                                  vec(f"{p}.A_log", Hv, torch.float32), vec(f"{p}.norm.weight", cfg.linear_value_head_dim),
                                  linear_w(f"{p}.out_proj", h, vd))
        p = f"{lp}.mlp"
        if cfg.is_moe:
            E, mi, si = cfg.num_experts, cfg.moe_intermediate_size, cfg.shared_expert_intermediate_size
            bare = find(f"{p}.experts.gate_up_proj") is not None
            gu = linear_w(f"{p}.experts.gate_up_proj", 2 * mi, h, "" if bare else ".weight")
            dn = linear_w(f"{p}.experts.down_proj", h, mi, "" if bare else ".weight")
            ffn = SparseMoeBlock(vec(f"{p}.gate.weight", E * h).reshape(E, h), gu, dn,
                                 MLP(linear_w(f"{p}.shared_expert.gate_proj", si, h), linear_w(f"{p}.shared_expert.up_proj", si, h),
                                     linear_w(f"{p}.shared_expert.down_proj", h, si)), linear_w(f"{p}.shared_expert_gate", 1, h))
        else:
            I = cfg.intermediate_size
            ffn = MLP(linear_w(f"{p}.gate_proj", I, h), linear_w(f"{p}.up_proj", I, h), linear_w(f"{p}.down_proj", h, I))
        layers.append(Layer(vec(f"{lp}.input_layernorm.weight", h), mixer, vec(f"{lp}.post_attention_layernorm.weight", h), ffn))
        info(f"  loaded layers {i + 1}/{cfg.num_hidden_layers}")
    norm = vec("model.norm.weight", h)
    hn = next((n for n in ("lm_head.weight", "language_model.lm_head.weight") if src.find(n) is not None), None)
    if hn is None:
        info("  lm_head.weight not found; tying to embeddings.")
        return Qwen35ForCausalLM(cfg, emb.reshape(cfg.vocab_size, h), layers, norm, emb.reshape(cfg.vocab_size, h), True)
    return Qwen35ForCausalLM(cfg, emb.reshape(cfg.vocab_size, h), layers, norm, src.load(hn).to(device=device, dtype=dtype), False)


def load_pretrained(model_dir: str, device="cpu", dtype=torch.bfloat16, log=None) -> Qwen35ForCausalLM:
    return load(Qwen35Config.load_from_pretrained_dir(model_dir), model_dir, device, dtype, log)


def state_dict(m: Qwen35ForCausalLM) -> Dict[str, torch.Tensor]:
    out = {"model.embed_tokens.weight": m.embed_tokens, "model.norm.weight": m.norm}
    if not m.tie_word_embeddings:
        out["lm_head.weight"] = m.lm_head
    for i, l in enumerate(m.layers):
        p = f"model.layers.{i}"
        out[f"{p}.input_layernorm.weight"], out[f"{p}.post_attention_layernorm.weight"] = l.input_layernorm, l.post_attention_layernorm
        x = l.mixer
        if isinstance(x, Attention):
            for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
                out[f"{p}.self_attn.{n}.weight"] = getattr(x, n)
            out[f"{p}.self_attn.q_norm.weight"], out[f"{p}.self_attn.k_norm.weight"] = x.q_norm, x.k_norm
        else:
            for n in ("in_proj_qkv", "in_proj_z", "in_proj_b", "in_proj_a", "out_proj"):
                out[f"{p}.linear_attn.{n}.weight"] = getattr(x, n)
            out[f"{p}.linear_attn.conv1d.weight"] = x.conv1d_weight
            if x.conv1d_bias is not None:
                out[f"{p}.linear_attn.conv1d.bias"] = x.conv1d_bias
            out[f"{p}.linear_attn.dt_bias"], out[f"{p}.linear_attn.A_log"], out[f"{p}.linear_attn.norm.weight"] = x.dt_bias, x.a_log, x.norm_weight
        f = l.ffn
        if isinstance(f, MLP):
            for n in ("gate_proj", "up_proj", "down_proj"):
                out[f"{p}.mlp.{n}.weight"] = getattr(f, n)
        else:
            out[f"{p}.mlp.gate.weight"] = f.router
            out[f"{p}.mlp.experts.gate_up_proj"], out[f"{p}.mlp.experts.down_proj"] = f.gate_up_proj, f.down_proj
            for n in ("gate_proj", "up_proj", "down_proj"):
                out[f"{p}.mlp.shared_expert.{n}.weight"] = getattr(f.shared_expert, n)
            out[f"{p}.mlp.shared_expert_gate.weight"] = f.shared_expert_gate
    return out
