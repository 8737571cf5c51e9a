"""Tensor-parallel Qwen3.5 (dense FFN): attention / GatedDeltaNet heads, MLP columns and the vocabulary are split over
the ranks of one NVLink domain; each rank keeps the K/V caches and recurrent states of its own heads.

Two activation layouts, chosen per call by the row count:

* **sequence-parallel** (prefill): between blocks every rank holds ``rows / world`` token rows.  A block is
  ``RMSNorm -> all-gather+GEMM (fused in-projection of all local heads) -> mixer core -> GEMM+reduce-scatter (+residual)``,
  both collectives running inside the tcgen05 GEMM kernel (parallel/tp.py).
* **replicated** (decode): the few rows live on every rank; the row-parallel projections end in a one-shot
  all-reduce over peer memory.

The in-projections of a block are stored as one fused weight per rank so that the gathered activations cross NVLink
once per block.  The single-GPU model (models/qwen35.py, Tyr/Model/Qwen35/Model.lean) is the numerics oracle; the
reference has no tensor parallelism.
"""
from __future__ import annotations

import dataclasses
import os
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..parallel.tp import TensorParallel
from . import qwen35 as Q
from ..ops.decode_attention import geometry_supported
from .common import KVCache, lin
from .generation import SamplingStrategy, generate_cached


@dataclass
class TPAttention:
    in_proj: torch.Tensor      # [(H_l*2D + 2*Hkv_l*D), hidden]: q‖gate per head, then k, then v
    o_proj: torch.Tensor       # [hidden, H_l*D]
    q_norm: torch.Tensor
    k_norm: torch.Tensor


@dataclass
class TPGatedDeltaNet:
    in_proj: torch.Tensor      # [conv_dim_l + vd_l + 2*Hv_l, hidden]: qkv, z, b, a
    conv1d_weight: torch.Tensor
    conv1d_bias: Optional[torch.Tensor]
    dt_bias: torch.Tensor
    a_log: torch.Tensor
    norm_weight: torch.Tensor
    out_proj: torch.Tensor     # [hidden, vd_l]


@dataclass
class TPMLP:
    gate_up: torch.Tensor      # [2*I_l, hidden]: gate rows then up rows
    down: torch.Tensor         # [hidden, I_l]


@dataclass
class TPLayer:
    input_layernorm: torch.Tensor
    mixer: object
    post_attention_layernorm: torch.Tensor
    ffn: TPMLP


@dataclass
class Qwen35TP:
    cfg: Q.Qwen35Config            # the full model
    local: Q.Qwen35Config          # head / column counts of this rank
    rank: int
    world: int
    embed_tokens: torch.Tensor     # replicated
    layers: List[TPLayer]
    norm: torch.Tensor
    lm_head: torch.Tensor          # [vocab / world, hidden]
    tp: TensorParallel

    @property
    def device(self): return self.embed_tokens.device
    @property
    def dtype(self): return self.embed_tokens.dtype


def local_config(cfg: Q.Qwen35Config, world: int) -> Q.Qwen35Config:
    if cfg.is_moe:
        raise NotImplementedError("tensor parallelism covers the dense Qwen3.5 models; MoE models use expert parallelism")
    for name, v in (("attention heads", cfg.num_attention_heads), ("linear key heads", cfg.linear_num_key_heads),
                    ("linear value heads", cfg.linear_num_value_heads), ("intermediate size", cfg.intermediate_size), ("vocabulary", cfg.vocab_size)):
        if v % world:
            raise ValueError(f"Qwen3.5 tensor parallel: {name} ({v}) do not divide over {world} ranks")
    Hkv = cfg.num_key_value_heads
    if Hkv % world and world % Hkv:
        raise ValueError(f"Qwen3.5 tensor parallel: {Hkv} K/V heads neither divide over nor replicate into {world} ranks")
    return dataclasses.replace(cfg, num_attention_heads=cfg.num_attention_heads // world, num_key_value_heads=max(1, Hkv // world),
                               linear_num_key_heads=cfg.linear_num_key_heads // world, linear_num_value_heads=cfg.linear_num_value_heads // world,
                               intermediate_size=cfg.intermediate_size // world, layer_types=list(cfg.layer_types))


def _rows(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = t.shape[0] // world
    return t[rank * n:(rank + 1) * n]


def _kv_rows(cfg, t, rank, world):
    Hkv, D = cfg.num_key_value_heads, cfg.head_dim
    if Hkv >= world:
        return _rows(t, rank, world)
    head = rank // (world // Hkv)            # K/V head shared by world/Hkv consecutive ranks
    return t[head * D:(head + 1) * D]


def shard(m: Q.Qwen35ForCausalLM, rank: int, world: int, tp: TensorParallel) -> Qwen35TP:
    """Cut this rank's slice out of a full model (tests, and loading checkpoints that fit one host)."""
    cfg = m.cfg
    loc = local_config(cfg, world)
    kd = cfg.linear_key_dim
    layers = []
    for i, l in enumerate(m.layers):
        x = l.mixer
        if cfg.is_full(i):
            mixer = TPAttention(torch.cat([_rows(x.q_proj, rank, world), _kv_rows(cfg, x.k_proj, rank, world), _kv_rows(cfg, x.v_proj, rank, world)]).contiguous(),
                                x.o_proj.chunk(world, dim=1)[rank].contiguous(), x.q_norm, x.k_norm)
        else:
            seg = lambda t: torch.cat([_rows(t[:kd], rank, world), _rows(t[kd:2 * kd], rank, world), _rows(t[2 * kd:], rank, world)])
            merged = torch.cat([seg(x.in_proj_qkv), _rows(x.in_proj_z, rank, world), _rows(x.in_proj_b, rank, world), _rows(x.in_proj_a, rank, world)])
            if merged.shape[0] % 8:      # zero rows up to a multiple of 8 output columns: keeps the merged projection on the tensor-core / fused path
                merged = F.pad(merged, (0, 0, 0, (-merged.shape[0]) % 8))
            mixer = TPGatedDeltaNet(merged.contiguous(),
                                    seg(x.conv1d_weight).contiguous(), None if x.conv1d_bias is None else seg(x.conv1d_bias).contiguous(),
                                    _rows(x.dt_bias, rank, world), _rows(x.a_log, rank, world), x.norm_weight, x.out_proj.chunk(world, dim=1)[rank].contiguous())
        f = l.ffn
        ffn = TPMLP(torch.cat([_rows(f.gate_proj, rank, world), _rows(f.up_proj, rank, world)]).contiguous(), f.down_proj.chunk(world, dim=1)[rank].contiguous())
        layers.append(TPLayer(l.input_layernorm, mixer, l.post_attention_layernorm, ffn))
    return Qwen35TP(cfg, loc, rank, world, m.embed_tokens, layers, m.norm, _rows(m.lm_head, rank, world).contiguous(), tp)


def init_sharded(cfg: Q.Qwen35Config, rank: int, world: int, tp: TensorParallel, device="cuda", dtype=torch.bfloat16, seed=0) -> Qwen35TP:
    """Random weights created directly in sharded form on ``device`` (benchmarks of models too large to build whole).
    Replicated tensors come from ``seed`` on every rank, sharded ones from a per-rank stream."""
    loc = local_config(cfg, world)
    shared = torch.Generator(device=device).manual_seed(seed)
    mine = torch.Generator(device=device).manual_seed(seed * 1000 + 17 + rank)
    mk = lambda shape, fan, g=mine: (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * fan ** -0.5).to(dtype)
    zeros = lambda n: torch.zeros(n, device=device, dtype=dtype)
    h, D = cfg.hidden_size, cfg.head_dim
    layers = []
    for i in range(cfg.num_hidden_layers):
        if cfg.is_full(i):
            Hl, Hkvl = loc.num_attention_heads, loc.num_key_value_heads
            mixer = TPAttention(mk((Hl * 2 * D + 2 * Hkvl * D, h), h), mk((h, Hl * D), cfg.num_attention_heads * D), zeros(D), zeros(D))
        else:
            Hv, cd, vd, K = loc.linear_num_value_heads, loc.linear_conv_dim, loc.linear_value_dim, cfg.linear_conv_kernel_dim
            a = torch.rand(Hv, generator=mine, device=device) * 16.0 + 1e-6
            mixer = TPGatedDeltaNet(mk((-(-(cd + vd + 2 * Hv) // 8) * 8, h), h), mk((cd, 1, K), K),      # width rounded up to 8 columns (the extra ones are unused)
                                    (torch.rand(cd, generator=mine, device=device) * 0.2 - 0.1).to(dtype),
                                    torch.ones(Hv, device=device), torch.log(a), torch.ones(cfg.linear_value_head_dim, device=device, dtype=dtype),
                                    mk((h, vd), cfg.linear_value_dim))
        I = loc.intermediate_size
        layers.append(TPLayer(zeros(h), mixer, zeros(h), TPMLP(mk((2 * I, h), h), mk((h, I), cfg.intermediate_size))))
    emb = (torch.randn((cfg.vocab_size, h), generator=shared, device=device, dtype=torch.float32) * 0.02).to(dtype)
    head = _rows(emb, rank, world).contiguous() if cfg.tie_word_embeddings else mk((cfg.vocab_size // world, h), h)
    return Qwen35TP(cfg, loc, rank, world, emb, layers, zeros(h), head, tp)


class TPCache:
    """Per-rank decoding state: K/V of the local heads of full layers, conv + recurrent state of the local heads of
    linear layers."""

    def __init__(self, m: Qwen35TP, batch: int, max_len: int):
        cfg, loc = m.cfg, m.local
        self.m, self.pos, self.max_len, self.batch = m, 0, max_len, batch
        self.cos, self.sin = Q.rope_tables(cfg, max_len, m.device)
        self.kv = [KVCache.allocate(batch, loc.num_key_value_heads, max_len, cfg.head_dim, m.device, m.dtype) if cfg.is_full(i) else None
                   for i in range(cfg.num_hidden_layers)]
        self.lin = [None if cfg.is_full(i) else Q.LinearState() for i in range(cfg.num_hidden_layers)]

    def _mixer(self, i, l: TPLayer, proj, B, S, cos, sin):
        loc = self.m.local
        proj = proj.reshape(B, S, -1)
        if isinstance(l.mixer, TPAttention):
            nq, nkv = loc.num_attention_heads * 2 * loc.head_dim, loc.num_key_value_heads * loc.head_dim
            return Q.attention_core(loc, l.mixer.q_norm, l.mixer.k_norm, proj[..., :nq], proj[..., nq:nq + nkv], proj[..., nq + nkv:], cos, sin, self.kv[i])
        cd, vd, Hv = loc.linear_conv_dim, loc.linear_value_dim, loc.linear_num_value_heads
        return Q.gated_delta_net_core(loc, l.mixer, proj[..., :cd], proj[..., cd:cd + vd], proj[..., cd + vd:cd + vd + Hv], proj[..., cd + vd + Hv:cd + vd + 2 * Hv], self.lin[i])

    @staticmethod
    def _mlp_hidden(h, gate_up):
        """silu(h gate^T) * (h up^T) for the local column slice; decode-sized rows take the one-pass weight-streaming kernel."""
        from ..ops import decode_gemm, skinny
        I = gate_up.shape[0] // 2
        if h.is_cuda and decode_gemm.supported(h, gate_up[:I], gate_up[I:], min_tiles=decode_gemm.GATED_MIN_ROW_TILES):
            return decode_gemm.decode_swiglu(h, gate_up[:I], gate_up[I:])
        if h.shape[0] <= skinny.MAX_ROWS and h.is_cuda and skinny.swiglu_supported(h, gate_up[:I], gate_up[I:]):
            return skinny.skinny_swiglu(h, gate_up[:I], gate_up[I:])
        return TPCache._swiglu(lin(h, gate_up))

    @staticmethod
    def _swiglu(gu):
        I = gu.shape[-1] // 2
        return (F.silu(gu[..., :I].float()) * gu[..., I:].float()).to(gu.dtype)

    def sequence_parallel(self, B: int, S: int) -> bool:
        """Whether ``run`` scatters the rows of a [B, S] chunk over the ranks (prefill) or keeps them replicated (decode)."""
        W, rows = self.m.world, B * S
        return W > 1 and S > 1 and rows % W == 0 and (rows // W) % (128 if self.m.tp.fused else 1) == 0

    @torch.no_grad()
    def layer_forward(self, i: int, x: torch.Tensor, B: int, S: int, cos, sin, seq_par: bool) -> torch.Tensor:
        """One decoder layer on the residual stream ``x``: this rank's ``[B*S / world, hidden]`` rows when ``seq_par``, else
        all ``[B*S, hidden]`` rows (replicated).  Advances layer i's cache.  ``run`` is a loop over this; tests drive it
        layer by layer with the single-device model's activations as input."""
        m, tp = self.m, self.m.tp
        l, eps, rows = m.layers[i], m.cfg.rms_norm_eps, B * S
        w_out = l.mixer.o_proj if isinstance(l.mixer, TPAttention) else l.mixer.out_proj
        if seq_par:
            proj = tp.allgather_gemm(Q.rms(x, l.input_layernorm, eps), l.mixer.in_proj)
            core = self._mixer(i, l, proj, B, S, cos, sin).reshape(rows, -1)
            x = tp.gemm_reduce_scatter(core, w_out, add=x)
            gu = tp.allgather_gemm(Q.rms(x, l.post_attention_layernorm, eps), l.ffn.gate_up)
            return tp.gemm_reduce_scatter(self._swiglu(gu), l.ffn.down, add=x)
        proj = lin(Q.rms(x, l.input_layernorm, eps), l.mixer.in_proj)
        core = self._mixer(i, l, proj, B, S, cos, sin).reshape(rows, -1)
        x = tp.linear_all_reduce(core, w_out, add=x)
        return tp.linear_all_reduce(self._mlp_hidden(Q.rms(x, l.post_attention_layernorm, eps), l.ffn.gate_up), l.ffn.down, add=x)

    @torch.no_grad()
    def run(self, ids: torch.Tensor) -> torch.Tensor:
        """ids: [B, S] (identical on every rank) -> full-vocabulary logits of the last position, [B, V], on every rank."""
        m, cfg, tp = self.m, self.m.cfg, self.m.tp
        B, S = ids.shape
        if self.pos + S > self.max_len:
            raise ValueError("Qwen3.5 cache overflow")
        cos, sin = self.cos[self.pos:self.pos + S], self.sin[self.pos:self.pos + S]
        rows, W, eps = B * S, m.world, cfg.rms_norm_eps
        seq_par = self.sequence_parallel(B, S)
        if seq_par:
            rpr = rows // W
            x = F.embedding(ids.reshape(-1)[m.rank * rpr:(m.rank + 1) * rpr], m.embed_tokens)               # this rank's rows
            for i in range(len(m.layers)):
                x = self.layer_forward(i, x, B, S, cos, sin, True)
            last = torch.zeros((B, cfg.hidden_size), dtype=torch.float32, device=x.device)
            want = torch.arange(B, device=x.device) * S + (S - 1)
            mine = (want >= m.rank * rpr) & (want < (m.rank + 1) * rpr)
            if bool(mine.any()):
                last[mine] = x[want[mine] - m.rank * rpr].float()
            dist.all_reduce(last, group=tp.group)
            x_last = last.to(x.dtype)
        else:
            x = F.embedding(ids.reshape(-1), m.embed_tokens)                                                # replicated rows
            for i in range(len(m.layers)):
                x = self.layer_forward(i, x, B, S, cos, sin, False)
            x_last = x.reshape(B, S, -1)[:, -1]
        self.pos += S
        return tp.all_gather_cols(lin(Q.rms(x_last, m.norm, eps), m.lm_head))

    def prefill(self, ids): return self.run(ids)

    # -- replicated decode with the position on the device (CUDA-graph body) ---------------------------------------------
    def device_step_supported(self) -> bool:
        m, loc = self.m, self.m.local
        return (m.tp.fused and m.dtype == torch.bfloat16 and os.environ.get("TYR_DECODE_GRAPH", "1") != "0"
                and geometry_supported(loc.num_attention_heads, loc.num_key_value_heads, loc.head_dim))

    def _device_step(self, tok: torch.Tensor) -> torch.Tensor:
        """Final normed hidden state [B, hidden] of the new token on every rank; the vocabulary-parallel head and its
        gather stay outside the graph."""
        m, cfg, loc, tp = self.m, self.m.cfg, self.m.local, self.m.tp
        eps, B = cfg.rms_norm_eps, tok.numel()
        x = F.embedding(tok.reshape(-1), m.embed_tokens)
        # every all-reduce hands back the residual stream and the next sub-layer's normed input from one kernel
        h = Q.rms(x, m.layers[0].input_layernorm, eps)
        n_layers = len(m.layers)
        for i, l in enumerate(m.layers):
            proj = lin(h, l.mixer.in_proj).reshape(B, 1, -1)
            if isinstance(l.mixer, TPAttention):
                nq, nkv = loc.num_attention_heads * 2 * loc.head_dim, loc.num_key_value_heads * loc.head_dim
                core = Q.attention_core_decode(loc, l.mixer.q_norm, l.mixer.k_norm, proj[..., :nq], proj[..., nq:nq + nkv], proj[..., nq + nkv:],
                                               self.cos, self.sin, self.pos_t, self.kv[i])
                w_out = l.mixer.o_proj
            else:
                cd, vd, Hv = loc.linear_conv_dim, loc.linear_value_dim, loc.linear_num_value_heads
                core = Q.gated_delta_net_core(loc, l.mixer, proj[..., :cd], proj[..., cd:cd + vd], proj[..., cd + vd:cd + vd + Hv], proj[..., cd + vd + Hv:cd + vd + 2 * Hv], self.lin[i])
                w_out = l.mixer.out_proj
            x, h = tp.linear_all_reduce_norm(core.reshape(B, -1), w_out, x, l.post_attention_layernorm, eps)
            next_w = m.layers[i + 1].input_layernorm if i + 1 < n_layers else m.norm
            x, h = tp.linear_all_reduce_norm(self._mlp_hidden(h, l.ffn.gate_up), l.ffn.down, x, next_w, eps)
        self.pos_t += 1
        return h

    def step(self, tok):
        if self.pos == 0 or not self.device_step_supported():
            return self.run(tok.reshape(-1, 1))
        if self.pos + 1 > self.max_len:
            raise ValueError("Qwen3.5 cache overflow")
        if getattr(self, "_graph", None) is None:
            from ..utils.graph import GraphedStep
            self.pos_t = torch.full((1,), self.pos, dtype=torch.int32, device=self.m.device)
            state = [self.pos_t] + [t for s in self.lin if s is not None for t in (s.conv, s.rec)]
            parity0 = self.m.tp._parity
            self._graph = GraphedStep(self._device_step, (tok.reshape(-1).clone(),), advancing_state=state)
            # the symmetric partial-product buffers alternate per call and the choice is baked into the captured graph: a
            # replay is only safe when one step makes an even number of such calls (two per layer here)
            if self.m.tp._parity != parity0:
                raise RuntimeError("tensor-parallel decode step made an odd number of double-buffered calls; it cannot be replayed from a graph")
        h = self._graph(tok.reshape(-1))
        self.pos += 1
        for c in self.kv:
            if c is not None:
                c.length += 1
        return self.m.tp.all_gather_cols(lin(h, self.m.lm_head))


def generate(m: Qwen35TP, input_ids, max_new_tokens=64, strategy=SamplingStrategy.greedy(), eos_token_ids=None, on_step=None):
    """Every rank runs the same call with the same ``input_ids`` and gets the same tokens (greedy, or sampling from
    identically seeded generators)."""
    eos = eos_token_ids if eos_token_ids is not None else (() if m.cfg.eos_token_id is None else (m.cfg.eos_token_id,))
    c = TPCache(m, input_ids.shape[0], input_ids.shape[1] + max_new_tokens)
    return generate_cached(c.prefill, c.step, input_ids, max_new_tokens, strategy, eos, on_step)
