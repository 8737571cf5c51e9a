"""Character-level GPT (GPT-2 style) through the typed API (Examples/GPT/GPT.lean).

LayerNorm with bias, learned positional embedding, separate q/k/v/c_proj matrices, GELU MLP 4x,
dropout, weight-tied head (logits = x @ wte^T, :203-205).  Presets as in the reference (:30-51).
The model is a ``@tensor_struct`` tree of typed tensors; ``forward`` / ``loss`` use typed ops only,
so every intermediate is shape/dtype/device checked.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch

from ..struct import Static, tensor_struct
from ..typed import DType, Device, Tensor
from ..typed import neural as N
from ..typed import ops as O


@dataclass(frozen=True)
class Config:
    vocab_size: int
    block_size: int
    n_embd: int
    n_head: int
    n_layer: int
    dropout: float = 0.0

    @staticmethod
    def gpt2_small(): return Config(50257, 1024, 768, 12, 12)
    @staticmethod
    def gpt2_mini(): return Config(50257, 256, 384, 6, 6)
    @staticmethod
    def gpt2_micro(): return Config(50257, 128, 128, 4, 4)
    @staticmethod
    def tiny_shakespeare(): return Config(65, 64, 64, 4, 2, 0.0)
    @staticmethod
    def nanogpt_cpu_shakespeare(): return Config(65, 64, 128, 4, 4, 0.0)
    @staticmethod
    def nanogpt_gpu_shakespeare(): return Config(65, 256, 384, 6, 6, 0.2)


@tensor_struct
class BlockParams:
    ln1_weight: Tensor
    ln1_bias: Tensor
    q_proj: Tensor
    k_proj: Tensor
    v_proj: Tensor
    c_proj: Tensor
    c_proj_bias: Tensor
    ln2_weight: Tensor
    ln2_bias: Tensor
    mlp_fc: Tensor
    mlp_fc_bias: Tensor
    mlp_proj: Tensor
    mlp_proj_bias: Tensor

    @staticmethod
    def init(n_embd: int, scale: float = 0.02, device: Device = Device.CPU, generator=None) -> "BlockParams":
        def w(*shape):
            return O.parameter(O.mul_scalar(O.randn(shape, DType.Float32, device, generator=generator), scale))
        one = lambda n: O.parameter(O.ones((n,), DType.Float32, device))
        zero = lambda n: O.parameter(O.zeros((n,), DType.Float32, device))
        return BlockParams(one(n_embd), zero(n_embd), w(n_embd, n_embd), w(n_embd, n_embd), w(n_embd, n_embd),
                           w(n_embd, n_embd), zero(n_embd), one(n_embd), zero(n_embd), w(4 * n_embd, n_embd),
                           zero(4 * n_embd), w(n_embd, 4 * n_embd), zero(n_embd))


@tensor_struct
class GPTParams:
    wte: Tensor
    wpe: Tensor
    blocks: List[BlockParams]
    ln_f_weight: Tensor
    ln_f_bias: Tensor
    cfg: Static

    @staticmethod
    def init(cfg: Config, device: Device = Device.CPU, seed=None) -> "GPTParams":
        gen = None
        if seed is not None:
            gen = torch.Generator(device="cpu").manual_seed(seed)

        def randn(*shape):
            t = O.randn(shape, DType.Float32, Device.CPU, generator=gen)
            return t.to(device) if device != Device.CPU else t
        wte = O.parameter(O.mul_scalar(randn(cfg.vocab_size, cfg.n_embd), 0.02))
        wpe = O.parameter(O.mul_scalar(randn(cfg.block_size, cfg.n_embd), 0.02))
        blocks = [BlockParams.init(cfg.n_embd, 0.02, device, gen if device == Device.CPU else None) for _ in range(cfg.n_layer)]
        return GPTParams(wte, wpe, blocks, O.parameter(O.ones((cfg.n_embd,), DType.Float32, device)),
                         O.parameter(O.zeros((cfg.n_embd,), DType.Float32, device)), Static(cfg))


def block_forward(b: BlockParams, x: Tensor, n_head: int, dropout: float, training: bool) -> Tensor:
    B, T, C = x.shape
    hd = C // n_head
    h = O.layer_norm(x, b.ln1_weight, b.ln1_bias)
    q, k, v = O.linear(h, b.q_proj), O.linear(h, b.k_proj), O.linear(h, b.v_proj)
    split = lambda t: O.transpose(O.reshape(t, (B, T, n_head, hd)), 1, 2)
    att = N.attention(split(q), split(k), split(v), causal=True)
    att = O.reshape(O.transpose(att, 1, 2), (B, T, C))
    att = O.linear(att, b.c_proj, b.c_proj_bias)
    if dropout > 0:
        att = O.dropout(att, dropout, training)
    x = O.add(x, att)
    h = O.layer_norm(x, b.ln2_weight, b.ln2_bias)
    h = O.gelu(O.linear(h, b.mlp_fc, b.mlp_fc_bias))
    h = O.linear(h, b.mlp_proj, b.mlp_proj_bias)
    if dropout > 0:
        h = O.dropout(h, dropout, training)
    return O.add(x, h)


def forward(params: GPTParams, idx: Tensor, training: bool = False) -> Tensor:
    """idx: Int64 [B, T] -> logits [B, T, vocab]."""
    cfg: Config = params.cfg.val
    B, T = idx.shape
    if T > cfg.block_size:
        raise ValueError(f"sequence length {T} exceeds block size {cfg.block_size}")
    pos = O.arange(T, DType.Int64, idx.device)
    x = O.add(O.embedding(idx, params.wte), O.embedding(pos, params.wpe))
    if cfg.dropout > 0:
        x = O.dropout(x, cfg.dropout, training)
    for b in params.blocks:
        x = block_forward(b, x, cfg.n_head, cfg.dropout, training)
    x = O.layer_norm(x, params.ln_f_weight, params.ln_f_bias)
    return O.linear(x, params.wte)          # weight tying


def loss(params: GPTParams, x: Tensor, y: Tensor, training: bool = True) -> Tensor:
    logits = forward(params, x, training)
    B, T, V = logits.shape
    return O.cross_entropy(O.reshape(logits, (B * T, V)), O.reshape(y, (B * T,)))


def generate(params: GPTParams, idx: Tensor, max_new_tokens: int, temperature: float = 1.0, top_k: int = 0,
             generator=None) -> Tensor:
    cfg: Config = params.cfg.val
    out = idx.raw
    with torch.no_grad():
        for _ in range(max_new_tokens):
            ctx = Tensor.of_tensor(out[:, -cfg.block_size:])
            logits = forward(params, ctx).raw[:, -1, :] / max(temperature, 1e-8)
            lt = Tensor.of_tensor(logits)
            if top_k > 0:
                lt = O.top_k_filter(lt, top_k)
            nxt = O.multinomial(O.softmax(lt), 1, generator=generator).raw
            out = torch.cat([out, nxt], dim=1)
    return Tensor.of_tensor(out)
