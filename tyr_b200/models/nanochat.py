"""NanoChat / modded-nanogpt decoder (the reference's ``torch.moddedGpt``,
Examples/NanoChat/ModdedGPT.lean).

Architecture kept exactly: token embedding with smear gate, weight-free RMSNorm everywhere,
four learnable sigmoid-squashed scalars per layer plus eight global ones (init 1.1),
``x = lam_x x + lam_0 x0`` blend, separate q/k/v/o projections with half-split RoPE followed by
QK RMSNorm, value-embedding blend on the first/last layers, causal (optionally sliding-window)
attention, ReLU^2 MLP with ``c_proj`` stored ``[4d, d]``, an attention-less layer 5 that adds
the layer-2 input as a skip, untied lm_head, 15*tanh(x/15) logit soft cap, mean cross-entropy.

Two execution paths share one parameter store:

* ``loss_fused`` - the training hot path.  bf16 activations, every matrix product on the
  hand-written tcgen05 GEMM, all elementwise work folded into a handful of fused kernels, the
  lm_head + soft cap + cross-entropy evaluated chunk by chunk.
* ``forward_reference`` / ``loss_reference`` - op-for-op restatement of the reference graph in
  plain PyTorch (any dtype/device): the numerics oracle and the generation path on CPU.

Parameters are stored stacked per shape class (``[layers, 4, d, d]`` attention matrices,
``[layers, 2, 4d, d]`` MLP matrices) so that the Muon update and its Newton-Schulz GEMMs run
batched over all matrices of one shape; the individual reference parameters (``wQ``, ``cFc`` ...)
are views.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, asdict
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from .. import ops
from ..ops.gemm import gemm
from ..ops.norm import rms_norm_ref


@dataclass
class Config:
    """Mirrors ``moddedGpt.Config`` (Examples/NanoChat/ModdedGPT.lean:30-57)."""
    vocab_size: int = 50304
    n_layer: int = 11
    n_head: int = 6
    half_head_dim: int = 64
    max_seq_len: int = 2048
    block_size: int = 128
    rope_base: float = 500000.0
    num_value_embeds: int = 3
    softcap_value: float = 15.0
    window_pattern: str = "L"

    def __post_init__(self):
        if self.vocab_size <= 0:
            raise ValueError("Invalid model config: vocabSize must be positive")
        if self.max_seq_len <= 0:
            raise ValueError("Invalid model config: maxSeqLen must be positive")

    @property
    def head_dim(self) -> int:
        return 2 * self.half_head_dim

    @property
    def model_dim(self) -> int:
        return self.n_head * self.head_dim

    def to_json(self) -> dict:
        d = asdict(self)
        return {"vocabSize": d["vocab_size"], "nLayer": d["n_layer"], "nHead": d["n_head"],
                "halfHeadDim": d["half_head_dim"], "maxSeqLen": d["max_seq_len"],
                "blockSize": d["block_size"], "ropeBase": d["rope_base"],
                "numValueEmbeds": d["num_value_embeds"], "softcapValue": d["softcap_value"],
                "windowPattern": d["window_pattern"]}

    @staticmethod
    def from_json(j: dict) -> "Config":
        return Config(vocab_size=j["vocabSize"], n_layer=j["nLayer"], n_head=j["nHead"],
                      half_head_dim=j["halfHeadDim"], max_seq_len=j["maxSeqLen"],
                      block_size=j["blockSize"], rope_base=j["ropeBase"],
                      num_value_embeds=j["numValueEmbeds"], softcap_value=j["softcapValue"],
                      window_pattern=j["windowPattern"])


def find_heads(model_dim: int, target_head_dim: int):
    """(n_head, half_head_dim) with head width closest to the target
    (Examples/NanoChat/Pipeline.lean:212-222)."""
    best = None
    for half in range(1, model_dim // 2 + 1):
        if model_dim % (2 * half) == 0:
            if best is None or abs(2 * half - target_head_dim) < abs(2 * best[1] - target_head_dim):
                best = (model_dim // (2 * half), half)
    return best


def depth_config(depth: int = 20, aspect_ratio: int = 64, target_head_dim: int = 128,
                 vocab_size: int = 65536, max_seq_len: int = 2048,
                 rope_base: float = 500000.0) -> Config:
    """``NanoChatConfig.toModelConfig?``: d20 -> dim 1280, 10 heads x 128."""
    model_dim = depth * aspect_ratio
    hh = find_heads(model_dim, target_head_dim)
    if hh is None:
        raise ValueError(f"model dim {model_dim} does not split into heads of even width")
    return Config(vocab_size=vocab_size, n_layer=depth, n_head=hh[0], half_head_dim=hh[1],
                  max_seq_len=max_seq_len, block_size=128, rope_base=rope_base)


def get_window_size_for_layer(pattern: str, layer_idx: int, n_layers: int, seq_len: int) -> Optional[int]:
    """None = full context; 'S' = half-context sliding window; the final layer is always full."""
    if layer_idx == n_layers - 1 or not pattern:
        return None
    c = pattern[layer_idx % len(pattern)]
    if c in "Ss":
        return seq_len // 2
    return None


def compute_window_sizes(cfg: Config) -> List[Optional[int]]:
    return [get_window_size_for_layer(cfg.window_pattern, i, cfg.n_layer, cfg.max_seq_len)
            for i in range(cfg.n_layer)]


def layer_value_embed_index(cfg: Config, layer_idx: int) -> Optional[int]:
    """Value embeddings go to the first and last ``span`` layers
    (Examples/NanoChat/ModdedGPT.lean:466-483)."""
    n_layers, n_value = cfg.n_layer, cfg.num_value_embeds
    if n_layers == 0 or n_value == 0:
        return None
    span = min(n_value, n_layers)
    if layer_idx < span:
        return layer_idx
    back_start = n_layers - span
    if layer_idx >= back_start:
        return (layer_idx - back_start) % span
    return None


SKIP_ATTN_LAYER = 5
SKIP_SOURCE_LAYER = 2


class ModdedGPTParams:
    """Parameter store.  fp32 master weights (``master[name]``), compute-dtype working copies
    (``work[name]``, autograd leaves) and fp32 gradient accumulators (``grad[name]``)."""

    MATRIX_GROUPS = ("attn_w", "mlp_w")
    ADAM_GROUPS = ("embed", "value_embeds", "lm_head")

    @staticmethod
    def storage_plan(cfg: Config, compute_dtype=torch.bfloat16):
        """(shape, dtype) of every tensor requested from ``alloc``, in allocation order."""
        d, V, L = cfg.model_dim, cfg.vocab_size, cfg.n_layer
        La = L - (1 if L > SKIP_ATTN_LAYER else 0)
        shapes = [(V, d), (cfg.num_value_embeds, V, d), (La, 4, d, d), (L, 2, 4 * d, d), (V, d)]
        plan = []
        for s in shapes:
            plan.append((s, compute_dtype))
            plan.append((s, torch.float32))
        return plan

    def __init__(self, cfg: Config, device="cpu", compute_dtype=torch.bfloat16, seed: Optional[int] = None,
                 alloc=None):
        """``alloc(shape, dtype) -> tensor`` (optional) provides the storage of the working copies
        and gradient accumulators, e.g. from a symmetric heap that peers can address."""
        self.cfg = cfg
        self.device = torch.device(device)
        self.compute_dtype = compute_dtype
        d, V, L = cfg.model_dim, cfg.vocab_size, cfg.n_layer
        gen = torch.Generator(device="cpu")
        if seed is not None:
            gen.manual_seed(seed)
        else:
            gen.seed()

        def randn(*shape, scale=1.0):
            return (torch.randn(*shape, generator=gen, dtype=torch.float32) * scale).to(self.device)

        self.attn_layers = [i for i in range(L) if i != SKIP_ATTN_LAYER]
        self.attn_slot = {l: j for j, l in enumerate(self.attn_layers)}
        La = len(self.attn_layers)
        s = math.sqrt(3.0) / math.sqrt(d)
        attn = torch.zeros(max(La, 1), 4, d, d, dtype=torch.float32, device=self.device)
        if La:
            attn[:La, :3] = randn(La, 3, d, d, scale=s)          # wQ, wK, wV; wO stays zero
        mlp = torch.zeros(L, 2, 4 * d, d, dtype=torch.float32, device=self.device)
        mlp[:, 0] = randn(L, 4 * d, d, scale=0.02)                # cFc; cProj stays zero
        self.master: Dict[str, torch.Tensor] = {
            "embed": randn(V, d, scale=0.02),
            "smear_gate": randn(1, 12, scale=0.02),
            "value_embeds": randn(cfg.num_value_embeds, V, d, scale=0.02),
            "attn_w": attn[:La] if La else attn[:0],
            "mlp_w": mlp,
            "lm_head": randn(V, d, scale=0.02),
            "scalars": torch.full((L * 4 + 8,), 1.1, dtype=torch.float32, device=self.device),
        }
        self.work: Dict[str, torch.Tensor] = {}
        self.grad: Dict[str, torch.Tensor] = {}
        for k, v in self.master.items():
            if k in ("scalars", "smear_gate"):
                self.work[k] = v.detach().clone().requires_grad_(True)
                self.grad[k] = None
            elif alloc is not None:
                self.work[k] = alloc(tuple(v.shape), compute_dtype)
                self.work[k].copy_(v)
                self.grad[k] = alloc(tuple(v.shape), torch.float32)
                self.grad[k].zero_()
            else:
                self.work[k] = v.to(compute_dtype)
                self.grad[k] = torch.zeros_like(v)
        self._leaves: Dict[str, torch.Tensor] = {}
        self.refresh_leaves()
        cos, sin = ops.rotary_freqs(cfg.max_seq_len, cfg.head_dim, cfg.rope_base, device=self.device)
        self.cos, self.sin = cos.contiguous(), sin.contiguous()

    # -- leaves -------------------------------------------------------------------------------
    def _leaf(self, name: str, work_view: torch.Tensor, grad_view: torch.Tensor) -> torch.Tensor:
        t = work_view.detach().requires_grad_(True)
        t.main_grad = grad_view
        t.grad_ready = False
        self._leaves[name] = t
        return t

    def refresh_leaves(self):
        """(Re)create the autograd leaves as views of the stacked working copies."""
        self._leaves = {}
        d = self.cfg.model_dim
        for l, j in self.attn_slot.items():
            self._leaf(f"blocks.{l}.attn.wQKV", self.work["attn_w"][j, :3].reshape(3 * d, d),
                       self.grad["attn_w"][j, :3].reshape(3 * d, d))
            self._leaf(f"blocks.{l}.attn.wO", self.work["attn_w"][j, 3], self.grad["attn_w"][j, 3])
        for l in range(self.cfg.n_layer):
            self._leaf(f"blocks.{l}.mlp.cFc", self.work["mlp_w"][l, 0], self.grad["mlp_w"][l, 0])
            self._leaf(f"blocks.{l}.mlp.cProj", self.work["mlp_w"][l, 1], self.grad["mlp_w"][l, 1])
        self._leaf("embed", self.work["embed"], self.grad["embed"])
        for i in range(self.cfg.num_value_embeds):
            self._leaf(f"valueEmbeds.{i}", self.work["value_embeds"][i], self.grad["value_embeds"][i])
        self._leaf("lmHead.weight", self.work["lm_head"], self.grad["lm_head"])
        self._leaves["scalars.values"] = self.work["scalars"]
        self._leaves["smearGate.weight"] = self.work["smear_gate"]

    def leaf(self, name: str) -> torch.Tensor:
        return self._leaves[name]

    def named_leaves(self):
        return dict(self._leaves)

    # -- reference-named views (wQ, wK, ...) used by checkpoints and the oracle path ----------------
    def named_parameters(self, which: str = "master") -> Dict[str, torch.Tensor]:
        src = getattr(self, which)
        out = {"embed": src["embed"], "smearGate.weight": src["smear_gate"]}
        for i in range(self.cfg.num_value_embeds):
            out[f"valueEmbeds.{i}"] = src["value_embeds"][i]
        for l in range(self.cfg.n_layer):
            if l in self.attn_slot:
                j = self.attn_slot[l]
                for n, nm in enumerate(("wQ", "wK", "wV", "wO")):
                    out[f"blocks.{l}.attn.{nm}"] = src["attn_w"][j, n]
            out[f"blocks.{l}.mlp.cFc"] = src["mlp_w"][l, 0]
            out[f"blocks.{l}.mlp.cProj"] = src["mlp_w"][l, 1]
        out["lmHead.weight"] = src["lm_head"]
        out["scalars.values"] = src["scalars"]
        return out

    def load_named(self, tensors: Dict[str, torch.Tensor]):
        """Copy reference-named tensors into the master store and refresh the working copies."""
        dst = self.named_parameters("master")
        for k, v in tensors.items():
            if k not in dst:
                raise KeyError(f"unexpected parameter {k}")
            if tuple(dst[k].shape) != tuple(v.shape):
                raise ValueError(f"{k}: shape {tuple(v.shape)} != expected {tuple(dst[k].shape)}")
            dst[k].copy_(v.to(dst[k].dtype))
        self.sync_work_from_master()

    def sync_work_from_master(self):
        with torch.no_grad():
            for k, v in self.master.items():
                self.work[k].copy_(v.to(self.work[k].dtype))

    def zero_grads(self):
        for k, g in self.grad.items():
            if g is not None:
                g.zero_()
        for k in ("scalars", "smear_gate"):
            self.work[k].grad = None
        for t in self._leaves.values():
            if hasattr(t, "grad_ready"):
                t.grad_ready = False
            t.grad = None

    def num_parameters(self) -> int:
        return sum(v.numel() for v in self.master.values())


# --------------------------------------------------------------------------------------------
# Embedding with gradient accumulation into the fp32 buffer
# --------------------------------------------------------------------------------------------
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, table, idx, sorted_ids, order):
        ctx.save_for_backward(idx, sorted_ids, order)
        ctx.table = table
        return F.embedding(idx, table)

    @staticmethod
    def backward(ctx, dy):
        idx, sorted_ids, order = ctx.saved_tensors
        table = ctx.table
        mg = getattr(table, "main_grad", None)
        flat = dy.reshape(-1, dy.shape[-1])
        if mg is not None:
            # rows sorted by token id, one table update per id and run of rows instead of one atomic per occurrence
            ops.embed.embedding_grad_(mg, flat, idx, sorted_ids, order)
            table.grad_ready = True
            return None, None, None, None
        g = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
        g.index_add_(0, idx.reshape(-1), flat.float())
        return g.to(table.dtype), None, None, None


def embedding(table: torch.Tensor, idx: torch.Tensor, sorted_ids=None, order=None) -> torch.Tensor:
    """``sorted_ids`` / ``order``: the result of ``ops.embed.sort_tokens(idx)`` when several tables share the tokens."""
    if sorted_ids is None and idx.is_cuda:
        sorted_ids, order = ops.embed.sort_tokens(idx)
    return _EmbeddingFn.apply(table, idx, sorted_ids, order)


# --------------------------------------------------------------------------------------------
# ReLU^2 MLP as one autograd node (both GEMMs + fused activation gradient)
# --------------------------------------------------------------------------------------------
def _accum_wgrad(w, dy2, x2):
    """dW += dy2^T @ x2 into w.main_grad when present; otherwise returns a gradient tensor."""
    mg = getattr(w, "main_grad", None)
    if mg is not None:
        gemm(dy2, x2, a_layout="MN", b_layout="MN", out=mg, accumulate=True)
        w.grad_ready = True
        return None
    dw32 = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
    gemm(dy2, x2, a_layout="MN", b_layout="MN", out=dw32, accumulate=True)
    return dw32.to(w.dtype)


class _MlpRelu2Fn(torch.autograd.Function):
    """out = relu(x @ cFc^T)^2 @ cProj with cFc, cProj both [4d, d]."""

    @staticmethod
    def forward(ctx, x, c_fc, c_proj):
        h = gemm(x, c_fc, a_layout="K", b_layout="K", act="relu2")
        out = gemm(h, c_proj, a_layout="K", b_layout="MN")
        ctx.save_for_backward(x, c_fc, c_proj, h)
        return out

    @staticmethod
    def backward(ctx, dy):
        x, c_fc, c_proj, h = ctx.saved_tensors
        dy = dy.contiguous()
        # dz = (dy @ cProj^T) * 2*sqrt(h): activation gradient fused into the GEMM epilogue
        dz = gemm(dy, c_proj, a_layout="K", b_layout="K", act="relu2_grad", aux=h)
        d_proj = _accum_wgrad(c_proj, h, dy)     # [4d, d] = h^T @ dy
        d_fc = _accum_wgrad(c_fc, dz, x)         # [4d, d] = dz^T @ x
        dx = gemm(dz, c_fc, a_layout="K", b_layout="MN") if ctx.needs_input_grad[0] else None
        return dx, d_fc, d_proj


def mlp_relu2(x, c_fc, c_proj):
    return _MlpRelu2Fn.apply(x, c_fc, c_proj)


# --------------------------------------------------------------------------------------------
# Fused training path
# --------------------------------------------------------------------------------------------
def _stack_scalars(*vals):
    return torch.stack([v.reshape(()) for v in vals]).float()


def loss_fused(params: ModdedGPTParams, input_seq: torch.Tensor, targets: torch.Tensor,
               loss_scale: float = 1.0, ce_chunk_rows: int = 8192) -> torch.Tensor:
    """Mean cross-entropy of the model on ``input_seq`` [B, T] against ``targets`` [B, T]."""
    cfg = params.cfg
    B, T = input_seq.shape
    if T > cfg.max_seq_len:
        raise ValueError(f"sequence length {T} exceeds maxSeqLen {cfg.max_seq_len}")
    d, H, D, L = cfg.model_dim, cfg.n_head, cfg.head_dim, cfg.n_layer
    if d < 12:
        raise ValueError("ModdedGPT requires modelDim >= 12 for the smear gate")
    N = B * T
    dt = params.compute_dtype
    dev = input_seq.device
    idx = input_seq.reshape(-1)

    sig = torch.sigmoid(params.leaf("scalars.values").float())
    one = torch.ones((), dtype=torch.float32, device=dev)

    # token embedding + smear gate + norm
    sorted_ids, order = ops.embed.sort_tokens(idx) if idx.is_cuda else (None, None)   # shared by the four tables' gradients
    tok = embedding(params.leaf("embed"), idx, sorted_ids, order)           # [N, d]
    gate = torch.sigmoid(F.linear(tok[:, :12].float(), params.leaf("smearGate.weight").float()))
    x0_pre = (tok.float() * (1.0 + gate)).to(dt)
    _, x0 = ops.lincomb_rmsnorm([x0_pre], None)

    ve = [embedding(params.leaf(f"valueEmbeds.{i}"), idx, sorted_ids, order) for i in range(cfg.num_value_embeds)]
    value_mix = sig[L * 4]
    skip_mix = sig[L * 4 + 1]
    final_scale = sig[L * 4 + 2]

    xa, xb, coef = x0, None, None
    skip = None
    cos, sin = params.cos[:T].contiguous(), params.sin[:T].contiguous()
    for i in range(L):
        lam_x, lam_x0, lam_attn, lam_mlp = sig[4 * i], sig[4 * i + 1], sig[4 * i + 2], sig[4 * i + 3]
        if xb is None:
            x_in, x_n = ops.lincomb_rmsnorm([xa, x0], _stack_scalars(lam_x, lam_x0))
        else:
            x_in, x_n = ops.lincomb_rmsnorm([xa, xb, x0], _stack_scalars(lam_x, lam_x * coef, lam_x0))
        if i == SKIP_SOURCE_LAYER:
            skip = x_in
        window = get_window_size_for_layer(cfg.window_pattern, i, L, T)
        if i in params.attn_slot:
            qkv = ops.linear(x_n, params.leaf(f"blocks.{i}.attn.wQKV"))
            vi = layer_value_embed_index(cfg, i)
            qkv = ops.qkv_post(qkv, ve[vi] if vi is not None else None,
                               value_mix if vi is not None else None, cos, sin, T, H, D)
            att = ops.attention_packed(qkv, B, T, H, D, causal=True, window=window)
            o = ops.linear(att, params.leaf(f"blocks.{i}.attn.wO"))
            x1, x_n2 = ops.lincomb_rmsnorm([x_in, o], _stack_scalars(one, lam_attn))
        else:
            if skip is not None:
                x1, x_n2 = ops.lincomb_rmsnorm([x_in, skip], _stack_scalars(one, skip_mix))
            else:
                x1, x_n2 = x_in, x_n
        h2 = mlp_relu2(x_n2, params.leaf(f"blocks.{i}.mlp.cFc"), params.leaf(f"blocks.{i}.mlp.cProj"))
        xa, xb, coef = x1, h2, lam_mlp

    _, x_f = ops.lincomb_rmsnorm([xa, xb], _stack_scalars(final_scale, final_scale * coef))
    return ops.lm_head_ce(x_f, params.leaf("lmHead.weight"), targets.reshape(-1),
                          cap=cfg.softcap_value, chunk_rows=ce_chunk_rows, loss_scale=loss_scale)


# --------------------------------------------------------------------------------------------
# Reference restatement (oracle / generation)
# --------------------------------------------------------------------------------------------
def forward_reference(p: Dict[str, torch.Tensor], cfg: Config, input_seq: torch.Tensor,
                      cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Op-for-op restatement of ``moddedGpt.forward`` (ModdedGPT.lean:552-635) on reference-named
    parameters ``p``; returns soft-capped logits [B, T, V] in the parameter dtype."""
    B, T = input_seq.shape
    d, H, D, L = cfg.model_dim, cfg.n_head, cfg.head_dim, cfg.n_layer
    dt = p["embed"].dtype

    def norm(x):
        return rms_norm_ref(x).to(dt)

    tok = F.embedding(input_seq, p["embed"])
    gate = torch.sigmoid(F.linear(tok[..., :12], p["smearGate.weight"].to(dt)))
    x0 = norm(tok + tok * gate)
    ves = [F.embedding(input_seq, p[f"valueEmbeds.{i}"]) for i in range(cfg.num_value_embeds)]
    sc = p["scalars.values"].float()
    sg = lambda i: torch.sigmoid(sc[i]).to(dt)
    value_mix, skip_mix, final_scale = sg(L * 4), sg(L * 4 + 1), sg(L * 4 + 2)
    x = x0
    skip = None
    for i in range(L):
        lam_x, lam_x0, lam_attn, lam_mlp = sg(4 * i), sg(4 * i + 1), sg(4 * i + 2), sg(4 * i + 3)
        x_in = x * lam_x + x0 * lam_x0
        if i == SKIP_SOURCE_LAYER:
            skip = x_in
        window = get_window_size_for_layer(cfg.window_pattern, i, L, T)
        if f"blocks.{i}.attn.wQ" in p:
            xn = norm(x_in)
            q = F.linear(xn, p[f"blocks.{i}.attn.wQ"])
            k = F.linear(xn, p[f"blocks.{i}.attn.wK"])
            v = F.linear(xn, p[f"blocks.{i}.attn.wV"])
            vi = layer_value_embed_index(cfg, i)
            if vi is not None:
                v = v * (1 - value_mix) + ves[vi] * value_mix
            q = q.reshape(B, T, H, D)
            k = k.reshape(B, T, H, D)
            v = v.reshape(B, T, H, D)
            q = norm(ops.apply_rotary(q, cos[:T], sin[:T]))
            k = norm(ops.apply_rotary(k, cos[:T], sin[:T]))
            o = ops.attention_ref(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                  causal=True, window=window)
            o = o.transpose(1, 2).reshape(B, T, H * D)
            x1 = x_in + F.linear(o, p[f"blocks.{i}.attn.wO"]) * lam_attn
            xn2 = norm(x1)
            h = F.linear(xn2, p[f"blocks.{i}.mlp.cFc"])
            h = torch.relu(h)
            h = h * h
            x = x1 + (h @ p[f"blocks.{i}.mlp.cProj"]) * lam_mlp
        else:
            x = x_in + skip * skip_mix if skip is not None else x_in
            xn = norm(x)
            h = torch.relu(F.linear(xn, p[f"blocks.{i}.mlp.cFc"]))
            h = h * h
            x = x + (h @ p[f"blocks.{i}.mlp.cProj"]) * lam_mlp
    xn = norm(x * final_scale)
    logits = F.linear(xn, p["lmHead.weight"])
    return (torch.tanh(logits.float() / cfg.softcap_value) * cfg.softcap_value).to(dt)


def loss_reference(p, cfg, input_seq, targets, cos, sin) -> torch.Tensor:
    logits = forward_reference(p, cfg, input_seq, cos, sin)
    return F.cross_entropy(logits.float().reshape(-1, cfg.vocab_size), targets.reshape(-1))
