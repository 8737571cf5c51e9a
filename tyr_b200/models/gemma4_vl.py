"""Gemma 4 multimodal wrapper: a ViT over a grid of image patches (optionally clipped linears, learned x / y position
tables, 2-D rotary attention with Q/K RMSNorm, GELU-gated MLP, average pooling to the soft-token grid), a projector into
the text width, and the text model run from embeddings with the image placeholders replaced.  With
``use_bidirectional_attention == "vision"`` the tokens of one image attend to each other in both directions during prefill
(Tyr/Model/Gemma4/{VLConfig,VLConfigIO,Multimodal,VLWeights,Media}.lean)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..io import safetensors as st
from ..ops.rope import apply_rotary, rotary_freqs
from . import gemma4 as G
from .generation import SamplingStrategy, generate_cached


@dataclass
class VisionConfig:
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_hidden_layers: int = 16
    num_attention_heads: int = 12
    num_key_value_heads: int = 12
    quarter_head_dim: int = 16
    patch_size: int = 16
    pooling_kernel_size: int = 3
    position_embedding_size: int = 10240
    rms_norm_eps: float = 1e-6
    rope_theta: float = 100.0
    standardize: bool = False
    use_clipped_linears: bool = False

    def __post_init__(self):
        hd = 4 * self.quarter_head_dim
        if self.quarter_head_dim <= 0 or self.num_attention_heads * hd != self.hidden_size or self.num_key_value_heads * hd != self.hidden_size:
            raise ValueError("Invalid Gemma4 vision config: hidden_size must split into heads of 4 * quarter_head_dim channels")
        if self.num_attention_heads % self.num_key_value_heads or self.patch_size <= 0 or self.pooling_kernel_size <= 0:
            raise ValueError("Invalid Gemma4 vision config: head grouping, patch size or pooling window")

    @property
    def head_dim(self): return 4 * self.quarter_head_dim
    @property
    def patch_dim(self): return 3 * self.patch_size ** 2


@dataclass
class ImageProcessorConfig:
    do_resize: bool = True
    do_rescale: bool = True
    do_normalize: bool = False
    image_seq_length: int = 280
    max_soft_tokens: int = 280
    patch_size: int = 16
    pooling_kernel_size: int = 3
    rescale_factor: float = 1.0 / 255.0

    def soft_token_count(self) -> int:
        return self.max_soft_tokens if self.max_soft_tokens > 0 else self.image_seq_length


@dataclass
class VLConfig:
    text_config: G.Gemma4Config = field(default_factory=G.Gemma4Config)
    vision_config: VisionConfig = field(default_factory=VisionConfig)
    image_processor: ImageProcessorConfig = field(default_factory=ImageProcessorConfig)
    boi_token_id: int = 255999
    image_token_id: int = 258880
    eoi_token_id: int = 258882
    video_token_id: int = 258884
    audio_token_id: int = 258881
    vision_soft_tokens_per_image: int = 280

    @staticmethod
    def from_json(j: dict) -> "VLConfig":
        d, vj = VLConfig(), j.get("vision_config", {})
        dv = VisionConfig()
        g = lambda k: vj.get(k, getattr(dv, k))
        hs, nh = g("hidden_size"), g("num_attention_heads")
        vis = VisionConfig(hs, g("intermediate_size"), g("num_hidden_layers"), nh, g("num_key_value_heads"), vj.get("head_dim", hs // nh) // 4, g("patch_size"),
                           g("pooling_kernel_size"), g("position_embedding_size"), float(g("rms_norm_eps")), float((vj.get("rope_parameters") or {}).get("rope_theta", dv.rope_theta)),
                           bool(g("standardize")), bool(g("use_clipped_linears")))
        t = lambda k: j.get(k, getattr(d, k))
        return VLConfig(G.Gemma4Config.from_json(j), vis, ImageProcessorConfig(), t("boi_token_id"), t("image_token_id"), t("eoi_token_id"), t("video_token_id"),
                        t("audio_token_id"), t("vision_soft_tokens_per_image"))


def rms_no_scale(x, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)


def rms_weighted(x, w, eps):
    return (rms_no_scale(x.float(), eps) * w.float()).to(x.dtype)


def rotary_2d(x: torch.Tensor, rows: int, cols: int, theta: float) -> torch.Tensor:
    """x: [1, rows*cols, H, 4q]: the first half of each head rotates with the patch's column, the second with its row."""
    q = x.shape[-1] // 4
    idx = torch.arange(rows * cols, device=x.device)
    xc, xs = rotary_freqs(cols, 2 * q, theta, x.device)
    yc, ys = rotary_freqs(rows, 2 * q, theta, x.device)
    xi, yi = idx % cols, idx // cols
    return torch.cat([apply_rotary(x[..., :2 * q], xc[xi], xs[xi]), apply_rotary(x[..., 2 * q:], yc[yi], ys[yi])], -1)


@dataclass
class VisionModel:
    cfg: VisionConfig
    p: Dict[str, torch.Tensor]
    clip: Dict[str, Tuple[Optional[float], Optional[float], Optional[float], Optional[float]]] = field(default_factory=dict)

    def _lin(self, x, name):
        lo_i, hi_i, lo_o, hi_o = self.clip.get(name, (None, None, None, None))
        w = self.p[name + ".weight"]
        x = x.to(w.dtype)
        if lo_i is not None or hi_i is not None:
            x = x.clamp(lo_i, hi_i)
        y = F.linear(x, w)
        return y.clamp(lo_o, hi_o) if lo_o is not None or hi_o is not None else y

    @torch.no_grad()
    def forward(self, grid: torch.Tensor) -> torch.Tensor:
        """grid: [rows, cols, patch_dim] with pixels in [0, 1] -> pooled fp32 features [(rows/pool) * (cols/pool), hidden]."""
        c, p = self.cfg, self.p
        rows, cols, _ = grid.shape
        n = rows * cols
        idx = torch.arange(n, device=grid.device)
        tab = p["patch_embedder.position_embedding_table"].float()
        x = self._lin((grid.reshape(n, -1) - 0.5) * 2.0, "patch_embedder.input_proj").float() + tab[0][idx % cols] + tab[1][idx // cols]
        H, Hkv, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        for i in range(c.num_hidden_layers):
            L = f"encoder.layers.{i}."
            h = rms_weighted(x, p[L + "input_layernorm.weight"], c.rms_norm_eps)
            q = rms_weighted(self._lin(h, L + "self_attn.q_proj").reshape(1, n, H, D), p[L + "self_attn.q_norm.weight"], c.rms_norm_eps)
            k = rms_weighted(self._lin(h, L + "self_attn.k_proj").reshape(1, n, Hkv, D), p[L + "self_attn.k_norm.weight"], c.rms_norm_eps)
            v = rms_no_scale(self._lin(h, L + "self_attn.v_proj").reshape(1, n, Hkv, D), c.rms_norm_eps)
            q, k = rotary_2d(q, rows, cols, c.rope_theta).transpose(1, 2), rotary_2d(k, rows, cols, c.rope_theta).transpose(1, 2)
            a = F.scaled_dot_product_attention(q, k, v.transpose(1, 2), scale=1.0, enable_gqa=H != Hkv).transpose(1, 2).reshape(n, H * D)
            x = x + rms_weighted(self._lin(a, L + "self_attn.o_proj"), p[L + "post_attention_layernorm.weight"], c.rms_norm_eps).float()
            h = rms_weighted(x, p[L + "pre_feedforward_layernorm.weight"], c.rms_norm_eps)
            mlp = self._lin(F.gelu(self._lin(h, L + "mlp.gate_proj")) * self._lin(h, L + "mlp.up_proj"), L + "mlp.down_proj")
            x = x + rms_weighted(mlp, p[L + "post_feedforward_layernorm.weight"], c.rms_norm_eps).float()
        pool = c.pooling_kernel_size
        g = F.avg_pool2d(x.reshape(1, rows, cols, -1).permute(0, 3, 1, 2), pool).permute(0, 2, 3, 1).reshape(-1, c.hidden_size) * math.sqrt(c.hidden_size)
        if "std_bias" in p and "std_scale" in p:
            g = (g - p["std_bias"].float()) * p["std_scale"].float()
        return g


def vision_shapes(c: VisionConfig) -> Dict[str, tuple]:
    s = {"patch_embedder.input_proj.weight": (c.hidden_size, c.patch_dim), "patch_embedder.position_embedding_table": (2, c.position_embedding_size, c.hidden_size)}
    for i in range(c.num_hidden_layers):
        L = f"encoder.layers.{i}."
        for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
            s[L + f"self_attn.{n}.weight"] = (c.hidden_size, c.hidden_size)
        s[L + "self_attn.q_norm.weight"] = s[L + "self_attn.k_norm.weight"] = (c.head_dim,)
        s[L + "mlp.gate_proj.weight"] = s[L + "mlp.up_proj.weight"] = (c.intermediate_size, c.hidden_size)
        s[L + "mlp.down_proj.weight"] = (c.hidden_size, c.intermediate_size)
        for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
            s[L + n + ".weight"] = (c.hidden_size,)
    return s


def init_vision(c: VisionConfig, device="cpu", dtype=torch.float32, seed=0) -> VisionModel:
    g = torch.Generator().manual_seed(seed)
    p = {}
    for name, shape in vision_shapes(c).items():
        if "norm" in name:
            t = torch.ones(shape)
        elif name.endswith("position_embedding_table"):
            t = torch.randn(shape, generator=g) * 0.02
        else:
            t = torch.randn(shape, generator=g) * shape[-1] ** -0.5
        p[name] = t.to(device=device, dtype=dtype)
    return VisionModel(c, p)


def patch_grid(image: torch.Tensor, patch: int) -> torch.Tensor:
    """image: [3, H, W] in [0, 1] -> [H/patch, W/patch, 3*patch*patch] (channel-major inside a patch)."""
    C, H, W = image.shape
    if H % patch or W % patch:
        raise ValueError("image height and width must be multiples of the patch size")
    x = image.reshape(C, H // patch, patch, W // patch, patch).permute(1, 3, 0, 2, 4)
    return x.reshape(H // patch, W // patch, C * patch * patch)


def vision_group_masks(ids: torch.Tensor, image_token_id: int, pad_id: int, sliding_window: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(sliding, full) [B, S, S] masks (True = may attend): causal (within the window for sliding layers) among non-pad
    tokens, plus every pair of tokens that belong to the same run of image placeholders."""
    B, S = ids.shape
    is_img = ids == image_token_id
    start = is_img & ~F.pad(is_img, (1, 0))[:, :S]
    group = torch.where(is_img, torch.cumsum(start.long(), 1), torch.full_like(ids, -1))
    valid = ids != pad_id
    q, k = torch.arange(S, device=ids.device)[:, None], torch.arange(S, device=ids.device)[None, :]
    base = valid[:, :, None] & valid[:, None, :] & (k <= q)[None]
    same = (group[:, :, None] >= 0) & (group[:, :, None] == group[:, None, :])
    return (base & ((q - k) < sliding_window)[None]) | same, base | same


@dataclass
class Gemma4VL:
    cfg: VLConfig
    vision_tower: VisionModel
    embedding_projection: torch.Tensor          # [text hidden, vision hidden]
    language_model: G.Gemma4ForCausalLM

    def get_image_features(self, grid: torch.Tensor) -> torch.Tensor:
        v = self.vision_tower.forward(grid.to(self.embedding_projection.device))
        return F.linear(rms_no_scale(v, self.cfg.text_config.rms_norm_eps).to(self.embedding_projection.dtype), self.embedding_projection)

    def get_image_features_many(self, grids: Sequence[torch.Tensor]) -> Optional[torch.Tensor]:
        return torch.cat([self.get_image_features(g) for g in grids], 0) if grids else None

    @staticmethod
    def repeat_features_for_batch(features: torch.Tensor, batch: int) -> torch.Tensor:
        return features if batch <= 1 else features.repeat(batch, 1)

    def build_inputs(self, input_ids: torch.Tensor, image_features: Optional[torch.Tensor]):
        """(embeddings, per-layer inputs): the placeholders are embedded as the pad token (their per-layer inputs too) and
        then overwritten by the image features."""
        lm, c = self.language_model, self.cfg
        text_ids = torch.where(input_ids == c.image_token_id, torch.full_like(input_ids, c.text_config.pad_token_id or 0), input_ids)
        emb = G.embed_tokens(lm, text_ids)
        pli = G.compute_per_layer_inputs(lm, text_ids, emb)
        if image_features is not None:
            mask = input_ids == c.image_token_id
            n = int(mask.sum())
            if n != image_features.shape[0]:
                raise ValueError(f"placeholder token count mismatch: ids={n} features={image_features.shape[0]}")
            emb = emb.clone()
            emb[mask] = image_features.to(emb.dtype)
        return emb, pli

    def _masks(self, input_ids):
        c = self.cfg
        if c.text_config.use_bidirectional_attention != "vision":
            return None
        return vision_group_masks(input_ids, c.image_token_id, c.text_config.pad_token_id or 0, c.text_config.sliding_window)

    @torch.no_grad()
    def forward(self, input_ids, image_features=None) -> torch.Tensor:
        if image_features is None:
            return G.forward(self.language_model, input_ids)
        emb, pli = self.build_inputs(input_ids, image_features)
        return G.forward(self.language_model, input_ids, emb, pli, self._masks(input_ids))

    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens=256, strategy=SamplingStrategy.greedy(), eos_token_ids: Optional[Sequence[int]] = None, image_features=None,
                 on_step=None):
        lm = self.language_model
        emb, pli = self.build_inputs(input_ids, image_features)
        masks = self._masks(input_ids) if image_features is not None else None
        cache = G.Gemma4Cache(lm, input_ids.shape[0], input_ids.shape[1] + max_new_tokens)
        eos = lm.cfg.eos_token_id if eos_token_ids is None else eos_token_ids
        return generate_cached(lambda ids: cache.run(ids, emb, pli, masks), cache.step, input_ids, max_new_tokens, strategy, eos, on_step)


def init(cfg: VLConfig, device="cpu", dtype=torch.float32, seed=0) -> Gemma4VL:
    g = torch.Generator().manual_seed(seed + 9)
    proj = (torch.randn(cfg.text_config.hidden_size, cfg.vision_config.hidden_size, generator=g) * cfg.vision_config.hidden_size ** -0.5).to(device=device, dtype=dtype)
    return Gemma4VL(cfg, init_vision(cfg.vision_config, device, dtype, seed + 1), proj, G.init(cfg.text_config, device, dtype, seed))


def load(cfg: VLConfig, source, device="cpu", dtype=torch.bfloat16, vision_dtype: Optional[torch.dtype] = None) -> Gemma4VL:
    src = source if isinstance(source, st.Source) else st.Source.open(source)
    vd = vision_dtype or dtype

    def find(name):
        return next((c for c in (f"model.{name}", name) if src.find(c) is not None), None)
    p, clip = {}, {}
    for name, shape in vision_shapes(cfg.vision_config).items():
        base = "vision_tower." + name
        if name.endswith(".weight") and "norm" not in name and find(base) is None and find(base[:-7] + ".linear.weight") is not None:
            base = base[:-7] + ".linear.weight"                     # clipped linears wrap the plain weight
        f = find(base)
        if f is None:
            raise st.SafeTensorsError(f"missing vision tensor {name}")
        t = src.load(f)
        if tuple(t.shape) != tuple(shape):
            raise st.SafeTensorsError(f"vision tensor {name} has shape {tuple(t.shape)}, expected {tuple(shape)}")
        p[name] = t.to(device=device, dtype=vd)
        if cfg.vision_config.use_clipped_linears and name.endswith(".weight") and "norm" not in name:
            lin_name = name[:-7]
            vals = []
            for k in ("input_min", "input_max", "output_min", "output_max"):
                fk = find(f"vision_tower.{lin_name}.{k}")
                vals.append(float(src.load(fk).reshape(-1)[0]) if fk is not None else None)
            if any(v is not None for v in vals):
                clip[lin_name] = tuple(vals)
    for extra in ("std_bias", "std_scale"):
        f = find("vision_tower." + extra)
        if f is not None:
            p[extra] = src.load(f).to(device=device, dtype=vd)
    f = find("embed_vision.embedding_projection.weight")
    if f is None:
        raise st.SafeTensorsError("missing tensor embed_vision.embedding_projection.weight")
    return Gemma4VL(cfg, VisionModel(cfg.vision_config, p, clip), src.load(f).to(device=device, dtype=dtype), G.load(cfg.text_config, src, device, dtype))
