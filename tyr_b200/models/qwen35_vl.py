"""Qwen3.5 / 3.6 multimodal wrapper: a ViT over patchified pixels (linear patch embedding, learned positions, rotary
attention over the patch index, GELU MLP, 2x2 patch merger to the text width) whose outputs replace the image / video
placeholder embeddings of the text model (Tyr/Model/Qwen35/{VLConfig,VLConfigIO,Multimodal,VLWeights,Media}.lean).

Media decoding is Apple-only in the reference (cc/src/apple_vl_processor.mm); here ``patchify`` cuts tensors that the
caller has already decoded."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from ..io import safetensors as st
from ..ops.rope import apply_rotary, rotary_freqs
from . import qwen35 as Q
from .generation import SamplingStrategy, generate_cached


@dataclass
class VisionConfig:
    depth: int = 27
    hidden_size: int = 1152
    hidden_act: str = "gelu_pytorch_tanh"
    intermediate_size: int = 4304
    num_heads: int = 16
    half_head_dim: int = 36
    in_channels: int = 3
    patch_size: int = 16
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2
    out_hidden_size: int = 3584
    num_position_embeddings: int = 2304

    def __post_init__(self):
        if self.num_heads <= 0 or self.num_heads * 2 * self.half_head_dim != self.hidden_size:
            raise ValueError("Invalid Qwen3.5 vision config: hidden_size must split into num_heads heads of even width")
        if self.spatial_merge_size <= 0:
            raise ValueError("Invalid Qwen3.5 vision config: spatial_merge_size must be positive")

    @property
    def patch_dim(self): return self.in_channels * self.temporal_patch_size * self.patch_size ** 2
    @property
    def merge_unit(self): return self.spatial_merge_size ** 2
    @property
    def head_dim(self): return 2 * self.half_head_dim

    @staticmethod
    def qwen35_0_8b(): return VisionConfig(12, 768, "gelu_pytorch_tanh", 3072, 12, 32, 3, 16, 2, 2, 1024, 2304)
    @staticmethod
    def qwen36_35b_a3b(): return VisionConfig(out_hidden_size=2048)

    @staticmethod
    def from_json(j: dict, defaults: Optional["VisionConfig"] = None) -> "VisionConfig":
        d = defaults or VisionConfig()
        g = lambda k: j.get(k, getattr(d, k))
        hs, nh = g("hidden_size"), g("num_heads")
        return VisionConfig(g("depth"), hs, g("hidden_act"), g("intermediate_size"), nh, hs // nh // 2, g("in_channels"), g("patch_size"),
                            g("spatial_merge_size"), g("temporal_patch_size"), g("out_hidden_size"), g("num_position_embeddings"))


@dataclass
class VLConfig:
    text_config: Q.Qwen35Config = field(default_factory=Q.Qwen35Config.qwen35_0_8b)
    vision_config: VisionConfig = field(default_factory=VisionConfig.qwen35_0_8b)
    image_token_id: int = 248056
    video_token_id: int = 248057
    vision_start_token_id: int = 248053
    vision_end_token_id: int = 248054
    tie_word_embeddings: bool = False

    def __post_init__(self):
        if self.vision_config.out_hidden_size != self.text_config.hidden_size:
            raise ValueError("Invalid Qwen3.5 VL config: vision features must have the text hidden size")

    @staticmethod
    def from_json(j: dict) -> "VLConfig":
        d = VLConfig()
        return VLConfig(Q.Qwen35Config.from_json(j.get("text_config", {})), VisionConfig.from_json(j.get("vision_config", {})),
                        j.get("image_token_id", d.image_token_id), j.get("video_token_id", d.video_token_id),
                        j.get("vision_start_token_id", d.vision_start_token_id), j.get("vision_end_token_id", d.vision_end_token_id),
                        bool(j.get("tie_word_embeddings", False)))


@dataclass
class VisionModel:
    cfg: VisionConfig
    p: Dict[str, torch.Tensor]

    @torch.no_grad()
    def forward(self, patches: torch.Tensor) -> torch.Tensor:
        """patches: [n, patch_dim] -> [n / merge_unit, out_hidden_size]."""
        c, p = self.cfg, self.p
        n = patches.shape[0]
        if n > c.num_position_embeddings:
            raise ValueError(f"vision patch count ({n}) exceeds num_position_embeddings ({c.num_position_embeddings})")
        if n % c.merge_unit:
            raise ValueError(f"vision token count ({n}) must be divisible by merge unit ({c.merge_unit})")
        w = p["patch_embed.proj.weight"]
        x = F.linear(patches.to(w.dtype), w.reshape(c.hidden_size, -1), p["patch_embed.proj.bias"]) + p["pos_embed.weight"][:n]
        cos, sin = rotary_freqs(n, c.head_dim, 10000.0, x.device)
        act = (lambda t: F.gelu(t, approximate="tanh")) if c.hidden_act == "gelu_pytorch_tanh" else F.gelu
        for i in range(c.depth):
            b = f"blocks.{i}."
            h = F.layer_norm(x, (c.hidden_size,), p[b + "norm1.weight"], p[b + "norm1.bias"], 1e-6)
            q, k, v = F.linear(h, p[b + "attn.qkv.weight"], p[b + "attn.qkv.bias"]).reshape(1, n, 3, c.num_heads, c.head_dim).unbind(2)
            q, k = apply_rotary(q, cos, sin), apply_rotary(k, cos, sin)
            a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).reshape(n, c.hidden_size)
            x = x + F.linear(a, p[b + "attn.proj.weight"], p[b + "attn.proj.bias"])
            h = F.layer_norm(x, (c.hidden_size,), p[b + "norm2.weight"], p[b + "norm2.bias"], 1e-6)
            x = x + F.linear(act(F.linear(h, p[b + "mlp.linear_fc1.weight"], p[b + "mlp.linear_fc1.bias"])), p[b + "mlp.linear_fc2.weight"], p[b + "mlp.linear_fc2.bias"])
        x = F.layer_norm(x, (c.hidden_size,), p["merger.norm.weight"], p["merger.norm.bias"], 1e-6).reshape(n // c.merge_unit, c.hidden_size * c.merge_unit)
        return F.linear(F.gelu(F.linear(x, p["merger.linear_fc1.weight"], p["merger.linear_fc1.bias"])), p["merger.linear_fc2.weight"], p["merger.linear_fc2.bias"])


def vision_shapes(c: VisionConfig) -> Dict[str, tuple]:
    s = {"patch_embed.proj.weight": (c.hidden_size, c.in_channels, c.temporal_patch_size, c.patch_size, c.patch_size), "patch_embed.proj.bias": (c.hidden_size,),
         "pos_embed.weight": (c.num_position_embeddings, c.hidden_size)}
    mh = c.hidden_size * c.merge_unit
    for i in range(c.depth):
        b = f"blocks.{i}."
        for n in ("norm1", "norm2"):
            s[b + n + ".weight"], s[b + n + ".bias"] = (c.hidden_size,), (c.hidden_size,)
        s[b + "attn.qkv.weight"], s[b + "attn.qkv.bias"] = (3 * c.hidden_size, c.hidden_size), (3 * c.hidden_size,)
        s[b + "attn.proj.weight"], s[b + "attn.proj.bias"] = (c.hidden_size, c.hidden_size), (c.hidden_size,)
        s[b + "mlp.linear_fc1.weight"], s[b + "mlp.linear_fc1.bias"] = (c.intermediate_size, c.hidden_size), (c.intermediate_size,)
        s[b + "mlp.linear_fc2.weight"], s[b + "mlp.linear_fc2.bias"] = (c.hidden_size, c.intermediate_size), (c.hidden_size,)
    s["merger.norm.weight"], s["merger.norm.bias"] = (c.hidden_size,), (c.hidden_size,)
    s["merger.linear_fc1.weight"], s["merger.linear_fc1.bias"] = (mh, mh), (mh,)
    s["merger.linear_fc2.weight"], s["merger.linear_fc2.bias"] = (c.out_hidden_size, mh), (c.out_hidden_size,)
    return s


def init_vision(c: VisionConfig, device="cpu", dtype=torch.float32, seed=0) -> VisionModel:
    g = torch.Generator().manual_seed(seed)
    p = {}
    for name, shape in vision_shapes(c).items():
        if name.endswith(".bias"):
            t = torch.zeros(shape)
        elif "norm" in name:
            t = torch.ones(shape)
        elif name == "pos_embed.weight":
            t = torch.randn(shape, generator=g) * 0.02
        else:
            fan = 1
            for d in shape[1:]:
                fan *= d
            t = torch.randn(shape, generator=g) * fan ** -0.5
        p[name] = t.to(device=device, dtype=dtype)
    return VisionModel(c, p)


def patchify(pixels: torch.Tensor, c: VisionConfig) -> torch.Tensor:
    """pixels: [frames, channels, H, W] (frames a multiple of ``temporal_patch_size``; one image = the frame repeated) ->
    ``[n_patches, patch_dim]`` with patches ordered so that each run of ``merge_unit`` rows is one 2x2 spatial group."""
    Tn, C, H, W = pixels.shape
    ps, tp, m = c.patch_size, c.temporal_patch_size, c.spatial_merge_size
    if Tn % tp or H % (ps * m) or W % (ps * m) or C != c.in_channels:
        raise ValueError("patchify: frames / height / width must be multiples of the temporal and (patch x merge) sizes")
    gh, gw = H // ps, W // ps
    x = pixels.reshape(Tn // tp, tp, C, gh // m, m, ps, gw // m, m, ps)
    x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)               # [t, gh/m, gw/m, m, m, C, tp, ps, ps]
    return x.reshape(-1, C * tp * ps * ps)


@dataclass
class Qwen35VL:
    cfg: VLConfig
    visual: VisionModel
    language_model: Q.Qwen35ForCausalLM

    def get_image_features(self, patches): return self.visual.forward(patches)
    def get_video_features(self, patches): return self.visual.forward(patches)

    def build_inputs_embeds(self, input_ids, image_features=None, video_features=None) -> torch.Tensor:
        emb = F.embedding(input_ids, self.language_model.embed_tokens).clone()
        for tok, feats in ((self.cfg.image_token_id, image_features), (self.cfg.video_token_id, video_features)):
            if feats is None:
                continue
            mask = input_ids == tok
            n = int(mask.sum())
            if n != feats.shape[0]:
                raise ValueError(f"placeholder token count mismatch for token={tok}: ids={n} features={feats.shape[0]}")
            emb[mask] = feats.to(emb.dtype)
        return emb

    @torch.no_grad()
    def forward(self, input_ids, image_patches=None, video_patches=None, attn_mask=None) -> torch.Tensor:
        fi = self.get_image_features(image_patches) if image_patches is not None else None
        fv = self.get_video_features(video_patches) if video_patches is not None else None
        if fi is None and fv is None:
            return Q.forward(self.language_model, input_ids, attn_mask)
        return Q.forward(self.language_model, None, attn_mask, self.build_inputs_embeds(input_ids, fi, fv))

    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens=256, strategy=SamplingStrategy.greedy(), eos_token_ids: Sequence[int] = (), image_features=None,
                 video_features=None, on_step=None):
        """Cached generation: the features enter once, at prefill, through the embeddings."""
        lm = self.language_model
        emb = self.build_inputs_embeds(input_ids, image_features, video_features)
        cache = Q.HybridCache(lm, input_ids.shape[0], input_ids.shape[1] + max_new_tokens)
        return generate_cached(lambda ids: cache.run(emb), cache.step, input_ids, max_new_tokens, strategy, eos_token_ids, on_step)


def init(cfg: VLConfig, device="cpu", dtype=torch.float32, seed=0) -> Qwen35VL:
    lm = Q.init(cfg.text_config, device, dtype, seed)
    return Qwen35VL(cfg, init_vision(cfg.vision_config, device, dtype, seed + 1), lm)


def load(cfg: VLConfig, source, device="cpu", dtype=torch.bfloat16, vision_dtype: Optional[torch.dtype] = None) -> Qwen35VL:
    """Vision tensors are found under ``model.visual.`` or ``visual.``; the text model under the usual names."""
    src = source if isinstance(source, st.Source) else st.Source.open(source)
    vd = vision_dtype or dtype
    p = {}
    for name, shape in vision_shapes(cfg.vision_config).items():
        found = next((c for c in (f"model.visual.{name}", f"visual.{name}") if src.find(c) is not None), None)
        if found is None:
            raise st.SafeTensorsError(f"missing vision tensor {name}")
        t = src.load(found)
        if tuple(t.shape) != tuple(shape):
            raise st.SafeTensorsError(f"vision tensor {name} has shape {tuple(t.shape)}, expected {tuple(shape)}")
        p[name] = t.to(device=device, dtype=vd)
    return Qwen35VL(cfg, VisionModel(cfg.vision_config, p), Q.load(cfg.text_config, src, device, dtype))
