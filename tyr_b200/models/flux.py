"""Flux (Klein 4B) rectified-flow DiT: model-level modulation, double- and single-stream blocks with
joint text+image attention, 4-axis RoPE, Flux2 SNR-shift schedule with Euler sampling, latent pack/unpack.

Contract: Tyr/Model/Flux/{Config,Modulation,QKNorm,RoPE,DoubleStreamBlock,SingleStreamBlock,Model,
Sampling,Weights}.lean.  On the GPU the LayerNorm+modulation and gated-residual steps run as single
fused kernels (csrc/modulate.cu), projections on the tcgen05 GEMM and attention on the flash kernel.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..io import safetensors as st
from ..ops.attention import attention
from ..ops import flash as _flash
from ..ops.gemm import gemm as _gemm, interleave_gate_up
from ..ops.modulate import flux_qk_post, flux_qk_post_supported, gate_residual, layernorm_modulate
from ..ops.norm import rms_norm_weighted
from .common import lin


@dataclass
class FluxConfig:
    hidden_size: int = 3072
    num_heads: int = 24
    half_head_dim: int = 64
    num_double_layers: int = 5
    num_single_layers: int = 20
    context_in_dim: int = 7680
    in_channels: int = 128
    time_dim: int = 256
    mlp_hidden_dim: int = 9216
    theta: int = 2000
    half_axes_dims: Tuple[int, ...] = (16, 16, 16, 16)

    def __post_init__(self):
        if len(self.half_axes_dims) != 4 or sum(self.half_axes_dims) != self.half_head_dim:
            raise ValueError("Invalid Flux config: four RoPE axis halves must sum to half_head_dim")
        if self.theta <= 0:
            raise ValueError("Invalid Flux config: theta must be positive")

    @property
    def head_dim(self) -> int:
        return 2 * self.half_head_dim

    @staticmethod
    def klein4b() -> "FluxConfig":
        return FluxConfig()


def timestep_embedding(t: torch.Tensor, dim: int, max_period: float = 10000.0, time_factor: float = 1000.0) -> torch.Tensor:
    """Sinusoidal embedding [batch, dim] (cos half first), fp32."""
    t = t.float() * time_factor
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t[:, None] * freqs[None]
    emb = torch.cat([torch.cos(args), torch.sin(args)], dim=-1)
    if dim % 2:
        emb = torch.cat([emb, torch.zeros_like(emb[:, :1])], dim=-1)
    return emb


def rope_embed(ids: torch.Tensor, half_axes_dims: Sequence[int], theta: int = 2000) -> Tuple[torch.Tensor, torch.Tensor]:
    """ids: int64 [B, S, 4] -> (cos, sin) fp32 [B, S, half_head_dim]; axis a owns ``half_axes_dims[a]`` pairs with
    ``omega_j = theta^(-2j / (2*half_a))``.  Equivalent to the 2x2 rotation matrices of RoPE.lean:10-56."""
    cos, sin = [], []
    for a, half in enumerate(half_axes_dims):
        scale = torch.arange(half, dtype=torch.float32, device=ids.device) * (2.0 / (2 * half))
        omega = torch.exp(scale * (-math.log(float(theta))))
        ang = ids[..., a].float().unsqueeze(-1) * omega
        cos.append(torch.cos(ang))
        sin.append(torch.sin(ang))
    return torch.cat(cos, -1), torch.cat(sin, -1)


def apply_rope(x: torch.Tensor, pe: Tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
    """x: [B, S, H, 2*half] with interleaved pairs (x0, x1) -> (cos x0 - sin x1, sin x0 + cos x1), fp32 math."""
    cos, sin = pe
    B, S, H, D = x.shape
    xf = x.float().reshape(B, S, H, D // 2, 2)
    c, s = cos[:, :, None, :], sin[:, :, None, :]
    o0 = c * xf[..., 0] - s * xf[..., 1]
    o1 = s * xf[..., 0] + c * xf[..., 1]
    return torch.stack([o0, o1], dim=-1).reshape(B, S, H, D).to(x.dtype)


@dataclass
class QKNorm:
    query_norm: torch.Tensor
    key_norm: torch.Tensor


@dataclass
class SelfAttention:
    qkv: torch.Tensor
    norm: QKNorm
    proj: torch.Tensor


@dataclass
class SwiGLUMLP:
    w1: torch.Tensor   # [2*mlp, hidden]: gate rows then up rows
    w2: torch.Tensor


@dataclass
class DoubleStreamBlock:
    img_attn: SelfAttention
    img_mlp: SwiGLUMLP
    txt_attn: SelfAttention
    txt_mlp: SwiGLUMLP


@dataclass
class SingleStreamBlock:
    linear1: torch.Tensor   # [3*hidden + 2*mlp, hidden]
    linear2: torch.Tensor   # [hidden, hidden + mlp]
    norm: QKNorm


@dataclass
class FluxModel:
    cfg: FluxConfig
    img_in: torch.Tensor
    txt_in: torch.Tensor
    time_in_layer: torch.Tensor
    time_out_layer: torch.Tensor
    double_blocks: List[DoubleStreamBlock]
    single_blocks: List[SingleStreamBlock]
    double_stream_modulation_img: torch.Tensor   # [6*hidden, hidden]
    double_stream_modulation_txt: torch.Tensor
    single_stream_modulation: torch.Tensor       # [3*hidden, hidden]
    final_linear: torch.Tensor
    final_modulation: torch.Tensor               # [2*hidden, hidden]

    @property
    def dtype(self): return self.img_in.dtype
    @property
    def device(self): return self.img_in.device


EPS = 1e-6


def init(cfg: FluxConfig, device="cpu", dtype=torch.float32, seed=0) -> FluxModel:
    gen = torch.Generator().manual_seed(seed)
    h, D, H, M = cfg.hidden_size, cfg.head_dim, cfg.num_heads, cfg.mlp_hidden_dim
    std = math.sqrt(2.0 / h)
    mk = lambda *shape, s=std: (torch.randn(shape, generator=gen) * s).to(device=device, dtype=dtype)
    ones = lambda n: torch.ones(n, device=device, dtype=dtype)
    qkn = lambda: QKNorm(ones(D), ones(D))
    sa = lambda: SelfAttention(mk(H * D * 3, h), qkn(), mk(h, H * D))
    mlp = lambda: SwiGLUMLP(mk(2 * M, h), mk(h, M))
    return FluxModel(cfg, mk(h, cfg.in_channels), mk(h, cfg.context_in_dim), mk(h, cfg.time_dim, s=math.sqrt(2.0 / cfg.time_dim)),
                     mk(h, h, s=math.sqrt(2.0 / cfg.time_dim)),
                     [DoubleStreamBlock(sa(), mlp(), sa(), mlp()) for _ in range(cfg.num_double_layers)],
                     [SingleStreamBlock(mk(3 * H * D + 2 * M, h), mk(h, H * D + M), qkn()) for _ in range(cfg.num_single_layers)],
                     mk(6 * h, h), mk(6 * h, h), mk(3 * h, h), mk(cfg.in_channels, h), mk(2 * h, h))


def modulation(vec: torch.Tensor, w: torch.Tensor, n: int) -> torch.Tensor:
    """silu(vec) @ w^T -> [B, n, hidden]."""
    return lin(F.silu(vec), w).reshape(vec.shape[0], n, -1)


def _qk(cfg, qkv, norm: QKNorm, pe):
    B, S, _ = qkv.shape
    H, D = cfg.num_heads, cfg.head_dim
    x = qkv.reshape(B, S, 3, H, D)
    q = rms_norm_weighted(x[:, :, 0].contiguous(), norm.query_norm, EPS)
    k = rms_norm_weighted(x[:, :, 1].contiguous(), norm.key_norm, EPS)
    return apply_rope(q, pe), apply_rope(k, pe), x[:, :, 2]


def _attend(q, k, v):
    """[B, S, H, D] x3 -> [B, S, H*D], non-causal."""
    o = attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal=False)
    B, H, S, D = o.shape
    return o.transpose(1, 2).reshape(B, S, H * D)


def _swiglu(x, w1, w2):
    gu = lin(x, w1)
    M = gu.shape[-1] // 2
    return lin(F.silu(gu[..., :M]) * gu[..., M:], w2)


# ---- fused GPU path (bf16 inference on the hand-written kernels) ---------------------------------------------------
# The same blocks with the element-wise glue folded into kernels: QK-norm + RoPE in one pass over the projection's output
# (text and image rows written straight into one packed [B, S, 3, H, D] buffer, so nothing is concatenated), attention on
# strided views of that buffer, SwiGLU in the epilogue of the gate/up product (weights re-ordered once per block), and the
# single-stream block's [attention | MLP] operand of linear2 assembled in place.  At batch 4 the unfused sequence spent
# 37 % of a denoising step in ATen element-wise and copy kernels.

def _fused_ok(cfg, x: torch.Tensor) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and not torch.is_grad_enabled() and cfg.head_dim == 128
            and cfg.mlp_hidden_dim % 128 == 0 and _flash.has_fwd() and flux_qk_post_supported(x, cfg.head_dim))


def _gate_up_interleaved(owner, name: str, w1: torch.Tensor) -> torch.Tensor:
    """``w1`` ([2*M, hidden], gate rows then up rows) in the gated epilogue's row order, cached on the block."""
    key = (w1.data_ptr(), tuple(w1.shape), w1._version)
    cached = getattr(owner, name, None)
    if cached is None or cached[0] != key:
        cached = (key, interleave_gate_up(w1))
        setattr(owner, name, cached)
    return cached[1]


def _swiglu_fused(owner, name, x, w1, w2):
    B, S, h = x.shape
    act = _gemm(x.reshape(B * S, h), _gate_up_interleaved(owner, name, w1), act="swiglu")
    return lin(act.reshape(B, S, -1), w2)


def _double_block_fused(cfg, b: DoubleStreamBlock, img, txt, img_pe, txt_pe, mod_img, mod_txt):
    B, Si, h = img.shape
    St = txt.shape[1]
    H, D = cfg.num_heads, cfg.head_dim
    qkv = torch.empty((B, St + Si, 3 * H * D), dtype=img.dtype, device=img.device)
    tproj = lin(layernorm_modulate(txt, mod_txt[:, 1], mod_txt[:, 0], EPS), b.txt_attn.qkv)
    flux_qk_post(tproj, qkv, b.txt_attn.norm.query_norm, b.txt_attn.norm.key_norm, txt_pe[0], txt_pe[1], H,
                 dst_row0=0, copy_v=True, eps=EPS)
    iproj = lin(layernorm_modulate(img, mod_img[:, 1], mod_img[:, 0], EPS), b.img_attn.qkv)
    flux_qk_post(iproj, qkv, b.img_attn.norm.query_norm, b.img_attn.norm.key_norm, img_pe[0], img_pe[1], H,
                 dst_row0=St, copy_v=True, eps=EPS)
    x5 = qkv.view(B, St + Si, 3, H, D)
    attn, _ = _flash.flash_fwd_bthd(x5[:, :, 0], x5[:, :, 1], x5[:, :, 2], causal=False, window=None, scale=None,
                                    need_lse=False)
    attn = attn.view(B, St + Si, H * D)
    img = gate_residual(img, lin(attn[:, St:].contiguous(), b.img_attn.proj), mod_img[:, 2])
    txt = gate_residual(txt, lin(attn[:, :St].contiguous(), b.txt_attn.proj), mod_txt[:, 2])
    img = gate_residual(img, _swiglu_fused(b, "_img_w1_il", layernorm_modulate(img, mod_img[:, 4], mod_img[:, 3], EPS),
                                           b.img_mlp.w1, b.img_mlp.w2), mod_img[:, 5])
    txt = gate_residual(txt, _swiglu_fused(b, "_txt_w1_il", layernorm_modulate(txt, mod_txt[:, 4], mod_txt[:, 3], EPS),
                                           b.txt_mlp.w1, b.txt_mlp.w2), mod_txt[:, 5])
    return img, txt


def _single_block_fused(cfg, b: SingleStreamBlock, x, pe, mod):
    B, S, h = x.shape
    H, D, M = cfg.num_heads, cfg.head_dim, cfg.mlp_hidden_dim
    xm = layernorm_modulate(x, mod[:, 1], mod[:, 0], EPS).reshape(B * S, h)
    qkv = _gemm(xm, b.linear1[:3 * H * D]).view(B, S, 3 * H * D)
    flux_qk_post(qkv, qkv, b.norm.query_norm, b.norm.key_norm, pe[0], pe[1], H, eps=EPS)      # in place; v untouched
    cat = torch.empty((B, S, H * D + M), dtype=x.dtype, device=x.device)                       # [attention | silu(gate) * up]
    _gemm(xm, _gate_up_interleaved(b, "_mlp_w1_il", b.linear1[3 * H * D:]), act="swiglu",
          out=cat.view(B * S, H * D + M)[:, H * D:])
    x5 = qkv.view(B, S, 3, H, D)
    _flash.flash_fwd_bthd(x5[:, :, 0], x5[:, :, 1], x5[:, :, 2], causal=False, window=None, scale=None, need_lse=False,
                          out=cat.view(B, S, -1)[:, :, :H * D].unflatten(-1, (H, D)))
    return gate_residual(x, lin(cat, b.linear2), mod[:, 2])


def double_block_forward(cfg, b: DoubleStreamBlock, img, txt, img_pe, txt_pe, mod_img, mod_txt):
    if _fused_ok(cfg, img):
        return _double_block_fused(cfg, b, img, txt, img_pe, txt_pe, mod_img, mod_txt)
    txt_seq = txt.shape[1]
    iq, ik, iv = _qk(cfg, lin(layernorm_modulate(img, mod_img[:, 1], mod_img[:, 0], EPS), b.img_attn.qkv), b.img_attn.norm, img_pe)
    tq, tk, tv = _qk(cfg, lin(layernorm_modulate(txt, mod_txt[:, 1], mod_txt[:, 0], EPS), b.txt_attn.qkv), b.txt_attn.norm, txt_pe)
    attn = _attend(torch.cat([tq, iq], 1), torch.cat([tk, ik], 1), torch.cat([tv, iv], 1))
    img = gate_residual(img, lin(attn[:, txt_seq:].contiguous(), b.img_attn.proj), mod_img[:, 2])
    txt = gate_residual(txt, lin(attn[:, :txt_seq].contiguous(), b.txt_attn.proj), mod_txt[:, 2])
    img = gate_residual(img, _swiglu(layernorm_modulate(img, mod_img[:, 4], mod_img[:, 3], EPS), b.img_mlp.w1, b.img_mlp.w2), mod_img[:, 5])
    txt = gate_residual(txt, _swiglu(layernorm_modulate(txt, mod_txt[:, 4], mod_txt[:, 3], EPS), b.txt_mlp.w1, b.txt_mlp.w2), mod_txt[:, 5])
    return img, txt


def single_block_forward(cfg, b: SingleStreamBlock, x, pe, mod):
    if _fused_ok(cfg, x):
        return _single_block_fused(cfg, b, x, pe, mod)
    H, D, M = cfg.num_heads, cfg.head_dim, cfg.mlp_hidden_dim
    y = lin(layernorm_modulate(x, mod[:, 1], mod[:, 0], EPS), b.linear1)
    q, k, v = _qk(cfg, y[..., :3 * H * D], b.norm, pe)
    attn = _attend(q, k, v)
    mlp = y[..., 3 * H * D:]
    out = lin(torch.cat([attn, F.silu(mlp[..., :M]) * mlp[..., M:]], dim=-1), b.linear2)
    return gate_residual(x, out, mod[:, 2])


def forward(m: FluxModel, img, txt, timesteps, img_ids, txt_ids) -> torch.Tensor:
    """img [B, Si, in_channels], txt [B, St, context], timesteps [B] -> predicted velocity [B, Si, in_channels]."""
    cfg = m.cfg
    h = cfg.hidden_size
    vec = lin(F.silu(lin(timestep_embedding(timesteps, cfg.time_dim).to(m.dtype), m.time_in_layer)), m.time_out_layer)
    mod_img = modulation(vec, m.double_stream_modulation_img, 6)
    mod_txt = modulation(vec, m.double_stream_modulation_txt, 6)
    mod_single = modulation(vec, m.single_stream_modulation, 3)
    img = lin(img, m.img_in)
    txt = lin(txt, m.txt_in)
    img_pe = rope_embed(img_ids, cfg.half_axes_dims, cfg.theta)
    txt_pe = rope_embed(txt_ids, cfg.half_axes_dims, cfg.theta)
    for b in m.double_blocks:
        img, txt = double_block_forward(cfg, b, img, txt, img_pe, txt_pe, mod_img, mod_txt)
    x = torch.cat([txt, img], dim=1)
    pe = (torch.cat([txt_pe[0], img_pe[0]], 1), torch.cat([txt_pe[1], img_pe[1]], 1))
    for b in m.single_blocks:
        x = single_block_forward(cfg, b, x, pe, mod_single)
    img_out = x[:, txt.shape[1]:].contiguous()
    mod2 = lin(F.silu(vec), m.final_modulation)
    shift, scale = mod2[:, :h], mod2[:, h:]
    return lin(layernorm_modulate(img_out, scale, shift, EPS), m.final_linear)


# ---- sampling (Sampling.lean) ------------------------------------------------------------------------------
def compute_empirical_mu(image_seq_len: int, num_steps: int) -> float:
    a1, b1, a2, b2 = 8.73809524e-05, 1.89833333, 0.00016927, 0.45666666
    if image_seq_len > 4300:
        return a2 * image_seq_len + b2
    m_200, m_10 = a2 * image_seq_len + b2, a1 * image_seq_len + b1
    a = (m_200 - m_10) / 190.0
    return a * num_steps + (m_200 - 200.0 * a)


def generalized_time_snr_shift(t: float, mu: float, sigma: float = 1.0) -> float:
    if t == 0.0:
        return 0.0
    return math.exp(mu) / (math.exp(mu) + (1.0 / t - 1.0) ** sigma)


def compute_timesteps(image_seq_len: int, num_steps: int) -> List[Tuple[float, float]]:
    mu = compute_empirical_mu(image_seq_len, num_steps)
    return [(generalized_time_snr_shift(1.0 - i / num_steps, mu), generalized_time_snr_shift(1.0 - (i + 1) / num_steps, mu))
            for i in range(num_steps)]


def euler_step(x, pred, t_curr: float, t_next: float):
    return x + pred * (t_next - t_curr)


@torch.no_grad()
def denoise(m: FluxModel, noise, txt, img_ids, txt_ids, num_steps: int = 4):
    x = noise
    for t_curr, t_next in compute_timesteps(noise.shape[1], num_steps):
        t = torch.full((noise.shape[0],), t_curr, dtype=torch.float32, device=noise.device)
        x = euler_step(x, forward(m, x, txt, t, img_ids, txt_ids), t_curr, t_next)
    return x


def sample(m: FluxModel, txt, img_ids, txt_ids, num_steps: int = 4, generator=None):
    noise = torch.randn((txt.shape[0], img_ids.shape[1], m.cfg.in_channels), generator=generator).to(device=m.device, dtype=m.dtype)
    return denoise(m, noise, txt, img_ids, txt_ids, num_steps)


def compute_image_position_ids(height: int, width: int, device="cpu") -> torch.Tensor:
    ids = torch.zeros(1, height * width, 4, dtype=torch.int64)
    idx = torch.arange(height * width)
    ids[0, :, 1], ids[0, :, 2] = idx // width, idx % width
    return ids.to(device)


def compute_text_position_ids(seq_len: int, device="cpu") -> torch.Tensor:
    ids = torch.zeros(1, seq_len, 4, dtype=torch.int64)
    ids[0, :, 3] = torch.arange(seq_len)
    return ids.to(device)


def unpack_latents(z: torch.Tensor, packed_h: int, packed_w: int) -> torch.Tensor:
    """[B, h*w, 128] -> [B, 32, 2h, 2w]: ``b (h w) (c p1 p2) -> b c (h p1) (w p2)``."""
    B = z.shape[0]
    return z.reshape(B, packed_h, packed_w, 32, 2, 2).permute(0, 3, 1, 4, 2, 5).reshape(B, 32, packed_h * 2, packed_w * 2)


def pack_latents(z: torch.Tensor) -> torch.Tensor:
    B, C, H2, W2 = z.shape
    return z.reshape(B, C, H2 // 2, 2, W2 // 2, 2).permute(0, 2, 4, 1, 3, 5).reshape(B, (H2 // 2) * (W2 // 2), C * 4)


# ---- weights ---------------------------------------------------------------------------------------------------
def load(cfg: FluxConfig, source, device="cpu", dtype=torch.bfloat16, log=None) -> FluxModel:
    src = source if isinstance(source, st.Source) else st.Source.open(source)
    info = log or (lambda s: None)
    h, D, H, M = cfg.hidden_size, cfg.head_dim, cfg.num_heads, cfg.mlp_hidden_dim

    def w(name, shape):
        t = src.load(name)
        if tuple(t.shape) != tuple(shape):
            raise st.SafeTensorsError(f"{name}: expected shape {list(shape)}, got {list(t.shape)}")
        return t.to(device=device, dtype=dtype)
    qkn = lambda p: QKNorm(w(f"{p}.query_norm.scale", (D,)), w(f"{p}.key_norm.scale", (D,)))
    sa = lambda p: SelfAttention(w(f"{p}.qkv.weight", (3 * H * D, h)), qkn(f"{p}.norm"), w(f"{p}.proj.weight", (h, H * D)))
    mlp = lambda p: SwiGLUMLP(w(f"{p}.0.weight", (2 * M, h)), w(f"{p}.2.weight", (h, M)))
    info("Loading Flux model...")
    doubles = [DoubleStreamBlock(sa(f"double_blocks.{i}.img_attn"), mlp(f"double_blocks.{i}.img_mlp"),
                                 sa(f"double_blocks.{i}.txt_attn"), mlp(f"double_blocks.{i}.txt_mlp")) for i in range(cfg.num_double_layers)]
    info(f"  Loaded {cfg.num_double_layers} double blocks")
    singles = [SingleStreamBlock(w(f"single_blocks.{i}.linear1.weight", (3 * H * D + 2 * M, h)),
                                 w(f"single_blocks.{i}.linear2.weight", (h, H * D + M)), qkn(f"single_blocks.{i}.norm"))
               for i in range(cfg.num_single_layers)]
    info(f"  Loaded {cfg.num_single_layers} single blocks")
    return FluxModel(cfg, w("img_in.weight", (h, cfg.in_channels)), w("txt_in.weight", (h, cfg.context_in_dim)),
                     w("time_in.in_layer.weight", (h, cfg.time_dim)), w("time_in.out_layer.weight", (h, h)), doubles, singles,
                     w("double_stream_modulation_img.lin.weight", (6 * h, h)), w("double_stream_modulation_txt.lin.weight", (6 * h, h)),
                     w("single_stream_modulation.lin.weight", (3 * h, h)), w("final_layer.linear.weight", (cfg.in_channels, h)),
                     w("final_layer.adaLN_modulation.1.weight", (2 * h, h)))


def state_dict(m: FluxModel) -> Dict[str, torch.Tensor]:
    out = {"img_in.weight": m.img_in, "txt_in.weight": m.txt_in, "time_in.in_layer.weight": m.time_in_layer,
           "time_in.out_layer.weight": m.time_out_layer, "double_stream_modulation_img.lin.weight": m.double_stream_modulation_img,
           "double_stream_modulation_txt.lin.weight": m.double_stream_modulation_txt,
           "single_stream_modulation.lin.weight": m.single_stream_modulation, "final_layer.linear.weight": m.final_linear,
           "final_layer.adaLN_modulation.1.weight": m.final_modulation}
    for i, b in enumerate(m.double_blocks):
        for s in ("img", "txt"):
            a, mlp = getattr(b, f"{s}_attn"), getattr(b, f"{s}_mlp")
            p = f"double_blocks.{i}.{s}"
            out[f"{p}_attn.qkv.weight"], out[f"{p}_attn.proj.weight"] = a.qkv, a.proj
            out[f"{p}_attn.norm.query_norm.scale"], out[f"{p}_attn.norm.key_norm.scale"] = a.norm.query_norm, a.norm.key_norm
            out[f"{p}_mlp.0.weight"], out[f"{p}_mlp.2.weight"] = mlp.w1, mlp.w2
    for i, b in enumerate(m.single_blocks):
        p = f"single_blocks.{i}"
        out[f"{p}.linear1.weight"], out[f"{p}.linear2.weight"] = b.linear1, b.linear2
        out[f"{p}.norm.query_norm.scale"], out[f"{p}.norm.key_norm.scale"] = b.norm.query_norm, b.norm.key_norm
    return out
