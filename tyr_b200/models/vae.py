"""Flux AutoEncoder decoder (BFL layout): latent BN de-normalisation, 2x2 unpack, conv/resnet/attention
decoder with nearest upsampling (Tyr/Model/VAE.lean, Tyr/Model/VAE/{Decoder,ResnetBlock,AttnBlock,Upsample,Weights}.lean)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

from ..io import safetensors as st
from ..ops.attention import attention

BN_EPS = 1e-4
GN_EPS = 1e-6


@dataclass
class Conv:
    weight: torch.Tensor
    bias: torch.Tensor
    padding: int = 1

    def __call__(self, x):
        return F.conv2d(x, self.weight, self.bias, padding=self.padding)


@dataclass
class GroupNorm:
    weight: torch.Tensor
    bias: torch.Tensor
    groups: int = 32

    def __call__(self, x):
        return F.group_norm(x, self.groups, self.weight, self.bias, GN_EPS)


@dataclass
class ResnetBlock:
    norm1: GroupNorm
    conv1: Conv
    norm2: GroupNorm
    conv2: Conv
    shortcut: Optional[Conv] = None

    def __call__(self, x):
        h = self.conv1(F.silu(self.norm1(x)))
        h = self.conv2(F.silu(self.norm2(h)))
        return (x if self.shortcut is None else self.shortcut(x)) + h


@dataclass
class AttnBlock:
    norm: GroupNorm
    q: Conv
    k: Conv
    v: Conv
    proj_out: Conv

    def __call__(self, x):
        B, C, H, W = x.shape
        h = self.norm(x)
        f = lambda c: c(h).reshape(B, 1, C, H * W).transpose(2, 3)          # [B, 1, HW, C] single head
        o = attention(f(self.q), f(self.k), f(self.v), causal=False)
        return x + self.proj_out(o.transpose(2, 3).reshape(B, C, H, W))


@dataclass
class Upsample:
    conv: Conv

    def __call__(self, x):
        return self.conv(F.interpolate(x, scale_factor=2.0, mode="nearest"))


@dataclass
class Decoder:
    post_quant_conv: Conv
    conv_in: Conv
    mid: List[object]
    ups: List[List[object]]     # lowest resolution first; each entry: 3 resnets (+ upsample)
    norm_out: GroupNorm
    conv_out: Conv

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        """[B, 32, H, W] -> [B, 3, 8H, 8W]."""
        h = self.conv_in(self.post_quant_conv(z))
        for blk in self.mid:
            h = blk(h)
        for stage in self.ups:
            for blk in stage:
                h = blk(h)
        return self.conv_out(F.silu(self.norm_out(h)))


STAGES = ((512, 512, True), (512, 512, True), (512, 256, True), (256, 128, False))


def _init_conv(cin, cout, k, gen, device, dtype):
    w = torch.randn((cout, cin, k, k), generator=gen) * (cin * k * k) ** -0.5
    return Conv(w.to(device=device, dtype=dtype), torch.zeros(cout, device=device, dtype=dtype), k // 2)


def _init_gn(c, device, dtype):
    return GroupNorm(torch.ones(c, device=device, dtype=dtype), torch.zeros(c, device=device, dtype=dtype))


def _init_res(cin, cout, gen, device, dtype):
    return ResnetBlock(_init_gn(cin, device, dtype), _init_conv(cin, cout, 3, gen, device, dtype), _init_gn(cout, device, dtype),
                       _init_conv(cout, cout, 3, gen, device, dtype), None if cin == cout else _init_conv(cin, cout, 1, gen, device, dtype))


def init_decoder(device="cpu", dtype=torch.float32, seed=0, stages=STAGES, z_channels=32) -> Decoder:
    gen = torch.Generator().manual_seed(seed)
    c0 = stages[0][0]
    mid = [_init_res(c0, c0, gen, device, dtype),
           AttnBlock(_init_gn(c0, device, dtype), *[_init_conv(c0, c0, 1, gen, device, dtype) for _ in range(4)]),
           _init_res(c0, c0, gen, device, dtype)]
    ups = []
    for cin, cout, up in stages:
        st_ = [_init_res(cin, cout, gen, device, dtype), _init_res(cout, cout, gen, device, dtype), _init_res(cout, cout, gen, device, dtype)]
        if up:
            st_.append(Upsample(_init_conv(cout, cout, 3, gen, device, dtype)))
        ups.append(st_)
    return Decoder(_init_conv(z_channels, z_channels, 1, gen, device, dtype), _init_conv(z_channels, c0, 3, gen, device, dtype), mid, ups,
                   _init_gn(stages[-1][1], device, dtype), _init_conv(stages[-1][1], 3, 3, gen, device, dtype))


@dataclass
class AutoEncoder:
    decoder: Decoder
    bn_running_mean: torch.Tensor    # [128]
    bn_running_var: torch.Tensor

    def inv_normalize(self, z: torch.Tensor) -> torch.Tensor:
        """Packed latents [B, 128, h, w]: ``z * sqrt(var + eps) + mean``."""
        scale = torch.sqrt(self.bn_running_var.float() + BN_EPS).reshape(1, -1, 1, 1)
        return (z.float() * scale + self.bn_running_mean.float().reshape(1, -1, 1, 1)).to(z.dtype)

    @staticmethod
    def unpack_packed(z: torch.Tensor) -> torch.Tensor:
        """[B, 128, h, w] -> [B, 32, 2h, 2w] (channel = c*4 + p1*2 + p2)."""
        B, C, H, W = z.shape
        return z.reshape(B, C // 4, 2, 2, H, W).permute(0, 1, 4, 2, 5, 3).reshape(B, C // 4, H * 2, W * 2)

    @torch.no_grad()
    def decode(self, z: torch.Tensor) -> torch.Tensor:
        return self.decoder.forward(self.unpack_packed(self.inv_normalize(z)))


def load_auto_encoder(path, device="cpu", dtype=torch.float32, log=None) -> AutoEncoder:
    src = path if isinstance(path, st.Source) else st.Source.open(path)
    g = lambda n: src.load(n).to(device=device, dtype=dtype)
    conv = lambda n, pad: Conv(g(f"{n}.weight"), g(f"{n}.bias"), pad)
    gn = lambda n: GroupNorm(g(f"{n}.weight"), g(f"{n}.bias"))

    def res(n):
        sc = conv(f"{n}.conv_shortcut", 0) if src.find(f"{n}.conv_shortcut.weight") is not None else None
        return ResnetBlock(gn(f"{n}.norm1"), conv(f"{n}.conv1", 1), gn(f"{n}.norm2"), conv(f"{n}.conv2", 1), sc)
    a = "decoder.mid_block.attentions.0"
    mid = [res("decoder.mid_block.resnets.0"),
           AttnBlock(gn(f"{a}.group_norm"), conv(f"{a}.to_q", 0), conv(f"{a}.to_k", 0), conv(f"{a}.to_v", 0), conv(f"{a}.to_out.0", 0)),
           res("decoder.mid_block.resnets.1")]
    ups = []
    for i, (_, _, up) in enumerate(STAGES):
        stage = [res(f"decoder.up_blocks.{i}.resnets.{j}") for j in range(3)]
        if up:
            stage.append(Upsample(conv(f"decoder.up_blocks.{i}.upsamplers.0.conv", 1)))
        ups.append(stage)
    dec = Decoder(conv("post_quant_conv", 0), conv("decoder.conv_in", 1), mid, ups, gn("decoder.conv_norm_out"), conv("decoder.conv_out", 1))
    return AutoEncoder(dec, src.load("bn.running_mean").to(device), src.load("bn.running_var").to(device))
