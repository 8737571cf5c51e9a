"""KittenTTS / Kokoro (StyleTTS2 family): ALBERT phoneme encoder, duration and prosody predictor (BiLSTM + adaptive
layer / instance norms driven by a style vector), decoder of AdaIN residual blocks and an ISTFTNet generator with a
harmonic-plus-noise source (Tyr/Model/KittenTTS/{Config,Model,Weights}.lean).

Parameters live in a flat dict under the checkpoint's names (weight-normalised convolutions keep ``weight_g`` / ``weight_v``
and are fused on load), so ``init`` and ``load`` produce the same structure.  One utterance per call (batch 1), as in the
reference.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


# ---- configuration -------------------------------------------------------------------------------------------------------------
@dataclass
class AlbertConfig:
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    hidden_size: int = 768
    intermediate_size: int = 3072
    max_position_embeddings: int = 512
    embedding_size: int = 128
    type_vocab_size: int = 2
    layer_norm_eps: float = 1e-12

    def __post_init__(self):
        if self.num_attention_heads <= 0 or self.hidden_size % self.num_attention_heads:
            raise ValueError("Invalid KittenTTS ALBERT config: hidden size must split evenly over the heads")


@dataclass
class GeneratorConfig:
    resblock_kernel_sizes: Tuple[int, ...] = (3, 7, 11)
    upsample_rates: Tuple[int, ...] = (10, 6)
    upsample_initial_channel: int = 512
    resblock_dilation_sizes: Tuple[Tuple[int, ...], ...] = ((1, 3, 5), (1, 3, 5), (1, 3, 5))
    upsample_kernel_sizes: Tuple[int, ...] = (20, 12)
    gen_istft_n_fft: int = 20
    gen_istft_hop_size: int = 5
    harmonic_count: int = 8

    def __post_init__(self):
        e = lambda m: ValueError(f"Invalid KittenTTS generator config: {m}")
        if not self.upsample_rates or len(self.upsample_kernel_sizes) != len(self.upsample_rates):
            raise e("one upsample kernel per rate")
        if any(r <= 1 or k < r or (k - r) % 2 for r, k in zip(self.upsample_rates, self.upsample_kernel_sizes)):
            raise e("every stage needs rate > 1 and a kernel that exceeds it by an even amount")
        if not self.resblock_kernel_sizes or any(k % 2 == 0 for k in self.resblock_kernel_sizes):
            raise e("residual blocks use odd kernels")
        if len(self.resblock_dilation_sizes) != len(self.resblock_kernel_sizes) or any(len(d) != 3 or min(d) <= 0 for d in self.resblock_dilation_sizes):
            raise e("three positive dilations per residual block")
        if 2 ** len(self.upsample_rates) > self.upsample_initial_channel:
            raise e("every stage halves the channels and keeps at least one")
        if self.gen_istft_hop_size <= 0 or self.gen_istft_n_fft <= 0 or self.gen_istft_n_fft % 2:
            raise e("the iSTFT needs a positive hop and a positive even FFT size")

    @property
    def total_upsample(self) -> int: return math.prod(self.upsample_rates)
    @property
    def source_upsample(self) -> int: return self.total_upsample * self.gen_istft_hop_size
    @property
    def freq_bins(self) -> int: return self.gen_istft_n_fft // 2 + 1

    def stage_out_channels(self, i: int) -> int: return self.upsample_initial_channel // 2 ** (i + 1)
    def suffix_upsample(self, start: int) -> int: return math.prod(self.upsample_rates[start:])


@dataclass
class KittenTTSConfig:
    hidden_dim: int = 512
    max_conv_dim: int = 512
    max_dur: int = 50
    n_layer: int = 3
    n_token: int = 178
    style_dim: int = 128
    text_encoder_kernel_size: int = 5
    asr_res_dim: int = 64
    sample_rate: int = 24000
    plbert: AlbertConfig = field(default_factory=AlbertConfig)
    generator: GeneratorConfig = field(default_factory=GeneratorConfig)

    def __post_init__(self):
        if self.hidden_dim % 2 or self.text_encoder_kernel_size % 2 == 0 or self.sample_rate <= 0 or self.max_dur <= 0:
            raise ValueError("Invalid KittenTTS config: even hidden dim, odd text kernel, positive sample rate and max duration")

    @property
    def full_style_dim(self) -> int: return 2 * self.style_dim
    @property
    def decoder_channels(self) -> int: return self.generator.upsample_initial_channel


# ---- primitives -----------------------------------------------------------------------------------------------------------------
def fuse_weight_norm(g: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """``w = g * v / ||v||`` with the norm over all dims but the first (both conv and transposed-conv checkpoints)."""
    n = v.flatten(1).norm(dim=1).reshape(-1, *([1] * (v.dim() - 1)))
    return v * (g / n)


def instance_norm(x, eps=1e-5):
    m = x.mean(2, keepdim=True)
    return (x - m) * torch.rsqrt(((x - m) ** 2).mean(2, keepdim=True) + eps)


def snake(x, alpha):
    return x + torch.sin(alpha * x).pow(2) / alpha


class P:
    """Read access to the parameter dict with a name prefix."""

    def __init__(self, d: Dict[str, torch.Tensor], prefix: str = ""):
        self.d, self.prefix = d, prefix

    def __call__(self, name: str) -> torch.Tensor: return self.d[self.prefix + name]
    def has(self, name: str) -> bool: return self.prefix + name in self.d
    def sub(self, name: str) -> "P": return P(self.d, self.prefix + name + ".")

    def conv(self, x, name, stride=1, padding=0, dilation=1, groups=1):
        return F.conv1d(x, self(name + ".weight"), self(name + ".bias") if self.has(name + ".bias") else None, stride, padding, dilation, groups)

    def linear(self, x, name):
        return F.linear(x, self(name + ".weight"), self(name + ".bias") if self.has(name + ".bias") else None)


def bilstm(p: P, x: torch.Tensor) -> torch.Tensor:
    """x: [1, T, in] -> [1, T, 2*hidden]; gates in the i, f, g, o order of the checkpoint's ``weight_ih_l0`` layout."""
    def run(suffix, seq):
        w_ih, w_hh, b = p("weight_ih_l0" + suffix), p("weight_hh_l0" + suffix), p("bias_ih_l0" + suffix) + p("bias_hh_l0" + suffix)
        Hd = w_hh.shape[1]
        h = c = torch.zeros(1, Hd, dtype=seq.dtype, device=seq.device)
        pre = F.linear(seq, w_ih, b)
        out = []
        for t in range(seq.shape[1]):
            i, f, g, o = (pre[:, t] + F.linear(h, w_hh)).chunk(4, -1)
            c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
            h = torch.sigmoid(o) * torch.tanh(c)
            out.append(h)
        return torch.stack(out, 1)
    return torch.cat([run("", x), run("_reverse", x.flip(1)).flip(1)], -1)


def ada_layer_norm(p: P, x, style):
    """x: [1, C, T]; LayerNorm over channels, then ``(1 + gamma) * x + beta`` from the style."""
    C = x.shape[1]
    gamma, beta = p.linear(style, "fc").split(C, dim=-1)
    n = F.layer_norm(x.transpose(1, 2), (C,), eps=1e-5)
    return ((1 + gamma[:, None]) * n + beta[:, None]).transpose(1, 2)


def adain(p: P, x, style):
    C = x.shape[1]
    gamma, beta = p.linear(style, "fc").split(C, dim=-1)
    n = instance_norm(x)
    if p.has("norm.weight"):
        n = n * p("norm.weight")[None, :, None] + p("norm.bias")[None, :, None]
    return (1 + gamma[:, :, None]) * n + beta[:, :, None]


def adain_resblk(p: P, x, style, upsample: bool = False):
    """StyleTTS2 ``AdainResBlk1d``: AdaIN -> LeakyReLU -> (depthwise transposed conv x2) -> conv, twice; nearest-upsampled
    1x1 shortcut; sum scaled by 1/sqrt(2)."""
    sc = F.interpolate(x, scale_factor=2, mode="nearest") if upsample else x
    if p.has("conv1x1.weight"):
        sc = p.conv(sc, "conv1x1")
    h = F.leaky_relu(adain(p.sub("norm1"), x, style), 0.2)
    if upsample:
        h = F.conv_transpose1d(h, p("pool.weight"), p("pool.bias"), stride=2, padding=1, output_padding=1, groups=h.shape[1])
    h = p.conv(h, "conv1", padding=1)
    h = p.conv(F.leaky_relu(adain(p.sub("norm2"), h, style), 0.2), "conv2", padding=1)
    return (h + sc) / math.sqrt(2.0)


# ---- ALBERT ---------------------------------------------------------------------------------------------------------------------------
def gelu_new(x):
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x.pow(3))))


def albert_forward(p: P, cfg: AlbertConfig, ids: torch.Tensor) -> torch.Tensor:
    """ids: [1, T] -> hidden states [1, T, hidden].  One transformer layer's weights are applied ``num_hidden_layers`` times."""
    T = ids.shape[1]
    e = p.sub("embeddings")
    x = F.embedding(ids, e("word_embeddings.weight")) + e("position_embeddings.weight")[:T][None] + e("token_type_embeddings.weight")[0][None, None]
    x = F.layer_norm(x, (cfg.embedding_size,), e("LayerNorm.weight"), e("LayerNorm.bias"), cfg.layer_norm_eps)
    x = p.linear(x, "encoder.embedding_hidden_mapping_in")
    l = p.sub("encoder.albert_layer_groups.0.albert_layers.0")
    H, D = cfg.num_attention_heads, cfg.hidden_size // cfg.num_attention_heads
    for _ in range(cfg.num_hidden_layers):
        q, k, v = (l.linear(x, f"attention.{n}").reshape(1, T, H, D).transpose(1, 2) for n in ("query", "key", "value"))
        a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(1, T, H * D)
        x = F.layer_norm(x + l.linear(a, "attention.dense"), (cfg.hidden_size,), l("attention.LayerNorm.weight"), l("attention.LayerNorm.bias"), cfg.layer_norm_eps)
        f = l.linear(gelu_new(l.linear(x, "ffn")), "ffn_output")
        x = F.layer_norm(x + f, (cfg.hidden_size,), l("full_layer_layer_norm.weight"), l("full_layer_layer_norm.bias"), cfg.layer_norm_eps)
    return x


# ---- model ----------------------------------------------------------------------------------------------------------------------------
def duration_to_frames(vals: Sequence[float], speed: float) -> List[int]:
    return [max(1, int(round(v / speed))) for v in vals]


def build_alignment(durations: Sequence[int], device) -> torch.Tensor:
    """[tokens, frames] 0/1 matrix: token i covers ``durations[i]`` consecutive frames."""
    idx = torch.repeat_interleave(torch.arange(len(durations), device=device), torch.tensor(list(durations), device=device))
    return F.one_hot(idx, len(durations)).T.float()


@dataclass
class KittenTTSOutput:
    audio: torch.Tensor
    pred_durations: List[int]
    alignment_frames: int


@dataclass
class KittenTTS:
    cfg: KittenTTSConfig
    params: Dict[str, torch.Tensor]

    @property
    def device(self): return self.params["bert.embeddings.word_embeddings.weight"].device

    # -- text side ------------------------------------------------------------------------------------------------------
    def text_encoder(self, ids: torch.Tensor) -> torch.Tensor:
        p, cfg = P(self.params, "text_encoder."), self.cfg
        x = F.embedding(ids, p("embedding.weight")).transpose(1, 2)
        for i in range(cfg.n_layer):
            x = p.conv(x, f"cnn.{i}.0", padding=cfg.text_encoder_kernel_size // 2)
            x = F.layer_norm(x.transpose(1, 2), (cfg.hidden_dim,), p(f"cnn.{i}.1.gamma"), p(f"cnn.{i}.1.beta"), 1e-5).transpose(1, 2)
            x = F.leaky_relu(x, 0.2)
        return bilstm(p.sub("lstm"), x.transpose(1, 2)).transpose(1, 2)

    def duration_encoding(self, d_en: torch.Tensor, style: torch.Tensor) -> torch.Tensor:
        """d_en: [1, hidden, T], style: [1, style] -> [1, hidden + style, T]: BiLSTM + AdaLayerNorm per layer, the style
        re-attached after each."""
        p, cfg = P(self.params, "predictor.text_encoder."), self.cfg
        s = style[:, :, None].expand(-1, -1, d_en.shape[2])
        h = torch.cat([d_en, s], 1)
        for i in range(cfg.n_layer):
            y = bilstm(p.sub(f"lstms.{2 * i}"), h.transpose(1, 2)).transpose(1, 2)
            h = torch.cat([ada_layer_norm(p.sub(f"lstms.{2 * i + 1}"), y, style), s], 1)
        return h

    @torch.no_grad()
    def predict_durations(self, ids: torch.Tensor, ref_style: torch.Tensor, speed: float = 1.0):
        """Returns (duration encoding [1, hidden+style, T], per-token frame counts)."""
        cfg, p = self.cfg, P(self.params)
        ids, ref_style = ids.to(self.device), ref_style.to(self.device)
        pred_style = ref_style[:, cfg.style_dim:]
        d_en = p.linear(albert_forward(p.sub("bert"), cfg.plbert, ids), "bert_encoder").transpose(1, 2)
        enc = self.duration_encoding(d_en, pred_style)
        h = bilstm(p.sub("predictor.lstm"), enc.transpose(1, 2))
        dur = torch.sigmoid(p.linear(h, "predictor.duration_proj.linear_layer")).sum(-1)[0]
        return enc, duration_to_frames(dur.tolist(), speed)

    def f0_n(self, enc_frames: torch.Tensor, style: torch.Tensor):
        """enc_frames: [1, hidden+style, F] -> pitch and energy curves [1, 1, 2F]."""
        p = P(self.params, "predictor.")
        shared = bilstm(p.sub("shared"), enc_frames.transpose(1, 2)).transpose(1, 2)
        out = []
        for name in ("F0", "N"):
            h = shared
            for i in range(3):
                h = adain_resblk(p.sub(f"{name}.{i}"), h, style, upsample=(i == 1))
            out.append(p.conv(h, f"{name}_proj"))
        return out[0], out[1]

    # -- generator ----------------------------------------------------------------------------------------------------------
    def harmonic_source(self, f0: torch.Tensor, generator: Optional[torch.Generator] = None) -> torch.Tensor:
        """f0: [1, samples, 1] (Hz, 0 when unvoiced) -> excitation [1, samples, 1]: harmonics 1..H+1 of f0 with phases
        accumulated at the frame rate, small noise, merged by a learned linear layer and tanh."""
        cfg, g = self.cfg, self.cfg.generator
        n, Hn = f0.shape[1], g.harmonic_count + 1
        mult = torch.arange(1, Hn + 1, device=f0.device, dtype=f0.dtype)
        rad = (f0 * mult / cfg.sample_rate) % 1.0
        ini = torch.rand(1, Hn, generator=generator).to(f0.device)
        ini[:, 0] = 0.0
        rad[:, 0] = rad[:, 0] + ini
        up = g.source_upsample
        down = F.interpolate(rad.transpose(1, 2), size=n // up, mode="linear", align_corners=False).transpose(1, 2)
        phase = torch.cumsum(down, 1) * 2 * math.pi
        phase = F.interpolate(phase.transpose(1, 2) * up, size=n, mode="linear", align_corners=False).transpose(1, 2)
        sine = torch.sin(phase) * 0.1
        uv = (f0 > 10.0).to(f0.dtype)
        noise_amp = uv * 0.003 + (1 - uv) * 0.1 / 3
        sine = sine * uv + noise_amp * torch.randn(sine.shape, generator=generator).to(f0.device)
        return torch.tanh(P(self.params, "decoder.generator.m_source.").linear(sine, "l_linear"))

    def generator(self, x: torch.Tensor, style: torch.Tensor, f0_curve: torch.Tensor, generator: Optional[torch.Generator] = None) -> torch.Tensor:
        """x: [1, C0, F] decoder features, f0_curve: [1, 1, F] -> waveform [samples]."""
        g, p = self.cfg.generator, P(self.params, "decoder.generator.")
        f0 = F.interpolate(f0_curve, scale_factor=g.source_upsample, mode="nearest").transpose(1, 2)
        har_wave = self.harmonic_source(f0, generator)[0, :, 0]
        window = torch.hann_window(g.gen_istft_n_fft, device=x.device)
        spec = torch.stft(har_wave, g.gen_istft_n_fft, g.gen_istft_hop_size, g.gen_istft_n_fft, window, center=True, return_complex=True)
        har = torch.cat([spec.abs(), spec.angle()], 0)[None]                                   # [1, 2*bins, F*total_up + 1]
        n_stage = len(g.upsample_rates)
        for i, (rate, k) in enumerate(zip(g.upsample_rates, g.upsample_kernel_sizes)):
            last = i + 1 == n_stage
            x = F.leaky_relu(x, 0.1)
            stride = 1 if last else g.suffix_upsample(i + 1)
            src = p.conv(har, f"noise_convs.{i}", stride=stride, padding=0 if last else (stride + 1) // 2)
            src = self._gen_resblock(p.sub(f"noise_res.{i}"), src, style, 11 if last else 7, (1, 3, 5))
            x = F.conv_transpose1d(x, p(f"ups.{i}.weight"), p(f"ups.{i}.bias"), stride=rate, padding=(k - rate) // 2)
            if last:
                x = torch.cat([x[:, :, 1:2] if x.shape[2] > 1 else x[:, :, :1], x], 2)           # reflect-pad one frame on the left
            x = x + src
            nk = len(g.resblock_kernel_sizes)
            x = sum(self._gen_resblock(p.sub(f"resblocks.{i * nk + j}"), x, style, g.resblock_kernel_sizes[j], g.resblock_dilation_sizes[j]) for j in range(nk)) / nk
        post = p.conv(F.leaky_relu(x, 0.01), "conv_post", padding=3)
        mag, phase = torch.exp(post[:, :g.freq_bins]), torch.sin(post[:, g.freq_bins:])
        wave = torch.istft(torch.polar(mag, phase)[0], g.gen_istft_n_fft, g.gen_istft_hop_size, g.gen_istft_n_fft, window, center=True)
        return wave

    @staticmethod
    def _gen_resblock(p: P, x, style, kernel: int, dilations: Sequence[int]):
        for m, d in enumerate(dilations):
            h = snake(adain(p.sub(f"adain1.{m}"), x, style), p(f"alpha1.{m}"))
            h = p.conv(h, f"convs1.{m}", padding=(kernel * d - d) // 2, dilation=d)
            h = snake(adain(p.sub(f"adain2.{m}"), h, style), p(f"alpha2.{m}"))
            x = x + p.conv(h, f"convs2.{m}", padding=(kernel - 1) // 2)
        return x

    def decoder(self, asr: torch.Tensor, f0_curve: torch.Tensor, n_curve: torch.Tensor, style: torch.Tensor, generator=None) -> torch.Tensor:
        """asr: [1, hidden, F]; pitch / energy curves [1, 1, 2F] -> waveform."""
        p = P(self.params, "decoder.")
        f0 = p.conv(f0_curve, "F0_conv", stride=2, padding=1)
        n = p.conv(n_curve, "N_conv", stride=2, padding=1)
        x = adain_resblk(p.sub("encode"), torch.cat([asr, f0, n], 1), style)
        res = p.conv(asr, "asr_res.0")
        for i in range(4):
            x = adain_resblk(p.sub(f"decode.{i}"), torch.cat([x, res, f0, n], 1), style, upsample=(i == 3))
        return self.generator(x, style, f0_curve, generator)

    # -- synthesis -------------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def synthesize(self, ids: torch.Tensor, ref_style: torch.Tensor, speed: float = 1.0, generator: Optional[torch.Generator] = None) -> KittenTTSOutput:
        """ids: [1, T] phoneme ids; ref_style: [1, 2*style] (decoder half first, predictor half second)."""
        cfg = self.cfg
        if ids.shape[1] == 0:
            return KittenTTSOutput(torch.zeros(0), [], 0)
        ids, ref_style = ids.to(self.device), ref_style.to(self.device)
        enc, durs = self.predict_durations(ids, ref_style, speed)
        aln = build_alignment(durs, self.device)
        pred_style, dec_style = ref_style[:, cfg.style_dim:], ref_style[:, :cfg.style_dim]
        f0, n = self.f0_n(enc @ aln[None], pred_style)
        asr = self.text_encoder(ids) @ aln[None]
        audio = self.decoder(asr, f0, n, dec_style, generator)
        return KittenTTSOutput(audio, durs, sum(durs))


# ---- parameters -------------------------------------------------------------------------------------------------------------------
def _shapes(cfg: KittenTTSConfig) -> Dict[str, Tuple[int, ...]]:
    s: Dict[str, Tuple[int, ...]] = {}
    a, g, H, S = cfg.plbert, cfg.generator, cfg.hidden_dim, cfg.style_dim

    def lin(name, o, i, bias=True):
        s[name + ".weight"] = (o, i)
        if bias:
            s[name + ".bias"] = (o,)

    def conv(name, o, i, k, bias=True):
        s[name + ".weight"] = (o, i, k)
        if bias:
            s[name + ".bias"] = (o,)

    def lstm(name, i, h):
        for sfx in ("", "_reverse"):
            s[f"{name}.weight_ih_l0{sfx}"], s[f"{name}.weight_hh_l0{sfx}"] = (4 * h, i), (4 * h, h)
            s[f"{name}.bias_ih_l0{sfx}"], s[f"{name}.bias_hh_l0{sfx}"] = (4 * h,), (4 * h,)

    def adain_(name, c):
        lin(name + ".fc", 2 * c, S)

    def resblk(name, i, o, up=False):
        conv(name + ".conv1", o, i, 3)
        conv(name + ".conv2", o, o, 3)
        adain_(name + ".norm1", i)
        adain_(name + ".norm2", o)
        if i != o:
            conv(name + ".conv1x1", o, i, 1, bias=False)
        if up:
            s[name + ".pool.weight"], s[name + ".pool.bias"] = (i, 1, 3), (i,)

    def gen_res(name, c, k):
        for m in range(3):
            conv(f"{name}.convs1.{m}", c, c, k)
            conv(f"{name}.convs2.{m}", c, c, k)
            adain_(f"{name}.adain1.{m}", c)
            adain_(f"{name}.adain2.{m}", c)
            s[f"{name}.alpha1.{m}"] = s[f"{name}.alpha2.{m}"] = (1, c, 1)

    e = "bert.embeddings."
    s[e + "word_embeddings.weight"], s[e + "position_embeddings.weight"] = (cfg.n_token, a.embedding_size), (a.max_position_embeddings, a.embedding_size)
    s[e + "token_type_embeddings.weight"], s[e + "LayerNorm.weight"], s[e + "LayerNorm.bias"] = (a.type_vocab_size, a.embedding_size), (a.embedding_size,), (a.embedding_size,)
    lin("bert.encoder.embedding_hidden_mapping_in", a.hidden_size, a.embedding_size)
    L = "bert.encoder.albert_layer_groups.0.albert_layers.0."
    for n in ("query", "key", "value", "dense"):
        lin(L + "attention." + n, a.hidden_size, a.hidden_size)
    lin(L + "ffn", a.intermediate_size, a.hidden_size)
    lin(L + "ffn_output", a.hidden_size, a.intermediate_size)
    for n in ("attention.LayerNorm", "full_layer_layer_norm"):
        s[L + n + ".weight"], s[L + n + ".bias"] = (a.hidden_size,), (a.hidden_size,)
    lin("bert_encoder", H, a.hidden_size)
    s["text_encoder.embedding.weight"] = (cfg.n_token, H)
    for i in range(cfg.n_layer):
        conv(f"text_encoder.cnn.{i}.0", H, H, cfg.text_encoder_kernel_size)
        s[f"text_encoder.cnn.{i}.1.gamma"], s[f"text_encoder.cnn.{i}.1.beta"] = (H,), (H,)
    lstm("text_encoder.lstm", H, H // 2)
    for i in range(cfg.n_layer):
        lstm(f"predictor.text_encoder.lstms.{2 * i}", H + S, H // 2)
        lin(f"predictor.text_encoder.lstms.{2 * i + 1}.fc", 2 * H, S)
    lstm("predictor.lstm", H + S, H // 2)
    lin("predictor.duration_proj.linear_layer", cfg.max_dur, H)
    lstm("predictor.shared", H + S, H // 2)
    for n in ("F0", "N"):
        resblk(f"predictor.{n}.0", H, H)
        resblk(f"predictor.{n}.1", H, H // 2, up=True)
        resblk(f"predictor.{n}.2", H // 2, H // 2)
        conv(f"predictor.{n}_proj", 1, H // 2, 1)
    conv("decoder.F0_conv", 1, 1, 3)
    conv("decoder.N_conv", 1, 1, 3)
    resblk("decoder.encode", H + 2, cfg.max_conv_dim)
    conv("decoder.asr_res.0", cfg.asr_res_dim, H, 1)
    cat = cfg.max_conv_dim + cfg.asr_res_dim + 2
    for i in range(3):
        resblk(f"decoder.decode.{i}", cat, cfg.max_conv_dim)
    resblk("decoder.decode.3", cat, cfg.decoder_channels, up=True)
    G = "decoder.generator."
    lin(G + "m_source.l_linear", 1, g.harmonic_count + 1)
    cin = g.upsample_initial_channel
    nk = len(g.resblock_kernel_sizes)
    for i, (r, k) in enumerate(zip(g.upsample_rates, g.upsample_kernel_sizes)):
        cout = g.stage_out_channels(i)
        s[f"{G}ups.{i}.weight"], s[f"{G}ups.{i}.bias"] = (cin, cout, k), (cout,)
        last = i + 1 == len(g.upsample_rates)
        conv(f"{G}noise_convs.{i}", cout, 2 * g.freq_bins, 1 if last else 2 * g.suffix_upsample(i + 1))
        gen_res(f"{G}noise_res.{i}", cout, 11 if last else 7)
        for j, kk in enumerate(g.resblock_kernel_sizes):
            gen_res(f"{G}resblocks.{i * nk + j}", cout, kk)
        cin = cout
    conv(G + "conv_post", g.gen_istft_n_fft + 2, cin, 7)
    return s


def init(cfg: KittenTTSConfig, device="cpu", seed: int = 0) -> KittenTTS:
    g = torch.Generator().manual_seed(seed)
    params = {}
    for name, shape in _shapes(cfg).items():
        if name.endswith((".bias", ".beta")) or "bias_" in name:
            t = torch.zeros(shape)
        elif name.endswith((".gamma", "LayerNorm.weight", "layer_norm.weight")) or ".alpha" in name:
            t = torch.ones(shape)
        else:
            fan = math.prod(shape[1:]) if len(shape) > 1 else shape[0]
            t = torch.randn(shape, generator=g) * fan ** -0.5
        params[name] = t.to(device)
    return KittenTTS(cfg, params)


def load(cfg: KittenTTSConfig, source, device="cpu") -> KittenTTS:
    """Reads a safetensors checkpoint with the names above; ``*.weight_g`` / ``*.weight_v`` pairs are fused into ``*.weight``.
    Every expected tensor must be present with the expected shape."""
    from ..io import safetensors as st
    src = source if isinstance(source, st.Source) else st.Source.open(source)
    have = set(src.names())
    params = {}
    for name, shape in _shapes(cfg).items():
        if name in have:
            t = src.load(name).float()
        elif name.endswith(".weight") and name[:-7] + ".weight_g" in have:
            t = fuse_weight_norm(src.load(name[:-7] + ".weight_g").float(), src.load(name[:-7] + ".weight_v").float())
        else:
            raise st.SafeTensorsError(f"KittenTTS checkpoint is missing {name}")
        if tuple(t.shape) != tuple(shape):
            raise st.SafeTensorsError(f"KittenTTS checkpoint: {name} has shape {tuple(t.shape)}, expected {tuple(shape)}")
        params[name] = t.to(device)
    return KittenTTS(cfg, params)


def load_voices(path: str) -> Dict[str, torch.Tensor]:
    """Voice-style table: one ``[n, 2*style]`` (or ``[2*style]``) tensor per voice name."""
    from ..io import safetensors as st
    src = st.Source.open(path)
    return {n: src.load(n).float() for n in src.names()}


def select_style(voice: torch.Tensor, num_tokens: int) -> torch.Tensor:
    """Kokoro voices store one style per utterance length; Kitten voices a single vector."""
    if voice.dim() == 1:
        return voice[None]
    v = voice.reshape(voice.shape[0], -1)
    return v[min(num_tokens, v.shape[0] - 1)][None]
