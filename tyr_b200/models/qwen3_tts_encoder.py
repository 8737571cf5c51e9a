"""Qwen3-TTS speech-tokenizer ENCODERS (waveform -> codec ids), the counterpart of the decoder in ``qwen3_tts.py``.

* 12 Hz family: a causal SEANet-style conv stack (strides 4, 5, 6, 8 with ELU residual blocks), a causal 8-layer transformer
  with rotary attention over a 250-frame window and layer scales, a stride-2 replicate-padded downsample, then split residual
  vector quantisation (1 semantic + up to 31 acoustic codebooks of 2048 x 256, stored as running sums and usage counts).
  24 kHz audio at 1920 samples per frame; streaming re-encodes a bounded left context and keeps the new rows
  (Tyr/Model/Qwen3TTS/SpeechTokenizerEncoder.lean:144-848).
* 25 Hz family: Whisper-style mel front end (128 bins) -> two convs -> 6 pre-norm transformer blocks with learned positions ->
  stride-2 conv -> nearest neighbour in one 32768 x 1280 codebook, in chunks of 200 mel frames
  (Tyr/Model/Qwen3TTS/SpeechTokenizer25HzEncoder.lean:36-390).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..audio import frontend as FE
from ..io import safetensors as st
from ..ops.attention import attention
from ..ops.rope import apply_rotary, rotary_freqs


def ceil_div(x: int, d: int) -> int:
    return 0 if d == 0 else (x + d - 1) // d


STRIDES_12HZ = (4, 5, 6, 8)


def frames_before_final_downsample(samples: int) -> int:
    for s in STRIDES_12HZ:
        samples = ceil_div(samples, s)
    return samples


def encoded_frames(samples: int) -> int:
    return ceil_div(frames_before_final_downsample(samples), 2)


def causal_conv(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], stride: int = 1, dilation: int = 1, replicate: bool = False) -> torch.Tensor:
    """Left-padded conv that emits exactly ceil(len / stride) frames; the right side gets just enough padding for the last
    window.  ``replicate`` pads with the edge samples instead of zeros."""
    n, k = x.shape[-1], w.shape[-1]
    eff = (k - 1) * dilation + 1
    left = eff - stride
    out = ceil_div(n, stride)
    extra = max(0, (out - 1) * stride + eff - (n + left))
    x = F.pad(x, (left, extra), mode="replicate" if replicate else "constant")
    return F.conv1d(x, w, b, stride=stride, dilation=dilation)


@dataclass
class Encoder12HzConfig:
    channels: Tuple[int, ...] = (64, 128, 256, 512, 1024)
    hidden: int = 512
    heads: int = 8
    layers: int = 8
    ffn: int = 2048
    window: int = 250
    codebook_size: int = 2048
    codebook_dim: int = 256
    semantic_codebooks: int = 1
    acoustic_codebooks: int = 15
    input_sample_rate: int = 24000
    encode_downsample_rate: int = 1920

    @staticmethod
    def from_json(j: dict) -> "Encoder12HzConfig":
        """``encoder_valid_num_quantizers`` counts the semantic group first (Config.encoderCodebookCounts)."""
        valid = int(j.get("encoder_valid_num_quantizers", 16))
        sem = int((j.get("encoder_config") or {}).get("num_semantic_quantizers", 1))
        if valid <= sem:
            raise ValueError(f"encoder_valid_num_quantizers={valid} leaves no acoustic codebook after {sem} semantic")
        return Encoder12HzConfig(semantic_codebooks=sem, acoustic_codebooks=valid - sem, input_sample_rate=int(j.get("input_sample_rate", 24000)),
                                 encode_downsample_rate=int(j.get("encode_downsample_rate", 1920)))


def encoder12hz_shapes(c: Encoder12HzConfig) -> Dict[str, tuple]:
    ch, s = c.channels, {}
    s["encoder.encoder.layers.0.conv.weight"], s["encoder.encoder.layers.0.conv.bias"] = (ch[0], 1, 7), (ch[0],)
    for i, (k, cin) in enumerate(zip((8, 10, 12, 16), ch[:4])):
        blk, down = 1 + 3 * i, 3 + 3 * i
        s[f"encoder.encoder.layers.{blk}.block.1.conv.weight"], s[f"encoder.encoder.layers.{blk}.block.1.conv.bias"] = (cin // 2, cin, 3), (cin // 2,)
        s[f"encoder.encoder.layers.{blk}.block.3.conv.weight"], s[f"encoder.encoder.layers.{blk}.block.3.conv.bias"] = (cin, cin // 2, 1), (cin,)
        s[f"encoder.encoder.layers.{down}.conv.weight"], s[f"encoder.encoder.layers.{down}.conv.bias"] = (ch[i + 1], cin, k), (ch[i + 1],)
    s["encoder.encoder.layers.14.conv.weight"], s["encoder.encoder.layers.14.conv.bias"] = (c.hidden, ch[4], 3), (c.hidden,)
    for i in range(c.layers):
        p = f"encoder.encoder_transformer.layers.{i}."
        for n in ("input_layernorm", "post_attention_layernorm"):
            s[p + n + ".weight"] = s[p + n + ".bias"] = (c.hidden,)
        for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
            s[p + f"self_attn.{n}.weight"] = (c.hidden, c.hidden)
        s[p + "self_attn_layer_scale.scale"] = s[p + "mlp_layer_scale.scale"] = (c.hidden,)
        s[p + "mlp.fc1.weight"], s[p + "mlp.fc2.weight"] = (c.ffn, c.hidden), (c.hidden, c.ffn)
    s["encoder.downsample.conv.weight"] = (c.hidden, c.hidden, 4)
    for kind, n in (("semantic", c.semantic_codebooks), ("acoustic", c.acoustic_codebooks)):
        p = f"encoder.quantizer.{kind}_residual_vector_quantizer."
        s[p + "input_proj.weight"] = (c.codebook_dim, c.hidden, 1)
        for i in range(n):
            s[p + f"layers.{i}.codebook.cluster_usage"] = (c.codebook_size,)
            s[p + f"layers.{i}.codebook.embed_sum"] = (c.codebook_size, c.codebook_dim)
    return s


def nearest_code(x: torch.Tensor, embed: torch.Tensor) -> torch.Tensor:
    """Index of the closest row of ``embed`` for every row of ``x`` (squared distance through one GEMM)."""
    dist = (x * x).sum(1, keepdim=True) + (embed * embed).sum(1)[None, :] - 2.0 * (x @ embed.t())
    return dist.argmin(1)


@dataclass
class SpeechTokenizer12HzEncoder:
    cfg: Encoder12HzConfig
    p: Dict[str, torch.Tensor]

    @property
    def num_code_groups(self) -> int:
        return self.cfg.semantic_codebooks + self.cfg.acoustic_codebooks

    def _res(self, x, blk):
        p = self.p
        h = causal_conv(F.elu(x), p[f"encoder.encoder.layers.{blk}.block.1.conv.weight"], p[f"encoder.encoder.layers.{blk}.block.1.conv.bias"])
        return x + causal_conv(F.elu(h), p[f"encoder.encoder.layers.{blk}.block.3.conv.weight"], p[f"encoder.encoder.layers.{blk}.block.3.conv.bias"])

    def _layer(self, x, i, cos, sin):
        c, p, L = self.cfg, self.p, f"encoder.encoder_transformer.layers.{i}."
        B, S, H = x.shape[0], x.shape[1], c.heads
        h = F.layer_norm(x, (c.hidden,), p[L + "input_layernorm.weight"], p[L + "input_layernorm.bias"], 1e-5)
        q, k, v = (F.linear(h, p[L + f"self_attn.{n}.weight"]).reshape(B, S, H, c.hidden // H) for n in ("q_proj", "k_proj", "v_proj"))
        q, k = apply_rotary(q, cos, sin), apply_rotary(k, cos, sin)
        a = attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal=True, window=c.window).transpose(1, 2).reshape(B, S, c.hidden)
        x = x + F.linear(a.to(x.dtype), p[L + "self_attn.o_proj.weight"]) * p[L + "self_attn_layer_scale.scale"]
        h = F.layer_norm(x, (c.hidden,), p[L + "post_attention_layernorm.weight"], p[L + "post_attention_layernorm.bias"], 1e-5)
        return x + F.linear(F.gelu(F.linear(h, p[L + "mlp.fc1.weight"])), p[L + "mlp.fc2.weight"]) * p[L + "mlp_layer_scale.scale"]

    def codebook(self, kind: str, i: int) -> torch.Tensor:
        p = f"encoder.quantizer.{kind}_residual_vector_quantizer.layers.{i}.codebook."
        usage = self.p[p + "cluster_usage"].float().clamp_min(1e-5)
        return (self.p[p + "embed_sum"].float() / usage[:, None]).to(self.p["encoder.downsample.conv.weight"].dtype)

    def _rvq(self, kind: str, n: int, x: torch.Tensor) -> torch.Tensor:
        """x: [B, hidden, frames] -> [n, B, frames] indices, each codebook quantising what the previous ones left."""
        B, _, T = x.shape
        res = F.conv1d(x, self.p[f"encoder.quantizer.{kind}_residual_vector_quantizer.input_proj.weight"]).transpose(1, 2).reshape(B * T, -1)
        out = []
        for i in range(n):
            e = self.codebook(kind, i)
            idx = nearest_code(res.float(), e.float())
            res = res - e[idx]
            out.append(idx.reshape(B, T))
        return torch.stack(out) if out else torch.zeros(0, B, T, dtype=torch.long, device=x.device)

    @torch.no_grad()
    def encode(self, audio: torch.Tensor, rope_start: int = 0) -> torch.Tensor:
        """audio: [B, 1, samples] -> codec ids [B, groups, encoded_frames(samples)].  ``rope_start`` is the position of the first
        frame on the pre-downsample transformer timeline (960 samples per step), used when a stream re-encodes a left context."""
        if audio.dim() != 3 or audio.shape[1] != 1 or audio.shape[2] == 0:
            raise ValueError("audio must be [batch, 1, samples] with at least one sample")
        c, p = self.cfg, self.p
        x = causal_conv(audio.to(p["encoder.encoder.layers.0.conv.weight"].dtype), p["encoder.encoder.layers.0.conv.weight"], p["encoder.encoder.layers.0.conv.bias"])
        for i, s in enumerate(STRIDES_12HZ):
            x = self._res(x, 1 + 3 * i)
            x = causal_conv(F.elu(x), p[f"encoder.encoder.layers.{3 + 3 * i}.conv.weight"], p[f"encoder.encoder.layers.{3 + 3 * i}.conv.bias"], stride=s)
        x = causal_conv(F.elu(x), p["encoder.encoder.layers.14.conv.weight"], p["encoder.encoder.layers.14.conv.bias"]).transpose(1, 2)
        t4 = x.shape[1]
        cos, sin = rotary_freqs(rope_start + t4, c.hidden // c.heads, 10000.0, x.device)
        cos, sin = cos[rope_start:], sin[rope_start:]
        for i in range(c.layers):
            x = self._layer(x, i, cos, sin)
        x = causal_conv(x.transpose(1, 2), p["encoder.downsample.conv.weight"], None, stride=2, replicate=True)
        codes = torch.cat([self._rvq("semantic", c.semantic_codebooks, x), self._rvq("acoustic", c.acoustic_codebooks, x)], 0)
        return codes.transpose(0, 1).contiguous()

    def encode_mono_frame_major(self, wave: torch.Tensor, rope_start: int = 0) -> torch.Tensor:
        """wave: [samples] -> [frames, groups]."""
        return self.encode(wave.reshape(1, 1, -1), rope_start)[0].t().contiguous()


@dataclass
class EncodeStreamState:
    chunk_samples: int = 240000
    left_context_samples: int = 288000
    offset_samples: int = 0
    history: List[float] = field(default_factory=list)


def push_encode_stream(m: SpeechTokenizer12HzEncoder, state: EncodeStreamState, new_samples: Sequence[float]) -> Tuple[EncodeStreamState, List[int]]:
    """Encodes history + new samples with the rotary offset of the history start and returns the flat ids (rows x groups) of the
    rows that belong to the new samples; keeps at most ``left_context_samples`` of audio for the next call."""
    new_samples = list(new_samples)
    if not new_samples:
        return state, []
    ctx_start = state.offset_samples - len(state.history)
    chunk = state.history + new_samples
    dev = m.p["encoder.downsample.conv.weight"].device
    codes = m.encode_mono_frame_major(torch.tensor(chunk, dtype=torch.float32, device=dev), frames_before_final_downsample(ctx_start))
    drop, keep = encoded_frames(len(state.history)), encoded_frames(len(new_samples))
    vals = codes[drop:drop + keep].reshape(-1).tolist()
    hist = chunk[max(0, len(chunk) - state.left_context_samples):]
    return EncodeStreamState(state.chunk_samples, state.left_context_samples, state.offset_samples + len(new_samples), hist), vals


def init_encoder_12hz(cfg: Encoder12HzConfig, device="cpu", dtype=torch.float32, seed=0) -> SpeechTokenizer12HzEncoder:
    g, p = torch.Generator().manual_seed(seed), {}
    for name, shape in encoder12hz_shapes(cfg).items():
        if name.endswith("cluster_usage"):
            t = torch.rand(shape, generator=g) + 0.5
        elif name.endswith("layernorm.weight"):
            t = torch.ones(shape)
        elif name.endswith(".bias"):
            t = torch.zeros(shape)
        elif name.endswith(".scale"):
            t = torch.full(shape, 0.1)
        elif name.endswith("embed_sum"):
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (math.prod(shape[1:]) ** -0.5)
        p[name] = t.to(device=device, dtype=torch.float32 if "codebook" in name else dtype)
    return SpeechTokenizer12HzEncoder(cfg, p)


def _load_named(src, shapes: Dict[str, tuple], device, dtype, keep_fp32=(), optional_zero=()) -> Dict[str, torch.Tensor]:
    p = {}
    for name, shape in shapes.items():
        if src.find(name) is None:
            if name in optional_zero:
                p[name] = torch.zeros(shape, device=device, dtype=dtype)
                continue
            raise st.SafeTensorsError(f"missing speech-tokenizer tensor {name}")
        t = src.load(name)
        if tuple(t.shape) != tuple(shape):
            raise st.SafeTensorsError(f"speech-tokenizer tensor {name} has shape {tuple(t.shape)}, expected {tuple(shape)}")
        p[name] = t.to(device=device, dtype=torch.float32 if any(k in name for k in keep_fp32) else dtype)
    return p


def load_encoder_12hz(speech_tokenizer_dir: str, device="cpu", dtype=torch.float32, flexible: bool = True) -> SpeechTokenizer12HzEncoder:
    """``flexible=False`` insists on the fixed 16-group layout (1 semantic + 15 acoustic) like the reference's ``loadFromDir``."""
    with open(os.path.join(speech_tokenizer_dir, "config.json"), encoding="utf-8") as f:
        cfg = Encoder12HzConfig.from_json(json.load(f))
    if not flexible and (cfg.semantic_codebooks, cfg.acoustic_codebooks) != (1, 15):
        raise ValueError("Fixed 16-group encoder requires encoder_valid_num_quantizers=16 and one semantic quantizer")
    src = st.Source.open(os.path.join(speech_tokenizer_dir, "model.safetensors"))
    return SpeechTokenizer12HzEncoder(cfg, _load_named(src, encoder12hz_shapes(cfg), device, dtype, keep_fp32=("codebook",)))


# ---- 25 Hz family -------------------------------------------------------------------------------------------------------------
@dataclass
class Encoder25HzConfig:
    n_mels: int = 128
    n_ctx: int = 1500
    n_state: int = 1280
    n_head: int = 20
    n_blocks: int = 6                 # only the blocks in front of the quantiser are run
    codebook_size: int = 32768
    input_sample_rate: int = 24000
    encode_downsample_rate: int = 1920
    chunk_mel_frames: int = 200

    @staticmethod
    def from_json(j: dict) -> "Encoder25HzConfig":
        if j.get("model_type") != "qwen3_tts_tokenizer_25hz":
            raise ValueError(f"model_type must be qwen3_tts_tokenizer_25hz, got {j.get('model_type')!r}")
        e = j.get("encoder_config")
        if e is not None:
            for k, want in (("n_mels", 128), ("n_ctx", 1500), ("n_state", 1280), ("n_head", 20), ("n_window", 100), ("audio_vq_layers", 6),
                            ("audio_vq_codebook_size", 32768), ("audio_vq_codebook_dim", 1280), ("audio_vq_ds_rate", 2)):
                if k in e and e[k] != want:
                    raise ValueError(f"encoder_config.{k} must be {want}, got {e[k]}")
            if e.get("audio_vq_type", "GRVQ") != "GRVQ":
                raise ValueError("encoder_config.audio_vq_type must be GRVQ")
            if int(e.get("n_layer", 32)) < 6:
                raise ValueError(f"Invalid n_layer={e.get('n_layer')}: the six quantized encoder blocks come first")
        rate, down = int(j.get("input_sample_rate", 24000)), int(j.get("encode_downsample_rate", 1920))
        if rate <= 0 or down <= 0:
            raise ValueError(f"Invalid input_sample_rate={rate}/encode_downsample_rate={down}: both must be positive")
        return Encoder25HzConfig(input_sample_rate=rate, encode_downsample_rate=down)


def encoder25hz_shapes(c: Encoder25HzConfig) -> Dict[str, tuple]:
    d, s = c.n_state, {}
    s["encoder.tokenizer.conv1.weight"], s["encoder.tokenizer.conv1.bias"] = (d, c.n_mels, 3), (d,)
    s["encoder.tokenizer.conv2.weight"], s["encoder.tokenizer.conv2.bias"] = (d, d, 3), (d,)
    s["encoder.tokenizer.positional_embedding"] = (c.n_ctx, d)
    for i in range(c.n_blocks):
        p = f"encoder.tokenizer.blocks.{i}."
        for n in ("attn_ln", "mlp_ln"):
            s[p + n + ".weight"] = s[p + n + ".bias"] = (d,)
        for n in ("query", "key", "value", "out"):
            s[p + f"attn.{n}.weight"], s[p + f"attn.{n}.bias"] = (d, d), (d,)
        s[p + "mlp.0.weight"], s[p + "mlp.0.bias"] = (4 * d, d), (4 * d,)
        s[p + "mlp.2.weight"], s[p + "mlp.2.bias"] = (d, 4 * d), (d,)
    s["encoder.tokenizer.audio_vq_downsample.weight"], s["encoder.tokenizer.audio_vq_downsample.bias"] = (d, d, 2), (d,)
    s["encoder.tokenizer.audio_quantizer.rvqs.0.embed"] = (1, c.codebook_size, d)
    return s


def mel_features(wave: torch.Tensor, n_mels: int, sample_rate: int) -> torch.Tensor:
    """Whisper-style log-mel [n_mels, frames] (Hann 400 / hop 160, last frame dropped, log10 clamped to max - 8, (x + 4) / 4) with
    the filter bank laid out for ``sample_rate``."""
    win = torch.hann_window(FE.N_FFT, periodic=True, device=wave.device)
    spec = torch.stft(wave.float(), FE.N_FFT, FE.HOP, window=win, center=True, pad_mode="reflect", return_complex=True)
    mel = FE.mel_filter_bank(n_mels, FE.N_FFT, sample_rate).to(wave.device) @ (spec[:, :-1].abs() ** 2)
    log = torch.log10(mel.clamp_min(1e-10))
    return (torch.maximum(log, log.max() - 8.0) + 4.0) / 4.0


@dataclass
class SpeechTokenizer25HzEncoder:
    cfg: Encoder25HzConfig
    p: Dict[str, torch.Tensor]

    def _block(self, x, i):
        c, p, L = self.cfg, self.p, f"encoder.tokenizer.blocks.{i}."
        S, H = x.shape[1], c.n_head
        h = F.layer_norm(x, (c.n_state,), p[L + "attn_ln.weight"], p[L + "attn_ln.bias"], 1e-5)
        q, k, v = (F.linear(h, p[L + f"attn.{n}.weight"], p[L + f"attn.{n}.bias"]).reshape(1, S, H, -1).transpose(1, 2) for n in ("query", "key", "value"))
        a = attention(q, k, v, causal=False).transpose(1, 2).reshape(1, S, c.n_state).to(x.dtype)
        x = x + F.linear(a, p[L + "attn.out.weight"], p[L + "attn.out.bias"])
        h = F.layer_norm(x, (c.n_state,), p[L + "mlp_ln.weight"], p[L + "mlp_ln.bias"], 1e-5)
        return x + F.linear(F.gelu(F.linear(h, p[L + "mlp.0.weight"], p[L + "mlp.0.bias"])), p[L + "mlp.2.weight"], p[L + "mlp.2.bias"])

    @torch.no_grad()
    def encode_mel_chunk(self, mel: torch.Tensor) -> torch.Tensor:
        """mel: [n_mels, frames] -> ids [((frames + 1) // 2) // 2]."""
        c, p = self.cfg, self.p
        frames = mel.shape[1]
        c2 = (frames + 1) // 2
        if c2 > c.n_ctx:
            raise ValueError(f"{frames} mel frames exceed the {c.n_ctx} learned positions")
        if frames < 2 or c2 // 2 == 0:
            return torch.zeros(0, dtype=torch.long, device=mel.device)
        x = F.gelu(F.conv1d(mel[None].to(p["encoder.tokenizer.conv1.weight"].dtype), p["encoder.tokenizer.conv1.weight"], p["encoder.tokenizer.conv1.bias"], padding=1))
        x = F.gelu(F.conv1d(x, p["encoder.tokenizer.conv2.weight"], p["encoder.tokenizer.conv2.bias"], stride=2, padding=1)).transpose(1, 2)
        x = x + p["encoder.tokenizer.positional_embedding"][:c2][None]
        for i in range(c.n_blocks):
            x = self._block(x, i)
        x = F.conv1d(x.transpose(1, 2), p["encoder.tokenizer.audio_vq_downsample.weight"], p["encoder.tokenizer.audio_vq_downsample.bias"], stride=2)
        return nearest_code(x[0].t().float(), p["encoder.tokenizer.audio_quantizer.rvqs.0.embed"][0].float())

    def encode_wave_to_codes(self, wave: torch.Tensor) -> Tuple[int, List[int]]:
        """(number of code groups = 1, flat ids) for a mono waveform at ``cfg.input_sample_rate``."""
        if wave.numel() == 0:
            raise ValueError("Audio encode input is empty")
        dev = self.p["encoder.tokenizer.conv1.weight"].device
        mel = mel_features(wave.reshape(-1).to(dev), self.cfg.n_mels, self.cfg.input_sample_rate)
        out: List[int] = []
        for s in range(0, mel.shape[1], self.cfg.chunk_mel_frames):
            chunk = mel[:, s:s + self.cfg.chunk_mel_frames]
            if chunk.shape[1] >= 2:
                out.extend(self.encode_mel_chunk(chunk).tolist())
        return 1, out


def init_encoder_25hz(cfg: Encoder25HzConfig, device="cpu", dtype=torch.float32, seed=0) -> SpeechTokenizer25HzEncoder:
    g, p = torch.Generator().manual_seed(seed), {}
    for name, shape in encoder25hz_shapes(cfg).items():
        if name.endswith("_ln.weight"):
            t = torch.ones(shape)
        elif name.endswith(".bias"):
            t = torch.zeros(shape)
        elif name.endswith("positional_embedding") or name.endswith(".embed"):
            t = torch.randn(shape, generator=g) * (0.02 if name.endswith("positional_embedding") else 1.0)
        else:
            t = torch.randn(shape, generator=g) * (math.prod(shape[1:]) ** -0.5)
        p[name] = t.to(device=device, dtype=dtype)
    return SpeechTokenizer25HzEncoder(cfg, p)


def load_encoder_25hz(speech_tokenizer_dir: str, device="cpu", dtype: Optional[torch.dtype] = None) -> SpeechTokenizer25HzEncoder:
    """The checkpoint's own floating dtype is kept unless ``dtype`` is given; a missing key bias loads as zeros."""
    with open(os.path.join(speech_tokenizer_dir, "config.json"), encoding="utf-8") as f:
        cfg = Encoder25HzConfig.from_json(json.load(f))
    src = st.Source.open(os.path.join(speech_tokenizer_dir, "model.safetensors"))
    anchor = src.load("encoder.tokenizer.conv1.weight")
    if not anchor.dtype.is_floating_point:
        raise st.SafeTensorsError("encoder.tokenizer.conv1.weight is not a floating tensor")
    shapes = encoder25hz_shapes(cfg)
    zero_ok = tuple(n for n in shapes if n.endswith("attn.key.bias"))
    return SpeechTokenizer25HzEncoder(cfg, _load_named(src, shapes, device, dtype or anchor.dtype, optional_zero=zero_ok))
