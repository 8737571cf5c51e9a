"""Qwen3-TTS: a talker (Qwen3 decoder over codec + projected text embeddings) that emits codebook 0 of each 12 Hz frame, a
code predictor that completes the residual codebooks of the frame, an ECAPA-TDNN speaker encoder for voice cloning, and the
12 Hz speech-tokenizer decoder (split RVQ -> causal transformer -> ConvNeXt upsampling -> SnakeBeta transposed-conv stack)
with chunked and streaming decoding.

Contract: Tyr/Model/Qwen3TTS/{Config,Talker,SpeakerEncoder,SpeechTokenizer,Streaming,Model}.lean.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..ops.attention import attention
from . import qwen as Q
from .common import KVCache, apply_rotary_partial, norm_w
from .generation import top_k_filter, top_p_filter


# ---- configuration -----------------------------------------------------------------------------------------------------------
@dataclass
class SpeakerEncoderConfig:
    mel_dim: int = 128
    enc_dim: int = 1024
    enc_channels: Tuple[int, ...] = (512, 512, 512, 512, 1536)
    enc_kernel_sizes: Tuple[int, ...] = (5, 3, 3, 3, 1)
    enc_dilations: Tuple[int, ...] = (1, 2, 3, 4, 1)
    enc_attention_channels: int = 128
    enc_res2net_scale: int = 8
    enc_se_channels: int = 128
    sample_rate: int = 24000

    def __post_init__(self):
        e = lambda m: ValueError(f"Invalid Qwen3-TTS speaker encoder config: {m}")
        c, k, d = self.enc_channels, self.enc_kernel_sizes, self.enc_dilations
        if not (len(c) == len(k) == len(d) == 5):
            raise e("five TDNN blocks are described by channels, kernel sizes and dilations")
        if any(kk <= 0 or dd <= 0 or (dd * (kk - 1)) % 2 for kk, dd in zip(k, d)):
            raise e("every convolution must admit 'same' padding")
        if not (c[0] == c[1] == c[2] == c[3]) or c[4] != c[1] + c[2] + c[3]:
            raise e("residual blocks keep their channels and the aggregation layer takes their concatenation")
        if self.enc_res2net_scale < 2 or c[0] % self.enc_res2net_scale:
            raise e("Res2Net splits the channels into >= 2 equal parts")


@dataclass
class CodePredictorConfig:
    vocab_size: int = 2048
    hidden_size: int = 1024
    intermediate_size: int = 3072
    num_hidden_layers: int = 5
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    half_head_dim: int = 64
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0

    def qwen(self) -> Q.QwenConfig:
        return Q.QwenConfig(vocab_size=self.vocab_size, hidden_size=self.hidden_size, intermediate_size=self.intermediate_size,
                            num_hidden_layers=self.num_hidden_layers, num_attention_heads=self.num_attention_heads,
                            num_key_value_heads=self.num_key_value_heads, half_head_dim=self.half_head_dim, rope_theta=self.rope_theta, rms_norm_eps=self.rms_norm_eps)


@dataclass
class TalkerConfig:
    code_predictor: CodePredictorConfig = field(default_factory=CodePredictorConfig)
    vocab_size: int = 3072
    hidden_size: int = 1024
    intermediate_size: int = 2048
    num_hidden_layers: int = 20
    num_attention_heads: int = 16
    num_key_value_heads: int = 2
    half_head_dim: int = 32
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    num_code_groups: int = 32
    text_hidden_size: int = 2048
    text_vocab_size: int = 151936
    codec_eos_token_id: int = 2150
    codec_think_id: int = 2154
    codec_nothink_id: int = 2155
    codec_think_bos_id: int = 2156
    codec_think_eos_id: int = 2157
    codec_pad_id: int = 2148
    codec_bos_id: int = 2149
    spk_id: Dict[str, int] = field(default_factory=dict)
    spk_is_dialect: Dict[str, str] = field(default_factory=dict)
    codec_language_id: Dict[str, int] = field(default_factory=dict)

    def __post_init__(self):
        if self.num_code_groups <= 1:
            raise ValueError("Invalid Qwen3-TTS talker config: a frame has codebook 0 plus at least one residual codebook")
        ids = [self.codec_eos_token_id, self.codec_think_id, self.codec_nothink_id, self.codec_think_bos_id, self.codec_think_eos_id, self.codec_pad_id,
               self.codec_bos_id, *self.spk_id.values(), *self.codec_language_id.values()]
        if any(i >= self.vocab_size for i in ids):
            raise ValueError("Invalid Qwen3-TTS talker config: codec special, speaker and language ids must index the codec embedding")

    def qwen(self) -> Q.QwenConfig:
        return Q.QwenConfig(vocab_size=self.vocab_size, hidden_size=self.hidden_size, intermediate_size=self.intermediate_size,
                            num_hidden_layers=self.num_hidden_layers, num_attention_heads=self.num_attention_heads,
                            num_key_value_heads=self.num_key_value_heads, half_head_dim=self.half_head_dim, rope_theta=self.rope_theta, rms_norm_eps=self.rms_norm_eps)


@dataclass
class Qwen3TTSConfig:
    talker: TalkerConfig = field(default_factory=TalkerConfig)
    speaker_encoder: SpeakerEncoderConfig = field(default_factory=SpeakerEncoderConfig)
    tts_model_type: str = "base"            # base / custom_voice / voice_design
    im_start_token_id: int = 151644
    im_end_token_id: int = 151645
    tts_pad_token_id: int = 151671
    tts_bos_token_id: int = 151672
    tts_eos_token_id: int = 151673

    def __post_init__(self):
        t = self.talker
        if any(i >= t.text_vocab_size for i in (self.im_start_token_id, self.im_end_token_id, self.tts_pad_token_id, self.tts_bos_token_id, self.tts_eos_token_id)):
            raise ValueError("Invalid Qwen3-TTS config: prompt text ids must index the talker text embedding")
        if self.tts_model_type == "base" and self.speaker_encoder.enc_dim != t.hidden_size:
            raise ValueError("Invalid Qwen3-TTS config: base models condition on a speaker embedding of the talker's hidden size")

    def supported_languages(self) -> List[str]:
        return ["auto"] + [k for k in self.talker.codec_language_id if "dialect" not in k]

    def supported_speakers(self) -> List[str]:
        return list(self.talker.spk_id)


# ---- talker ---------------------------------------------------------------------------------------------------------------------
@dataclass
class CodePredictor:
    input_embeddings: List[torch.Tensor]        # numCodeGroups-1 tables [cp_vocab, talker_hidden]
    input_projection: torch.Tensor              # [cp_hidden, talker_hidden]
    input_projection_bias: torch.Tensor
    model: Q.Qwen3Model                         # layers + norm (its embedding table is unused)
    lm_heads: List[torch.Tensor]                # numCodeGroups-1 heads [cp_vocab, cp_hidden]


@dataclass
class Talker:
    cfg: TalkerConfig
    codec_embedding: torch.Tensor
    text_embedding: torch.Tensor
    text_fc1: torch.Tensor; text_fc1_b: torch.Tensor; text_fc2: torch.Tensor; text_fc2_b: torch.Tensor
    model: Q.Qwen3Model
    code_predictor: CodePredictor
    codec_head: torch.Tensor

    @property
    def device(self): return self.codec_embedding.device

    def embed_codec(self, ids): return F.embedding(ids.to(self.device), self.codec_embedding)

    def embed_text(self, ids):
        t = F.embedding(ids.to(self.device), self.text_embedding)
        return F.linear(F.silu(F.linear(t, self.text_fc1, self.text_fc1_b)), self.text_fc2, self.text_fc2_b)

    def build_inputs_from_text(self, text_ids, instruct_ids=None):
        """``codec_bos`` embedding followed by the projected (instruct +) text embeddings."""
        emb = self.embed_text(text_ids) if instruct_ids is None else torch.cat([self.embed_text(instruct_ids), self.embed_text(text_ids)], 1)
        bos = self.embed_codec(torch.full((emb.shape[0], 1), self.cfg.codec_bos_id, dtype=torch.int64))
        return torch.cat([bos, emb], 1)


def init_talker(cfg: TalkerConfig, device="cpu", dtype=torch.float32, seed=0) -> Talker:
    g = torch.Generator().manual_seed(seed)
    w = lambda *s: (torch.randn(*s, generator=g) * s[-1] ** -0.5).to(device=device, dtype=dtype)
    cp = cfg.code_predictor
    n = cfg.num_code_groups - 1
    predictor = CodePredictor([w(cp.vocab_size, cfg.hidden_size) for _ in range(n)], w(cp.hidden_size, cfg.hidden_size), w(cp.hidden_size) * 0,
                              Q.init_model(cp.qwen(), device, dtype, seed + 1), [w(cp.vocab_size, cp.hidden_size) for _ in range(n)])
    return Talker(cfg, w(cfg.vocab_size, cfg.hidden_size), w(cfg.text_vocab_size, cfg.text_hidden_size), w(cfg.text_hidden_size, cfg.text_hidden_size),
                  w(cfg.text_hidden_size) * 0, w(cfg.hidden_size, cfg.text_hidden_size), w(cfg.hidden_size) * 0, Q.init_model(cfg.qwen(), device, dtype, seed + 2),
                  predictor, w(cfg.vocab_size, cfg.hidden_size))


class _Stack:
    """Cached run of a Qwen3 layer stack over embeddings (no embedding table, final norm applied)."""

    def __init__(self, model: Q.Qwen3Model, cfg: Q.QwenConfig, batch: int, max_len: int):
        self.model, self.cfg, self.pos = model, cfg, 0
        dev, dt = model.norm.device, model.norm.dtype
        self.rope = Q.RoPECache.init(max_len, cfg.half_head_dim, cfg.rope_theta, dev)
        self.caches = [KVCache.allocate(batch, cfg.num_key_value_heads, max_len, cfg.head_dim, dev, dt) for _ in model.layers]

    def run(self, x: torch.Tensor) -> torch.Tensor:
        cos, sin = self.rope.rows(self.pos, x.shape[1])
        for l, c in zip(self.model.layers, self.caches):
            x = Q.layer_forward(self.cfg, l, x, cos, sin, c)
        self.pos += x.shape[1]
        return norm_w(x, self.model.norm, self.cfg.rms_norm_eps)


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


@dataclass
class SamplingOptions:
    temperature: float = 0.9
    top_k: Optional[int] = None
    top_p: float = 1.0
    repetition_penalty: float = 1.05
    suppress_tail: int = 1024
    subtalker_temperature: float = 0.9
    subtalker_top_k: Optional[int] = None
    subtalker_top_p: float = 1.0
    subtalker_temperatures_by_group: Optional[Sequence[float]] = None
    subtalker_top_ks_by_group: Optional[Sequence[Optional[int]]] = None
    subtalker_top_ps_by_group: Optional[Sequence[float]] = None


def apply_sampling(logits: torch.Tensor, temperature: float, top_k: Optional[int], top_p: float, generator=None) -> torch.Tensor:
    if temperature <= 0.0:
        raise ValueError(f"sampling requires temperature > 0, got {temperature}")
    x = logits.float() if temperature == 1.0 else logits.float() / temperature
    x = top_k_filter(x, top_k)
    if top_p < 1.0:
        x = top_p_filter(x, top_p)
    return torch.multinomial(torch.softmax(x, -1), 1, generator=generator).reshape(-1)


def suppress_tail(logits: torch.Tensor, n: int, eos: int) -> torch.Tensor:
    """The last ``n`` codec ids are control tokens that must not be sampled as audio, except end-of-sequence."""
    V = logits.shape[-1]
    idx = torch.arange(V, device=logits.device)
    mask = (idx >= max(0, V - n)) & (idx != eos)
    return logits.masked_fill(mask[None], -1e9)


def repetition_penalty(logits: torch.Tensor, history: Optional[torch.Tensor], penalty: float) -> torch.Tensor:
    if history is None or history.shape[1] == 0 or penalty == 1.0 or penalty <= 0.0:
        return logits
    g = torch.gather(logits, 1, history)
    return logits.scatter(1, history, torch.where(g < 0, g * penalty, g / penalty))


@torch.no_grad()
def generate_frame_from_last_hidden(t: Talker, last_hidden: torch.Tensor, history: Optional[torch.Tensor] = None, allow_eos: bool = True,
                                    opt: SamplingOptions = SamplingOptions(), generator=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """last_hidden: [B, 1, hidden].  Returns (codes [B, numCodeGroups], summed embedding [B, 1, hidden] of all codes, the
    next talker input).  Codebook 0 comes from the talker head; the code predictor then reads
    ``[last_hidden, emb(code0), emb(code1), ...]`` with a K/V cache and emits one residual codebook per step."""
    cfg = t.cfg
    B = last_hidden.shape[0]
    first = suppress_tail(F.linear(last_hidden[:, 0], t.codec_head).float(), opt.suppress_tail, cfg.codec_eos_token_id)
    if not allow_eos:
        first[:, cfg.codec_eos_token_id] = -1e30
    first = repetition_penalty(first, history, opt.repetition_penalty)
    code0 = apply_sampling(first, opt.temperature, opt.top_k, opt.top_p, generator)
    cols = [code0]
    emb = t.embed_codec(code0[:, None])
    summed = emb
    cp, cpc = t.code_predictor, cfg.code_predictor
    stack = _Stack(cp.model, cpc.qwen(), B, cfg.num_code_groups + 1)
    proj = lambda x: F.linear(x, cp.input_projection, cp.input_projection_bias)
    stack.run(proj(last_hidden))
    h = stack.run(proj(emb))
    pick = lambda xs, g, d: d if xs is None or g >= len(xs) else xs[g]
    for g in range(cfg.num_code_groups - 1):
        logits = F.linear(h[:, 0], cp.lm_heads[g])
        code = apply_sampling(logits, pick(opt.subtalker_temperatures_by_group, g, opt.subtalker_temperature),
                              pick(opt.subtalker_top_ks_by_group, g, opt.subtalker_top_k), pick(opt.subtalker_top_ps_by_group, g, opt.subtalker_top_p), generator)
        cols.append(code)
        e = F.embedding(code[:, None], cp.input_embeddings[g])
        summed = summed + e
        if g + 1 < cfg.num_code_groups - 1:
            h = stack.run(proj(e))
    return torch.stack(cols, 1), summed


@torch.no_grad()
def stream_codes(t: Talker, talker_inputs: torch.Tensor, on_frame: Callable[[int, torch.Tensor], None], max_frames: int = 256, min_new_tokens: int = 2,
                 opt: SamplingOptions = SamplingOptions(), trailing_text_hidden: Optional[torch.Tensor] = None, tts_pad_embed: Optional[torch.Tensor] = None,
                 generator=None) -> List[int]:
    """Calls ``on_frame(step, codes [B, groups])`` per generated frame; returns per-row lengths (the step at which the row
    sampled end-of-sequence, ``max_frames`` if it never did).  The next talker input is the sum of the frame's code
    embeddings plus the step-th trailing text embedding (the pad embedding once the text has run out)."""
    cfg = t.cfg
    B, S, _ = talker_inputs.shape
    if max_frames == 0:
        return [0] * B
    stack = _Stack(t.model, cfg.qwen(), B, S + max_frames + 1)
    last = stack.run(talker_inputs)[:, -1:]
    pad = tts_pad_embed if tts_pad_embed is not None else torch.zeros(B, 1, cfg.hidden_size, dtype=talker_inputs.dtype, device=talker_inputs.device)
    done, lengths = [False] * B, [max_frames] * B
    hist: List[torch.Tensor] = []
    for step in range(max_frames):
        if all(done):
            break
        allow = step >= min_new_tokens
        codes, summed = generate_frame_from_last_hidden(t, last, torch.stack(hist, 1) if hist else None, allow, opt, generator)
        on_frame(step, codes)
        hist.append(codes[:, 0])
        for b, tok in enumerate(codes[:, 0].tolist()):
            if not done[b] and allow and tok == cfg.codec_eos_token_id:
                done[b], lengths[b] = True, step
        add = trailing_text_hidden[:, step:step + 1] if trailing_text_hidden is not None and step < trailing_text_hidden.shape[1] else pad
        last = stack.run(summed + add)
    return lengths


def generate_codes_with_lengths(t: Talker, talker_inputs, max_frames=256, **kw) -> Tuple[torch.Tensor, List[int]]:
    """[B, max_frames, groups] padded with ``codec_pad_id`` after generation stops, plus the per-row lengths."""
    frames: List[torch.Tensor] = []
    lengths = stream_codes(t, talker_inputs, lambda s, f: frames.append(f), max_frames, **kw)
    B = talker_inputs.shape[0]
    pad = torch.full((B, t.cfg.num_code_groups), t.cfg.codec_pad_id, dtype=torch.int64, device=talker_inputs.device)
    frames += [pad] * (max_frames - len(frames))
    return (torch.stack(frames, 1) if frames else torch.zeros(B, 0, t.cfg.num_code_groups, dtype=torch.int64)), lengths


# ---- speaker encoder (ECAPA-TDNN) ---------------------------------------------------------------------------------------------------
def _tdnn(x, w, b, dilation):
    k = w.shape[-1]
    return F.relu(F.conv1d(x, w, b, padding=dilation * (k - 1) // 2, dilation=dilation))


@dataclass
class SERes2Block:
    tdnn1: Tuple[torch.Tensor, torch.Tensor]
    res2: List[Tuple[torch.Tensor, torch.Tensor]]
    tdnn2: Tuple[torch.Tensor, torch.Tensor]
    se1: Tuple[torch.Tensor, torch.Tensor]
    se2: Tuple[torch.Tensor, torch.Tensor]
    dilation: int

    def forward(self, x):
        h = _tdnn(x, *self.tdnn1, 1)
        parts = h.chunk(len(self.res2) + 1, dim=1)
        outs, prev = [parts[0]], None
        for i, (w, b) in enumerate(self.res2):
            prev = _tdnn(parts[i + 1] if i == 0 else parts[i + 1] + prev, w, b, self.dilation)
            outs.append(prev)
        h = _tdnn(torch.cat(outs, 1), *self.tdnn2, 1)
        gate = torch.sigmoid(F.conv1d(F.relu(F.conv1d(h.mean(2, keepdim=True), *self.se1)), *self.se2))
        return h * gate + x


@dataclass
class SpeakerEncoder:
    cfg: SpeakerEncoderConfig
    tdnn0: Tuple[torch.Tensor, torch.Tensor]
    blocks: List[SERes2Block]
    mfa: Tuple[torch.Tensor, torch.Tensor]
    asp_tdnn: Tuple[torch.Tensor, torch.Tensor]
    asp_conv: Tuple[torch.Tensor, torch.Tensor]
    fc: Tuple[torch.Tensor, torch.Tensor]

    @torch.no_grad()
    def forward(self, mel: torch.Tensor) -> torch.Tensor:
        """mel: [B, frames, mel_dim] -> speaker embedding [B, enc_dim]."""
        c = self.cfg
        x = _tdnn(mel.transpose(1, 2), *self.tdnn0, c.enc_dilations[0])
        feats = []
        for blk in self.blocks:
            x = blk.forward(x)
            feats.append(x)
        x = _tdnn(torch.cat(feats, 1), *self.mfa, c.enc_dilations[4])
        T = x.shape[2]
        mean = x.mean(2, keepdim=True)
        std = torch.sqrt(((x - mean) ** 2).mean(2, keepdim=True) + 1e-12)
        att = torch.tanh(_tdnn(torch.cat([x, mean.expand(-1, -1, T), std.expand(-1, -1, T)], 1), *self.asp_tdnn, 1))
        att = torch.softmax(F.conv1d(att, *self.asp_conv), 2)
        wm = (att * x).sum(2, keepdim=True)
        ws = torch.sqrt((att * (x - wm) ** 2).sum(2, keepdim=True) + 1e-12)
        return F.conv1d(torch.cat([wm, ws], 1), *self.fc)[:, :, 0]


def init_speaker_encoder(cfg: SpeakerEncoderConfig, device="cpu", dtype=torch.float32, seed=0) -> SpeakerEncoder:
    g = torch.Generator().manual_seed(seed)

    def conv(o, i, k):
        return ((torch.randn(o, i, k, generator=g) * (i * k) ** -0.5).to(device=device, dtype=dtype), torch.zeros(o, device=device, dtype=dtype))
    c, k, d = cfg.enc_channels, cfg.enc_kernel_sizes, cfg.enc_dilations
    part = c[0] // cfg.enc_res2net_scale
    blocks = [SERes2Block(conv(c[i], c[i - 1], 1), [conv(part, part, k[i]) for _ in range(cfg.enc_res2net_scale - 1)], conv(c[i], c[i], 1),
                          conv(cfg.enc_se_channels, c[i], 1), conv(c[i], cfg.enc_se_channels, 1), d[i]) for i in (1, 2, 3)]
    return SpeakerEncoder(cfg, conv(c[0], cfg.mel_dim, k[0]), blocks, conv(c[4], c[1] + c[2] + c[3], k[4]), conv(cfg.enc_attention_channels, 3 * c[4], 1),
                          conv(c[4], cfg.enc_attention_channels, 1), conv(cfg.enc_dim, 2 * c[4], 1))


# ---- 12 Hz speech tokenizer decoder ----------------------------------------------------------------------------------------------------
@dataclass
class SpeechDecoderConfig:
    num_quantizers: int = 16
    num_semantic_quantizers: int = 1
    codebook_size: int = 2048
    codebook_dim: int = 256
    rvq_out_dim: int = 512
    latent_dim: int = 1024
    hidden_size: int = 512
    num_layers: int = 8
    num_heads: int = 16
    head_dim: int = 64
    ffn_dim: int = 1024
    sliding_window: int = 72
    upsample_stages: int = 2
    decoder_dim: int = 1536
    decoder_rates: Tuple[int, ...] = (8, 5, 4, 3)
    sample_rate: int = 24000

    @property
    def upsample_rate(self) -> int:
        r = 2 ** self.upsample_stages
        for x in self.decoder_rates:
            r *= x
        return r


def snake_beta(x, alpha, beta):
    a, b = torch.exp(alpha)[None, :, None], torch.exp(beta)[None, :, None]
    return x + torch.sin(x * a).pow(2) / (b + 1e-9)


def causal_conv1d(x, w, b, dilation=1, groups=1):
    return F.conv1d(F.pad(x, (dilation * (w.shape[-1] - 1), 0)), w, b, dilation=dilation, groups=groups)


def causal_trans_conv1d(x, w, b, stride, right_pad):
    y = F.conv_transpose1d(x, w, b, stride=stride)
    return y[:, :, :y.shape[2] - right_pad] if right_pad else y


@dataclass
class SpeechDecoder:
    cfg: SpeechDecoderConfig
    p: Dict[str, torch.Tensor]

    @property
    def device(self): return self.p["decoder.pre_conv.conv.weight"].device

    def _codebook(self, prefix: str, k: int) -> torch.Tensor:
        usage = self.p[f"{prefix}.vq.layers.{k}._codebook.cluster_usage"].float().clamp_min(1e-5)
        return (self.p[f"{prefix}.vq.layers.{k}._codebook.embedding_sum"].float() / usage[:, None]).to(self.p[f"{prefix}.output_proj.weight"].dtype)

    def _rvq(self, prefix: str, codes: torch.Tensor) -> torch.Tensor:
        q = sum(F.embedding(codes[:, k], self._codebook(prefix, k)) for k in range(codes.shape[1]))
        return F.conv1d(q.transpose(1, 2), self.p[f"{prefix}.output_proj.weight"])

    def _res_unit(self, pre: str, x, dilation):
        p = self.p
        h = causal_conv1d(snake_beta(x, p[pre + ".act1.alpha"], p[pre + ".act1.beta"]), p[pre + ".conv1.conv.weight"], p[pre + ".conv1.conv.bias"], dilation)
        return x + causal_conv1d(snake_beta(h, p[pre + ".act2.alpha"], p[pre + ".act2.beta"]), p[pre + ".conv2.conv.weight"], p[pre + ".conv2.conv.bias"])

    @torch.no_grad()
    def decode(self, codes: torch.Tensor) -> torch.Tensor:
        """codes: [B, num_quantizers, frames] -> waveform [B, 1, frames * upsample_rate] in [-1, 1]."""
        c, p = self.cfg, self.p
        ns = c.num_semantic_quantizers
        x = self._rvq("decoder.quantizer.rvq_first", codes[:, :ns]) + self._rvq("decoder.quantizer.rvq_rest", codes[:, ns:])
        x = causal_conv1d(x, p["decoder.pre_conv.conv.weight"], p["decoder.pre_conv.conv.bias"])
        B, _, T = x.shape
        h = F.linear(x.transpose(1, 2), p["decoder.pre_transformer.input_proj.weight"], p["decoder.pre_transformer.input_proj.bias"])
        rope = Q.RoPECache.init(T, c.head_dim // 2, 10000.0, h.device)
        cos, sin = rope.rows(0, T)
        for i in range(c.num_layers):
            L = f"decoder.pre_transformer.layers.{i}."
            n = _rms(h, p[L + "input_layernorm.weight"], 1e-5)
            q, k, v = (F.linear(n, p[L + f"self_attn.{x_}_proj.weight"]).reshape(B, T, c.num_heads, c.head_dim) for x_ in ("q", "k", "v"))
            q, k = apply_rotary_partial(q, cos, sin).transpose(1, 2), apply_rotary_partial(k, cos, sin).transpose(1, 2)
            a = attention(q, k, v.transpose(1, 2), causal=True, window=c.sliding_window).transpose(1, 2).reshape(B, T, -1)
            h = h + F.linear(a, p[L + "self_attn.o_proj.weight"]) * p[L + "self_attn_layer_scale.scale"]
            n = _rms(h, p[L + "post_attention_layernorm.weight"], 1e-5)
            mlp = F.linear(F.silu(F.linear(n, p[L + "mlp.gate_proj.weight"])) * F.linear(n, p[L + "mlp.up_proj.weight"]), p[L + "mlp.down_proj.weight"])
            h = h + mlp * p[L + "mlp_layer_scale.scale"]
        h = _rms(h, p["decoder.pre_transformer.norm.weight"], 1e-5)
        x = F.linear(h, p["decoder.pre_transformer.output_proj.weight"], p["decoder.pre_transformer.output_proj.bias"]).transpose(1, 2)
        for s in range(c.upsample_stages):
            U = f"decoder.upsample.{s}."
            x = causal_trans_conv1d(x, p[U + "0.conv.weight"], p[U + "0.conv.bias"], 2, 0)
            r = causal_conv1d(x, p[U + "1.dwconv.conv.weight"], p[U + "1.dwconv.conv.bias"], groups=x.shape[1]).transpose(1, 2)
            r = F.layer_norm(r, (r.shape[-1],), p[U + "1.norm.weight"], p[U + "1.norm.bias"], 1e-6)
            r = F.linear(F.gelu(F.linear(r, p[U + "1.pwconv1.weight"], p[U + "1.pwconv1.bias"])), p[U + "1.pwconv2.weight"], p[U + "1.pwconv2.bias"])
            x = x + (r * p[U + "1.gamma"]).transpose(1, 2)
        x = causal_conv1d(x, p["decoder.decoder.0.conv.weight"], p["decoder.decoder.0.conv.bias"])
        for i, rate in enumerate(c.decoder_rates, start=1):
            Bk = f"decoder.decoder.{i}.block."
            x = snake_beta(x, p[Bk + "0.alpha"], p[Bk + "0.beta"])
            x = causal_trans_conv1d(x, p[Bk + "1.conv.weight"], p[Bk + "1.conv.bias"], rate, rate)
            for j, dil in enumerate((1, 3, 9), start=2):
                x = self._res_unit(f"{Bk}{j}", x, dil)
        n = len(c.decoder_rates)
        x = snake_beta(x, p[f"decoder.decoder.{n + 1}.alpha"], p[f"decoder.decoder.{n + 1}.beta"])
        x = causal_conv1d(x, p[f"decoder.decoder.{n + 2}.conv.weight"], p[f"decoder.decoder.{n + 2}.conv.bias"])
        return x.clamp(-1.0, 1.0)

    def decode_chunked(self, codes: torch.Tensor, chunk_size: int = 300, left_context: int = 25) -> torch.Tensor:
        """Long inputs in chunks of ``chunk_size`` frames, each decoded with up to ``left_context`` earlier frames whose
        samples are dropped again."""
        T, r = codes.shape[2], self.cfg.upsample_rate
        if T == 0:
            return torch.zeros(codes.shape[0], 1, 0, device=codes.device)
        chunk_size, out, start = max(1, chunk_size), [], 0
        while start < T:
            cur, ctx = min(chunk_size, T - start), min(start, left_context)
            wav = self.decode(codes[:, :, start - ctx:start + cur])
            out.append(wav[:, :, ctx * r:(ctx + cur) * r])
            start += cur
        return torch.cat(out, 2)


class DecodeStream:
    """Incremental decoding: frames are pushed as the talker emits them; every ``chunk_size`` new frames one chunk is decoded
    with left context and its samples returned."""

    def __init__(self, dec: SpeechDecoder, batch: int = 1, chunk_size: int = 1, left_context: int = 25):
        self.dec, self.chunk_size, self.left_context = dec, max(1, chunk_size), left_context
        self.codes = torch.zeros(batch, dec.cfg.num_quantizers, 0, dtype=torch.int64, device=dec.device)
        self.emitted = 0

    def _emit(self, upto: int) -> torch.Tensor:
        ctx, r = min(self.emitted, self.left_context), self.dec.cfg.upsample_rate
        wav = self.dec.decode(self.codes[:, :, self.emitted - ctx:upto])
        self.emitted, out = upto, wav[:, :, ctx * r:]
        return out

    def push(self, frames: torch.Tensor) -> torch.Tensor:
        """frames: [B, num_quantizers, n] -> newly available samples [B, 1, m] (m may be 0)."""
        self.codes = torch.cat([self.codes, frames.to(self.codes.device)], 2)
        outs = []
        while self.codes.shape[2] - self.emitted >= self.chunk_size:
            outs.append(self._emit(self.emitted + self.chunk_size))
        return torch.cat(outs, 2) if outs else torch.zeros(self.codes.shape[0], 1, 0, device=self.codes.device)

    def flush(self) -> torch.Tensor:
        if self.codes.shape[2] == self.emitted:
            return torch.zeros(self.codes.shape[0], 1, 0, device=self.codes.device)
        return self._emit(self.codes.shape[2])


def init_speech_decoder(cfg: SpeechDecoderConfig, device="cpu", dtype=torch.float32, seed=0) -> SpeechDecoder:
    g = torch.Generator().manual_seed(seed)
    p: Dict[str, torch.Tensor] = {}
    w = lambda *s, fan=None: (torch.randn(*s, generator=g) * (fan or s[-1]) ** -0.5).to(device=device, dtype=dtype)
    z = lambda *s: torch.zeros(*s, device=device, dtype=dtype)
    o = lambda *s: torch.ones(*s, device=device, dtype=dtype)
    for name, n in (("rvq_first", cfg.num_semantic_quantizers), ("rvq_rest", cfg.num_quantizers - cfg.num_semantic_quantizers)):
        pre = f"decoder.quantizer.{name}"
        p[pre + ".output_proj.weight"] = w(cfg.rvq_out_dim, cfg.codebook_dim, 1, fan=cfg.codebook_dim)
        for k in range(n):
            p[f"{pre}.vq.layers.{k}._codebook.cluster_usage"] = (torch.rand(cfg.codebook_size, generator=g) + 0.5).to(device)
            p[f"{pre}.vq.layers.{k}._codebook.embedding_sum"] = torch.randn(cfg.codebook_size, cfg.codebook_dim, generator=g).to(device)
    H, Ld = cfg.hidden_size, cfg.latent_dim
    p["decoder.pre_conv.conv.weight"], p["decoder.pre_conv.conv.bias"] = w(Ld, cfg.rvq_out_dim, 3, fan=3 * cfg.rvq_out_dim), z(Ld)
    p["decoder.pre_transformer.input_proj.weight"], p["decoder.pre_transformer.input_proj.bias"] = w(H, Ld), z(H)
    p["decoder.pre_transformer.output_proj.weight"], p["decoder.pre_transformer.output_proj.bias"] = w(Ld, H), z(Ld)
    p["decoder.pre_transformer.norm.weight"] = o(H)
    A = cfg.num_heads * cfg.head_dim
    for i in range(cfg.num_layers):
        L = f"decoder.pre_transformer.layers.{i}."
        p[L + "input_layernorm.weight"], p[L + "post_attention_layernorm.weight"] = o(H), o(H)
        for n_ in ("q", "k", "v"):
            p[L + f"self_attn.{n_}_proj.weight"] = w(A, H)
        p[L + "self_attn.o_proj.weight"] = w(H, A)
        p[L + "mlp.gate_proj.weight"], p[L + "mlp.up_proj.weight"], p[L + "mlp.down_proj.weight"] = w(cfg.ffn_dim, H), w(cfg.ffn_dim, H), w(H, cfg.ffn_dim)
        p[L + "self_attn_layer_scale.scale"], p[L + "mlp_layer_scale.scale"] = o(H) * 0.1, o(H) * 0.1
    for s in range(cfg.upsample_stages):
        U = f"decoder.upsample.{s}."
        p[U + "0.conv.weight"], p[U + "0.conv.bias"] = w(Ld, Ld, 2, fan=Ld), z(Ld)
        p[U + "1.dwconv.conv.weight"], p[U + "1.dwconv.conv.bias"] = w(Ld, 1, 7, fan=7), z(Ld)
        p[U + "1.norm.weight"], p[U + "1.norm.bias"] = o(Ld), z(Ld)
        p[U + "1.pwconv1.weight"], p[U + "1.pwconv1.bias"], p[U + "1.pwconv2.weight"], p[U + "1.pwconv2.bias"] = w(4 * Ld, Ld), z(4 * Ld), w(Ld, 4 * Ld), z(Ld)
        p[U + "1.gamma"] = o(Ld) * 0.1
    dim = cfg.decoder_dim
    p["decoder.decoder.0.conv.weight"], p["decoder.decoder.0.conv.bias"] = w(dim, Ld, 7, fan=7 * Ld), z(dim)
    for i, rate in enumerate(cfg.decoder_rates, start=1):
        Bk, out = f"decoder.decoder.{i}.block.", dim // 2
        p[Bk + "0.alpha"], p[Bk + "0.beta"] = z(dim), z(dim)
        p[Bk + "1.conv.weight"], p[Bk + "1.conv.bias"] = w(dim, out, 2 * rate, fan=dim), z(out)
        for j in (2, 3, 4):
            R = f"{Bk}{j}"
            p[R + ".act1.alpha"], p[R + ".act1.beta"], p[R + ".act2.alpha"], p[R + ".act2.beta"] = z(out), z(out), z(out), z(out)
            p[R + ".conv1.conv.weight"], p[R + ".conv1.conv.bias"] = w(out, out, 7, fan=7 * out), z(out)
            p[R + ".conv2.conv.weight"], p[R + ".conv2.conv.bias"] = w(out, out, 1, fan=out), z(out)
        dim = out
    n = len(cfg.decoder_rates)
    p[f"decoder.decoder.{n + 1}.alpha"], p[f"decoder.decoder.{n + 1}.beta"] = z(dim), z(dim)
    p[f"decoder.decoder.{n + 2}.conv.weight"], p[f"decoder.decoder.{n + 2}.conv.bias"] = w(1, dim, 7, fan=7 * dim), z(1)
    return SpeechDecoder(cfg, p)


def load_speech_decoder(path: str, cfg: Optional[SpeechDecoderConfig] = None, device="cpu", dtype=torch.float32) -> SpeechDecoder:
    """The decoder keeps the checkpoint's tensor names; codebook statistics stay in fp32."""
    from ..io import safetensors as st
    src = st.Source.open(path)
    p = {}
    for n in src.names():
        if n.startswith("decoder."):
            t = src.load(n)
            p[n] = t.to(device) if "_codebook" in n else t.to(device=device, dtype=dtype)
    return SpeechDecoder(cfg or SpeechDecoderConfig(), p)


# ---- full model -----------------------------------------------------------------------------------------------------------------------
@dataclass
class Qwen3TTS:
    cfg: Qwen3TTSConfig
    talker: Talker
    speaker_encoder: Optional[SpeakerEncoder]
    speech_decoder: Optional[SpeechDecoder] = None

    def get_supported_languages(self): return self.cfg.supported_languages()
    def get_supported_speakers(self): return self.cfg.supported_speakers()

    def extract_speaker_embedding(self, mel: torch.Tensor) -> torch.Tensor:
        if self.speaker_encoder is None:
            raise ValueError("this Qwen3-TTS variant has no speaker encoder")
        return self.speaker_encoder.forward(mel.to(self.talker.device))

    def build_talker_inputs(self, text_ids, instruct_ids=None, speaker_embedding: Optional[torch.Tensor] = None, speaker: Optional[str] = None,
                            language: Optional[str] = None) -> torch.Tensor:
        """``[codec_bos, (language tag), (speaker), text...]``: a named speaker / language enters as its codec-token embedding,
        a cloned voice as the speaker-encoder embedding."""
        t, c = self.talker, self.talker.cfg
        x = t.build_inputs_from_text(text_ids, instruct_ids)
        extra = []
        if language and language != "auto":
            if language not in c.codec_language_id:
                raise ValueError(f"Unsupported language: {language}")
            extra.append(t.embed_codec(torch.full((x.shape[0], 1), c.codec_language_id[language], dtype=torch.int64)))
        if speaker is not None:
            if speaker not in c.spk_id:
                raise ValueError(f"Unsupported speaker: {speaker}")
            extra.append(t.embed_codec(torch.full((x.shape[0], 1), c.spk_id[speaker], dtype=torch.int64)))
        elif speaker_embedding is not None:
            extra.append(speaker_embedding.to(x.dtype)[:, None])
        return torch.cat([x[:, :1], *extra, x[:, 1:]], 1) if extra else x

    def generate_from_text(self, text_ids, max_frames=256, opt: SamplingOptions = SamplingOptions(), generator=None, **cond) -> Tuple[torch.Tensor, List[int]]:
        return generate_codes_with_lengths(self.talker, self.build_talker_inputs(text_ids, **cond), max_frames, opt=opt, generator=generator)

    def synthesize(self, text_ids, max_frames=256, opt: SamplingOptions = SamplingOptions(), generator=None, **cond) -> List[torch.Tensor]:
        """Waveforms per row (the first ``num_quantizers`` codebooks of every generated frame go to the speech decoder)."""
        if self.speech_decoder is None:
            raise ValueError("no speech decoder attached")
        codes, lengths = self.generate_from_text(text_ids, max_frames, opt, generator, **cond)
        nq = self.speech_decoder.cfg.num_quantizers
        return [self.speech_decoder.decode_chunked(codes[b:b + 1, :max(1, n), :nq].transpose(1, 2))[0, 0] for b, n in enumerate(lengths)]

    def stream(self, text_ids, on_audio: Callable[[torch.Tensor], None], max_frames=256, chunk_frames: int = 4, opt: SamplingOptions = SamplingOptions(),
               generator=None, **cond) -> int:
        """Single-row streaming: audio chunks are handed to ``on_audio`` while the talker is still generating.  Returns
        the number of frames."""
        ds = DecodeStream(self.speech_decoder, 1, chunk_frames)
        nq, eos = self.speech_decoder.cfg.num_quantizers, self.talker.cfg.codec_eos_token_id
        n = [0]

        def on_frame(step, codes):
            if int(codes[0, 0]) == eos and step >= 2:
                return
            n[0] += 1
            wav = ds.push(codes[:, :nq, None])
            if wav.shape[2]:
                on_audio(wav[0, 0])
        stream_codes(self.talker, self.build_talker_inputs(text_ids, **cond), on_frame, max_frames, opt=opt, generator=generator)
        tail = ds.flush()
        if tail.shape[2]:
            on_audio(tail[0, 0])
        return n[0]


def init(cfg: Qwen3TTSConfig, device="cpu", dtype=torch.float32, seed=0, speech_decoder_cfg: Optional[SpeechDecoderConfig] = None) -> Qwen3TTS:
    enc = init_speaker_encoder(cfg.speaker_encoder, device, dtype, seed + 5) if cfg.tts_model_type == "base" else None
    dec = init_speech_decoder(speech_decoder_cfg, device, dtype, seed + 7) if speech_decoder_cfg is not None else None
    return Qwen3TTS(cfg, init_talker(cfg.talker, device, dtype, seed), enc, dec)
