"""Whisper: conv + transformer audio encoder, transformer decoder with self- and cross-attention KV caches,
greedy / sampled / beam decoding with timestamp rules, temperature fallback and chunked transcription
(Tyr/Model/Whisper/{Config,ConfigIO,Model,Weights,Transcribe}.lean)."""
from __future__ import annotations

import json
import math
import os
import zlib
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..audio import frontend as fe
from ..io import safetensors as st
from ..ops.attention import attention
from .common import KVCache, lin


@dataclass
class WhisperConfig:
    num_mel_bins: int = 80
    vocab_size: int = 51865
    d_model: int = 384
    encoder_layers: int = 4
    encoder_attention_heads: int = 6
    encoder_ffn_dim: int = 1536
    decoder_layers: int = 4
    decoder_attention_heads: int = 6
    decoder_ffn_dim: int = 1536
    max_source_positions: int = 1500
    max_target_positions: int = 448
    activation_function: str = "gelu"
    layer_norm_eps: float = 1e-5
    eos_token_id: int = 50257
    decoder_start_token_id: int = 50258
    suppress_tokens: Tuple[int, ...] = ()
    begin_suppress_tokens: Tuple[int, ...] = ()

    def __post_init__(self):
        e = lambda m: ValueError(f"Invalid Whisper config: {m}")
        if self.num_mel_bins <= 0 or self.vocab_size <= 0 or self.max_target_positions <= 0 or self.layer_norm_eps <= 0:
            raise e("mel bins, vocabulary, target positions and layer-norm eps must be positive")
        for h in (self.encoder_attention_heads, self.decoder_attention_heads):
            if h <= 0 or self.d_model % h:
                raise e(f"attention heads ({h}) must divide d_model ({self.d_model})")
        if self.activation_function not in ("gelu", "relu"):
            raise e(f"unsupported activation {self.activation_function!r}")
        for t in (self.eos_token_id, self.decoder_start_token_id, *self.suppress_tokens, *self.begin_suppress_tokens):
            if not 0 <= t < self.vocab_size:
                raise e(f"token id {t} is outside the vocabulary")

    @staticmethod
    def conv2_output_seq(frames: int) -> int:
        return (frames + 2 - 2 - 1) // 2 + 1

    @staticmethod
    def from_json(j: dict) -> "WhisperConfig":
        d = WhisperConfig()
        g = lambda k, a: j.get(k, getattr(d, a))
        return WhisperConfig(g("num_mel_bins", "num_mel_bins"), g("vocab_size", "vocab_size"), g("d_model", "d_model"),
                             g("encoder_layers", "encoder_layers"), g("encoder_attention_heads", "encoder_attention_heads"),
                             g("encoder_ffn_dim", "encoder_ffn_dim"), g("decoder_layers", "decoder_layers"),
                             g("decoder_attention_heads", "decoder_attention_heads"), g("decoder_ffn_dim", "decoder_ffn_dim"),
                             g("max_source_positions", "max_source_positions"), g("max_target_positions", "max_target_positions"),
                             g("activation_function", "activation_function"), float(g("layer_norm_eps", "layer_norm_eps")) if "layer_norm_eps" in j else d.layer_norm_eps,
                             g("eos_token_id", "eos_token_id"), g("decoder_start_token_id", "decoder_start_token_id"),
                             tuple(j.get("suppress_tokens") or ()), tuple(j.get("begin_suppress_tokens") or ()))

    @staticmethod
    def load_from_pretrained_dir(d: str) -> "WhisperConfig":
        with open(os.path.join(d, "config.json")) as f:
            return WhisperConfig.from_json(json.load(f))


@dataclass
class LayerNorm:
    weight: torch.Tensor
    bias: torch.Tensor

    def __call__(self, x, eps):
        return F.layer_norm(x.float(), (x.shape[-1],), self.weight.float(), self.bias.float(), eps).to(x.dtype)


@dataclass
class Attention:
    q_w: torch.Tensor
    k_w: torch.Tensor
    v_w: torch.Tensor
    o_w: torch.Tensor
    q_b: Optional[torch.Tensor] = None
    v_b: Optional[torch.Tensor] = None
    o_b: Optional[torch.Tensor] = None
    k_b: Optional[torch.Tensor] = None


@dataclass
class EncoderLayer:
    self_attn: Attention
    self_attn_layer_norm: LayerNorm
    fc1_w: torch.Tensor
    fc1_b: torch.Tensor
    fc2_w: torch.Tensor
    fc2_b: torch.Tensor
    final_layer_norm: LayerNorm


@dataclass
class DecoderLayer:
    self_attn: Attention
    self_attn_layer_norm: LayerNorm
    encoder_attn: Attention
    encoder_attn_layer_norm: LayerNorm
    fc1_w: torch.Tensor
    fc1_b: torch.Tensor
    fc2_w: torch.Tensor
    fc2_b: torch.Tensor
    final_layer_norm: LayerNorm


@dataclass
class WhisperModel:
    cfg: WhisperConfig
    conv1_w: torch.Tensor
    conv1_b: torch.Tensor
    conv2_w: torch.Tensor
    conv2_b: torch.Tensor
    enc_pos: torch.Tensor
    enc_layers: List[EncoderLayer]
    enc_ln: LayerNorm
    embed_tokens: torch.Tensor
    dec_pos: torch.Tensor
    dec_layers: List[DecoderLayer]
    dec_ln: LayerNorm
    proj_out: torch.Tensor            # tied to embed_tokens when the checkpoint has no proj_out

    @property
    def device(self): return self.embed_tokens.device
    @property
    def dtype(self): return self.embed_tokens.dtype


def _act(cfg, x):
    return F.gelu(x) if cfg.activation_function == "gelu" else F.relu(x)


def _heads(x, H):
    B, S, C = x.shape
    return x.reshape(B, S, H, C // H).transpose(1, 2)


def attn_forward(a: Attention, x, H: int, kv_src=None, causal=False, cache: Optional[KVCache] = None, static_kv=None):
    """Self attention (``kv_src`` None) with an optional growing cache, or cross attention over ``kv_src`` /
    precomputed ``static_kv``.  Whisper scales q by head_dim^-0.5, which equals the default softmax scale."""
    q = _heads(lin(x, a.q_w, a.q_b), H)
    if static_kv is not None:
        k, v = static_kv
    else:
        src = x if kv_src is None else kv_src
        k, v = _heads(lin(src, a.k_w, a.k_b), H), _heads(lin(src, a.v_w, a.v_b), H)
        if cache is not None:
            cache.write(k, v)
            k, v = cache.view()
    is_causal = causal and q.shape[2] > 1
    o = attention(q, k, v, causal=is_causal)
    B, _, S, D = o.shape
    return lin(o.transpose(1, 2).reshape(B, S, H * D), a.o_w, a.o_b)


def encode(m: WhisperModel, features: torch.Tensor) -> torch.Tensor:
    """features [B, mels, frames] -> [B, frames/2, d_model]."""
    cfg = m.cfg
    x = F.gelu(F.conv1d(features.to(m.dtype), m.conv1_w, m.conv1_b, padding=1))
    x = F.gelu(F.conv1d(x, m.conv2_w, m.conv2_b, stride=2, padding=1)).transpose(1, 2)
    if x.shape[1] > cfg.max_source_positions:
        raise ValueError(f"encoder input has {x.shape[1]} positions, the model supports {cfg.max_source_positions}")
    x = x + m.enc_pos[:x.shape[1]]
    for l in m.enc_layers:
        x = x + attn_forward(l.self_attn, l.self_attn_layer_norm(x, cfg.layer_norm_eps), cfg.encoder_attention_heads)
        h = l.final_layer_norm(x, cfg.layer_norm_eps)
        x = x + lin(_act(cfg, lin(h, l.fc1_w, l.fc1_b)), l.fc2_w, l.fc2_b)
    return m.enc_ln(x, cfg.layer_norm_eps)


def decode(m: WhisperModel, tokens: torch.Tensor, enc: torch.Tensor, position: int = 0,
           self_caches: Optional[List[KVCache]] = None, cross_kv: Optional[List[Tuple[torch.Tensor, torch.Tensor]]] = None) -> torch.Tensor:
    """tokens [B, S] at positions ``position..`` -> logits [B, S, V].  With caches, earlier tokens are not recomputed."""
    cfg = m.cfg
    S = tokens.shape[1]
    if position + S > cfg.max_target_positions:
        raise ValueError("decoder position exceeds max_target_positions")
    x = F.embedding(tokens, m.embed_tokens) + m.dec_pos[position:position + S]
    H = cfg.decoder_attention_heads
    for i, l in enumerate(m.dec_layers):
        c = self_caches[i] if self_caches is not None else None
        x = x + attn_forward(l.self_attn, l.self_attn_layer_norm(x, cfg.layer_norm_eps), H, causal=True, cache=c)
        x = x + attn_forward(l.encoder_attn, l.encoder_attn_layer_norm(x, cfg.layer_norm_eps), H, kv_src=enc,
                             static_kv=cross_kv[i] if cross_kv is not None else None)
        h = l.final_layer_norm(x, cfg.layer_norm_eps)
        x = x + lin(_act(cfg, lin(h, l.fc1_w, l.fc1_b)), l.fc2_w, l.fc2_b)
    return lin(m.dec_ln(x, cfg.layer_norm_eps), m.proj_out)


class DecodeSession:
    """Cross-attention K/V computed once per audio chunk; self-attention caches grow per token
    (``LayerCrossCache`` / ``SelfKVCaches`` of Model.lean:402-463)."""

    def __init__(self, m: WhisperModel, enc: torch.Tensor):
        cfg = m.cfg
        self.m, self.enc, self.pos = m, enc, 0
        H = cfg.decoder_attention_heads
        self.cross = [(_heads(lin(enc, l.encoder_attn.k_w, l.encoder_attn.k_b), H), _heads(lin(enc, l.encoder_attn.v_w, l.encoder_attn.v_b), H))
                      for l in m.dec_layers]
        self.caches = [KVCache.allocate(enc.shape[0], H, cfg.max_target_positions, cfg.d_model // H, m.device, m.dtype)
                       for _ in m.dec_layers]

    @torch.no_grad()
    def step(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B, S] -> logits of the last position [B, V]."""
        logits = decode(self.m, tokens, self.enc, self.pos, self.caches, self.cross)
        self.pos += tokens.shape[1]
        return logits[:, -1].float()

    def fork(self) -> "DecodeSession":
        o = object.__new__(DecodeSession)
        o.m, o.enc, o.pos, o.cross = self.m, self.enc, self.pos, self.cross
        o.caches = [c.clone() for c in self.caches]
        return o


def init(cfg: WhisperConfig, device="cpu", dtype=torch.float32, seed=0) -> WhisperModel:
    g = torch.Generator().manual_seed(seed)
    d = cfg.d_model
    w = lambda *s: (torch.randn(*s, generator=g) * (s[-1] ** -0.5)).to(device=device, dtype=dtype)
    z = lambda n: torch.zeros(n, device=device, dtype=dtype)
    ln = lambda: LayerNorm(torch.ones(d, device=device, dtype=dtype), z(d))
    at = lambda: Attention(w(d, d), w(d, d), w(d, d), w(d, d), z(d), z(d), z(d))
    enc = [EncoderLayer(at(), ln(), w(cfg.encoder_ffn_dim, d), z(cfg.encoder_ffn_dim), w(d, cfg.encoder_ffn_dim), z(d), ln()) for _ in range(cfg.encoder_layers)]
    dec = [DecoderLayer(at(), ln(), at(), ln(), w(cfg.decoder_ffn_dim, d), z(cfg.decoder_ffn_dim), w(d, cfg.decoder_ffn_dim), z(d), ln())
           for _ in range(cfg.decoder_layers)]
    emb = (torch.randn(cfg.vocab_size, d, generator=g) * 0.02).to(device=device, dtype=dtype)
    # sinusoidal encoder positions (fixed in Whisper), learned decoder positions
    half = d // 2
    inv = torch.exp(-math.log(10000.0) / (half - 1) * torch.arange(half))
    ang = torch.arange(cfg.max_source_positions)[:, None] * inv[None]
    enc_pos = torch.cat([ang.sin(), ang.cos()], 1).to(device=device, dtype=dtype)
    return WhisperModel(cfg, (torch.randn(d, cfg.num_mel_bins, 3, generator=g) * (3 * cfg.num_mel_bins) ** -0.5).to(device=device, dtype=dtype), z(d),
                        (torch.randn(d, d, 3, generator=g) * (3 * d) ** -0.5).to(device=device, dtype=dtype), z(d), enc_pos, enc, ln(), emb,
                        (torch.randn(cfg.max_target_positions, d, generator=g) * 0.01).to(device=device, dtype=dtype), dec, ln(), emb)


def load_sharded(model_dir: str, cfg: Optional[WhisperConfig] = None, device="cpu", dtype=torch.float32, log=None) -> WhisperModel:
    cfg = cfg or WhisperConfig.load_from_pretrained_dir(model_dir)
    src = st.Source.open(model_dir)
    g = lambda n, shape=None: _checked(src, n, shape).to(device=device, dtype=dtype)
    opt = lambda n: src.load(n).to(device=device, dtype=dtype) if src.find(n) is not None else None
    d = cfg.d_model
    ln = lambda p: LayerNorm(g(f"{p}.weight", (d,)), g(f"{p}.bias", (d,)))
    at = lambda p: Attention(g(f"{p}.q_proj.weight", (d, d)), g(f"{p}.k_proj.weight", (d, d)), g(f"{p}.v_proj.weight", (d, d)),
                             g(f"{p}.out_proj.weight", (d, d)), opt(f"{p}.q_proj.bias"), opt(f"{p}.v_proj.bias"), opt(f"{p}.out_proj.bias"),
                             opt(f"{p}.k_proj.bias"))
    enc = []
    for i in range(cfg.encoder_layers):
        p = f"model.encoder.layers.{i}"
        enc.append(EncoderLayer(at(f"{p}.self_attn"), ln(f"{p}.self_attn_layer_norm"), g(f"{p}.fc1.weight", (cfg.encoder_ffn_dim, d)),
                                g(f"{p}.fc1.bias"), g(f"{p}.fc2.weight", (d, cfg.encoder_ffn_dim)), g(f"{p}.fc2.bias"), ln(f"{p}.final_layer_norm")))
    dec = []
    for i in range(cfg.decoder_layers):
        p = f"model.decoder.layers.{i}"
        dec.append(DecoderLayer(at(f"{p}.self_attn"), ln(f"{p}.self_attn_layer_norm"), at(f"{p}.encoder_attn"), ln(f"{p}.encoder_attn_layer_norm"),
                                g(f"{p}.fc1.weight", (cfg.decoder_ffn_dim, d)), g(f"{p}.fc1.bias"), g(f"{p}.fc2.weight", (d, cfg.decoder_ffn_dim)),
                                g(f"{p}.fc2.bias"), ln(f"{p}.final_layer_norm")))
    emb = g("model.decoder.embed_tokens.weight", (cfg.vocab_size, d))
    proj = opt("proj_out.weight")
    return WhisperModel(cfg, g("model.encoder.conv1.weight", (d, cfg.num_mel_bins, 3)), g("model.encoder.conv1.bias"),
                        g("model.encoder.conv2.weight", (d, d, 3)), g("model.encoder.conv2.bias"),
                        g("model.encoder.embed_positions.weight", (cfg.max_source_positions, d)), enc, ln("model.encoder.layer_norm"), emb,
                        g("model.decoder.embed_positions.weight", (cfg.max_target_positions, d)), dec, ln("model.decoder.layer_norm"),
                        proj if proj is not None else emb)


def _checked(src, name, shape):
    t = src.load(name)
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise st.SafeTensorsError(f"{name}: expected shape {list(shape)}, got {list(t.shape)}")
    return t


def state_dict(m: WhisperModel) -> Dict[str, torch.Tensor]:
    out = {"model.encoder.conv1.weight": m.conv1_w, "model.encoder.conv1.bias": m.conv1_b, "model.encoder.conv2.weight": m.conv2_w,
           "model.encoder.conv2.bias": m.conv2_b, "model.encoder.embed_positions.weight": m.enc_pos,
           "model.decoder.embed_tokens.weight": m.embed_tokens, "model.decoder.embed_positions.weight": m.dec_pos}

    def ln(p, l):
        out[f"{p}.weight"], out[f"{p}.bias"] = l.weight, l.bias

    def at(p, a):
        for n, t in (("q_proj.weight", a.q_w), ("k_proj.weight", a.k_w), ("v_proj.weight", a.v_w), ("out_proj.weight", a.o_w),
                     ("q_proj.bias", a.q_b), ("v_proj.bias", a.v_b), ("out_proj.bias", a.o_b), ("k_proj.bias", a.k_b)):
            if t is not None:
                out[f"{p}.{n}"] = t
    ln("model.encoder.layer_norm", m.enc_ln); ln("model.decoder.layer_norm", m.dec_ln)
    for kind, layers in (("encoder", m.enc_layers), ("decoder", m.dec_layers)):
        for i, l in enumerate(layers):
            p = f"model.{kind}.layers.{i}"
            at(f"{p}.self_attn", l.self_attn); ln(f"{p}.self_attn_layer_norm", l.self_attn_layer_norm)
            if kind == "decoder":
                at(f"{p}.encoder_attn", l.encoder_attn); ln(f"{p}.encoder_attn_layer_norm", l.encoder_attn_layer_norm)
            out[f"{p}.fc1.weight"], out[f"{p}.fc1.bias"], out[f"{p}.fc2.weight"], out[f"{p}.fc2.bias"] = l.fc1_w, l.fc1_b, l.fc2_w, l.fc2_b
            ln(f"{p}.final_layer_norm", l.final_layer_norm)
    if m.proj_out is not m.embed_tokens:
        out["proj_out.weight"] = m.proj_out
    return out


# ---- transcription ----------------------------------------------------------------------------------------------------
@dataclass
class WhisperDecodeOptions:
    beam_size: int = 1
    best_of: int = 1
    temperature: float = 0.0
    temperature_inc: float = 0.2
    max_temperature: float = 1.0
    top_k: Optional[int] = None
    top_p: float = 1.0
    logprob_threshold: float = -1.0
    no_speech_threshold: float = 0.6
    compression_ratio_threshold: float = 2.4
    condition_on_previous_text: bool = True
    max_context_tokens: Optional[int] = None
    max_new_tokens: Optional[int] = 128
    chunk_overlap_seconds: float = 2.0
    reset_context_on_fallback: bool = True
    no_fallback: bool = True

    def temperatures(self) -> List[float]:
        if self.no_fallback or self.temperature_inc <= 0:
            return [self.temperature]
        out, t = [], self.temperature
        while t <= self.max_temperature + 1e-9:
            out.append(round(t, 6))
            t += self.temperature_inc
        return out


@dataclass
class DecodeTokenRules:
    """Special-token ids of a Whisper vocabulary (resolved from the tokenizer)."""
    sot: int
    eot: int
    transcribe: Optional[int] = None
    translate: Optional[int] = None
    no_timestamps: Optional[int] = None
    timestamp_begin: Optional[int] = None      # id of <|0.00|>; ids above are later timestamps
    no_speech: Optional[int] = None
    language: Optional[int] = None
    suppress: Tuple[int, ...] = ()
    begin_suppress: Tuple[int, ...] = ()

    def prompt(self, with_timestamps: bool, task: str = "transcribe") -> List[int]:
        ids = [self.sot]
        if self.language is not None:
            ids.append(self.language)
        t = self.transcribe if task == "transcribe" else self.translate
        if t is not None:
            ids.append(t)
        if not with_timestamps and self.no_timestamps is not None:
            ids.append(self.no_timestamps)
        return ids


def apply_timestamp_rules(logits: torch.Tensor, generated: Sequence[int], rules: DecodeTokenRules, max_initial_ts: int = 50) -> torch.Tensor:
    """Timestamps come in pairs, never decrease, and the first token of a chunk is a timestamp no later than 1 s
    (Transcribe.lean:503-556, OpenAI's ApplyTimestampRules)."""
    tb = rules.timestamp_begin
    if tb is None:
        return logits
    logits = logits.clone()
    if rules.no_timestamps is not None:
        logits[rules.no_timestamps] = float("-inf")
    seq = list(generated)
    last_ts = len(seq) >= 1 and seq[-1] >= tb
    penult_ts = len(seq) < 2 or seq[-2] >= tb
    if last_ts:
        if penult_ts:
            logits[tb:] = float("-inf")                 # a pair just closed: text must follow
        else:
            logits[:rules.eot] = float("-inf")          # an opened timestamp must be closed (or eot)
    ts = [t for t in seq if t >= tb]
    if ts:
        lo = ts[-1] if (last_ts and not penult_ts) else ts[-1] + 1
        logits[tb:lo] = float("-inf")
    if not seq:
        logits[:tb] = float("-inf")
        logits[tb + max_initial_ts + 1:] = float("-inf")
    lp = torch.log_softmax(logits.float(), -1)
    if torch.logsumexp(lp[tb:], -1) > lp[:tb].max():
        logits[:tb] = float("-inf")                     # timestamps collectively more likely than any text token
    return logits


def compression_ratio(ids: Sequence[int]) -> float:
    raw = b",".join(str(i).encode() for i in ids)
    return len(raw) / max(1, len(zlib.compress(raw)))


def has_repetition_loop(ids: Sequence[int], pattern_len: int = 4, repeats: int = 4, run_len: int = 12) -> bool:
    ids = list(ids)
    if len(ids) >= run_len and len(set(ids[-run_len:])) == 1:
        return True
    for L in range(2, pattern_len + 1):
        if len(ids) >= L * repeats and all(ids[-L * (r + 1):len(ids) - L * r] == ids[-L:] for r in range(repeats)):
            return True
    return False


@dataclass
class DecodeCandidate:
    tokens: List[int]
    avg_logprob: float
    no_speech_prob: float
    temperature: float
    compression_ratio: float

    def needs_fallback(self, o: WhisperDecodeOptions) -> bool:
        return self.compression_ratio > o.compression_ratio_threshold or self.avg_logprob < o.logprob_threshold or has_repetition_loop(self.tokens)

    def is_no_speech(self, o: WhisperDecodeOptions) -> bool:
        return self.no_speech_prob > o.no_speech_threshold and self.avg_logprob < o.logprob_threshold


@torch.no_grad()
def decode_at_temperature(m: WhisperModel, enc: torch.Tensor, prompt: Sequence[int], rules: DecodeTokenRules, opts: WhisperDecodeOptions,
                          temperature: float, with_timestamps: bool, generator=None) -> DecodeCandidate:
    """Greedy (temperature 0, optionally beam search) or sampled decoding of one chunk."""
    cfg = m.cfg
    budget = min(opts.max_new_tokens or cfg.max_target_positions, cfg.max_target_positions - len(prompt))
    suppress = list(rules.suppress) + [rules.sot] + [t for t in (rules.transcribe, rules.translate, rules.language) if t is not None]

    def prepare(logits, gen):
        logits = logits.clone()
        logits[suppress] = float("-inf")
        if not gen:
            logits[list(rules.begin_suppress) + [rules.eot]] = float("-inf")
        return apply_timestamp_rules(logits, gen, rules) if with_timestamps else logits
    sess = DecodeSession(m, enc)
    logits = sess.step(torch.tensor([list(prompt)], device=m.device))[0]
    no_speech = float(torch.softmax(logits, -1)[rules.no_speech]) if rules.no_speech is not None else 0.0
    if temperature == 0.0 and opts.beam_size > 1:
        beams = [(0.0, [], sess, logits)]
        done: List[Tuple[float, List[int]]] = []
        for _ in range(budget):
            cand = []
            for score, gen, s, lg in beams:
                lp = torch.log_softmax(prepare(lg, gen), -1)
                top = torch.topk(lp, opts.beam_size)
                for v, i in zip(top.values.tolist(), top.indices.tolist()):
                    cand.append((score + v, gen + [i], s))
            cand.sort(key=lambda c: -c[0])
            beams = []
            for score, gen, s in cand[:opts.beam_size]:
                if gen[-1] == rules.eot:
                    done.append((score / len(gen), gen[:-1]))
                    continue
                s2 = s.fork()
                beams.append((score, gen, s2, s2.step(torch.tensor([[gen[-1]]], device=m.device))[0]))
            if not beams:
                break
        done += [(sc / max(1, len(g)), g) for sc, g, _, _ in beams]
        avg, toks = max(done, key=lambda d: d[0])
        return DecodeCandidate(toks, avg, no_speech, 0.0, compression_ratio(toks))
    gen, total, scored = [], 0.0, 0
    for _ in range(budget):
        lg = prepare(logits, gen)
        lp = torch.log_softmax(lg, -1)
        if temperature == 0.0:
            tok = int(torch.argmax(lg))
        else:
            from .generation import top_k_filter, top_p_filter
            f = top_p_filter(top_k_filter((lg / temperature)[None], opts.top_k), opts.top_p)[0]
            tok = int(torch.multinomial(torch.softmax(f, -1), 1, generator=generator))
        total += float(lp[tok])
        scored += 1
        if tok == rules.eot:
            break
        gen.append(tok)
        if has_repetition_loop(gen):
            break
        logits = sess.step(torch.tensor([[tok]], device=m.device))[0]
    return DecodeCandidate(gen, total / max(1, scored), no_speech, temperature, compression_ratio(gen))


def decode_with_fallback(m, enc, prompt, rules, opts: WhisperDecodeOptions, with_timestamps: bool, generator=None) -> DecodeCandidate:
    best = None
    for t in opts.temperatures():
        n = opts.best_of if t > 0 else 1
        cands = [decode_at_temperature(m, enc, prompt, rules, opts, t, with_timestamps, generator) for _ in range(n)]
        c = max(cands, key=lambda c: c.avg_logprob)
        best = c if best is None or c.avg_logprob > best.avg_logprob else best
        if not c.needs_fallback(opts):
            return c
    return best


def split_waveform_with_overlap(wave: torch.Tensor, chunk_samples: int, overlap_samples: int) -> List[torch.Tensor]:
    if wave.numel() <= chunk_samples:
        return [wave]
    step = max(1, chunk_samples - overlap_samples)
    return [wave[s:s + chunk_samples] for s in range(0, max(1, wave.numel() - overlap_samples), step)]


def token_overlap_length(a: Sequence[int], b: Sequence[int], max_len: int = 32) -> int:
    """Longest suffix of ``a`` that is a prefix of ``b``."""
    for n in range(min(len(a), len(b), max_len), 0, -1):
        if list(a[-n:]) == list(b[:n]):
            return n
    return 0


def append_with_token_stitch(acc: List[int], nxt: Sequence[int]) -> List[int]:
    return acc + list(nxt[token_overlap_length(acc, nxt):])


@dataclass
class WhisperTranscription:
    text: str
    tokens: List[int]
    segments: List[Tuple[float, float, List[int]]] = field(default_factory=list)


@dataclass
class WhisperBundle:
    model: WhisperModel
    rules: DecodeTokenRules
    decode_text: callable = lambda ids: " ".join(map(str, ids))


@torch.no_grad()
def transcribe_waveform_16k(bundle: WhisperBundle, wave: torch.Tensor, opts: Optional[WhisperDecodeOptions] = None,
                            with_timestamps: bool = False, generator=None) -> WhisperTranscription:
    """30-second chunks with overlap; the previous chunk's text conditions the next; overlapping token runs are
    stitched; chunks judged silent are dropped (Transcribe.lean:1262-1475)."""
    opts = opts or WhisperDecodeOptions()
    m, rules = bundle.model, bundle.rules
    chunk = 30 * fe.SAMPLE_RATE
    parts = split_waveform_with_overlap(wave, chunk, int(opts.chunk_overlap_seconds * fe.SAMPLE_RATE))
    acc: List[int] = []
    segs = []
    context: List[int] = []
    max_ctx = opts.max_context_tokens if opts.max_context_tokens is not None else m.cfg.max_target_positions // 2
    step_s = 30.0 - opts.chunk_overlap_seconds
    for ci, part in enumerate(parts):
        feats = fe.log_mel_spectrogram(part.to(m.device), m.cfg.num_mel_bins, 3000)[None]
        enc = encode(m, feats)
        prompt = rules.prompt(with_timestamps)
        cand = decode_with_fallback(m, enc, prompt, rules, opts, with_timestamps, generator)
        if cand.is_no_speech(opts):
            continue
        text_tokens = [t for t in cand.tokens if rules.timestamp_begin is None or t < rules.timestamp_begin]
        acc = append_with_token_stitch(acc, text_tokens)
        segs.append((ci * step_s, min(ci * step_s + 30.0, wave.numel() / fe.SAMPLE_RATE), text_tokens))
        if opts.condition_on_previous_text and not (opts.reset_context_on_fallback and cand.temperature > 0.5):
            context = (context + text_tokens)[-max_ctx:]
        else:
            context = []
    return WhisperTranscription(bundle.decode_text(acc), acc, segs)


def transcribe_wav(bundle: WhisperBundle, path: str, opts: Optional[WhisperDecodeOptions] = None, **kw) -> WhisperTranscription:
    wave, rate = fe.load_mono_pcm16_wav(path)
    return transcribe_waveform_16k(bundle, fe.resample_linear(wave, rate, fe.SAMPLE_RATE), opts, **kw)


def load_from_pretrained_dir(model_dir: str, device="cpu", dtype=torch.float32) -> WhisperBundle:
    """Model plus token rules resolved from ``tokenizer.json`` (added tokens ``<|startoftranscript|>`` etc.)."""
    from ..tokenizer.hf import HFTokenizer
    m = load_sharded(model_dir, device=device, dtype=dtype)
    tok = HFTokenizer.from_file(model_dir)
    tid = tok.token_id
    cfg = m.cfg
    rules = DecodeTokenRules(tid("<|startoftranscript|>") or cfg.decoder_start_token_id, tid("<|endoftext|>") or cfg.eos_token_id,
                             tid("<|transcribe|>"), tid("<|translate|>"), tid("<|notimestamps|>"), tid("<|0.00|>"),
                             tid("<|nospeech|>") or tid("<|nocaptions|>"), tid("<|en|>"), tuple(cfg.suppress_tokens), tuple(cfg.begin_suppress_tokens))
    return WhisperBundle(m, rules, lambda ids: tok.decode(ids, skip_special=True))
