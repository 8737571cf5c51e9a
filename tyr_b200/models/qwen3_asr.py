"""Qwen3-ASR: windowed audio transformer over a strided-conv front end, its features spliced into a Qwen3 decoder at the
audio placeholder tokens; greedy transcription with a reusable prompt cache, forced alignment (timestamp classification
head, monotonic repair), chunked long-form transcription and a streaming state machine.

Contract: Tyr/Model/Qwen3ASR/{Config,AudioEncoder,Model,Processor,ForcedAligner,Transcribe,Streaming}.lean.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..audio import frontend as fe
from ..io import safetensors as st
from ..text.streaming_consensus import ConsensusConfig, ConsensusState
from . import qwen as Q
from .common import lin

DEFAULT_LANGUAGES = ("Chinese", "English", "Cantonese", "Arabic", "German", "French", "Spanish", "Portuguese", "Indonesian", "Italian", "Korean", "Russian",
                     "Thai", "Vietnamese", "Japanese", "Turkish", "Hindi", "Malay", "Dutch", "Swedish", "Danish", "Finnish", "Polish", "Czech", "Filipino",
                     "Persian", "Greek", "Romanian", "Hungarian", "Macedonian")
DEFAULT_EOS = (151645, 151643)


# ---- configuration ---------------------------------------------------------------------------------------------------------
def downsample_once(n: int) -> int:
    return 0 if n == 0 else (n - 1) // 2 + 1


def feat_extract_output_length(n: int) -> int:
    """Audio tokens produced for ``n`` mel frames: 13 per full 100-frame block plus the thrice-halved remainder."""
    leave = n % 100
    feat = 0 if leave == 0 else (leave - 1) // 2 + 1
    out_leave = 0 if feat == 0 else (((feat - 1) // 2 + 1 - 1) // 2) + 1
    return out_leave + (n // 100) * 13


@dataclass
class AudioEncoderConfig:
    num_mel_bins: int = 128
    encoder_layers: int = 32
    encoder_attention_heads: int = 20
    encoder_ffn_dim: int = 5120
    d_model: int = 1280
    activation_function: str = "gelu"
    n_window: int = 100
    output_dim: int = 4096
    n_window_infer: int = 400
    downsample_hidden_size: int = 480

    def __post_init__(self):
        e = lambda m: ValueError(f"Invalid Qwen3-ASR audio config: {m}")
        if self.num_mel_bins <= 0:
            raise e("num_mel_bins must be positive")
        if self.encoder_attention_heads <= 0 or self.d_model % self.encoder_attention_heads or self.d_model % 2:
            raise e("d_model must be even and split into equal heads")
        if self.n_window <= 0 or self.n_window_infer <= 0 or self.n_window_infer % (2 * self.n_window):
            raise e("n_window_infer must be a whole number of 2*n_window chunks")
        if self.activation_function not in ("gelu", "relu", "silu"):
            raise e("activation must be gelu, relu or silu")

    @property
    def head_dim(self): return self.d_model // self.encoder_attention_heads
    @property
    def mel_after_conv3(self): return downsample_once(downsample_once(downsample_once(self.num_mel_bins)))
    @property
    def conv_out_in_dim(self): return self.downsample_hidden_size * self.mel_after_conv3


@dataclass
class ThinkerConfig:
    audio: AudioEncoderConfig = field(default_factory=AudioEncoderConfig)
    text: Q.QwenConfig = field(default_factory=lambda: Q.QwenConfig(vocab_size=151936, hidden_size=4096, intermediate_size=22016, num_hidden_layers=32,
                                                                     num_attention_heads=32, num_key_value_heads=32, half_head_dim=64, rope_theta=5000000.0))
    audio_token_id: int = 151646
    model_type: str = "qwen3_asr_thinker"
    classify_num: int = 0

    def __post_init__(self):
        if self.audio.output_dim != self.text.hidden_size:
            raise ValueError("Invalid Qwen3-ASR config: audio features must have the text hidden size")
        if self.audio_token_id >= self.text.vocab_size:
            raise ValueError("Invalid Qwen3-ASR config: the audio placeholder must be a text token")
        if self.is_forced_aligner and self.classify_num <= 0:
            raise ValueError("Invalid Qwen3-ASR config: a forced aligner needs classify_num > 0")

    @property
    def is_forced_aligner(self): return "forced_aligner" in self.model_type
    @property
    def lm_head_out_dim(self): return self.classify_num if self.is_forced_aligner else self.text.vocab_size


@dataclass
class Qwen3ASRConfig:
    thinker: ThinkerConfig = field(default_factory=ThinkerConfig)
    support_languages: Tuple[str, ...] = DEFAULT_LANGUAGES
    timestamp_token_id: int = 0
    timestamp_segment_time: float = 1.0

    def __post_init__(self):
        if self.timestamp_token_id >= self.thinker.text.vocab_size or not self.timestamp_segment_time > 0:
            raise ValueError("Invalid Qwen3-ASR config: timestamp token / segment time")

    @staticmethod
    def from_json(j: dict) -> "Qwen3ASRConfig":
        tj = j.get("thinker_config", j)
        aj, xj = tj.get("audio_config", {}), tj.get("text_config", {})
        d = AudioEncoderConfig()
        g = lambda k: aj.get(k, getattr(d, k))
        audio = AudioEncoderConfig(g("num_mel_bins"), g("encoder_layers"), g("encoder_attention_heads"), g("encoder_ffn_dim"), g("d_model"),
                                   g("activation_function"), g("n_window"), g("output_dim"), g("n_window_infer"), g("downsample_hidden_size"))
        text = Q.QwenConfig.from_json(xj, ThinkerConfig().text)
        th = ThinkerConfig(audio, text, tj.get("audio_token_id", 151646), tj.get("model_type", "qwen3_asr_thinker"), tj.get("classify_num", 0))
        return Qwen3ASRConfig(th, tuple(j.get("support_languages") or DEFAULT_LANGUAGES), j.get("timestamp_token_id", 0), float(j.get("timestamp_segment_time", 1.0)))


# ---- audio encoder ----------------------------------------------------------------------------------------------------------
@dataclass
class AudioLayer:
    q_w: torch.Tensor; q_b: torch.Tensor; k_w: torch.Tensor; k_b: torch.Tensor; v_w: torch.Tensor; v_b: torch.Tensor
    o_w: torch.Tensor; o_b: torch.Tensor
    ln1_w: torch.Tensor; ln1_b: torch.Tensor; fc1_w: torch.Tensor; fc1_b: torch.Tensor; fc2_w: torch.Tensor; fc2_b: torch.Tensor
    ln2_w: torch.Tensor; ln2_b: torch.Tensor


@dataclass
class AudioEncoder:
    cfg: AudioEncoderConfig
    conv_w: List[torch.Tensor]
    conv_b: List[torch.Tensor]
    conv_out: torch.Tensor
    layers: List[AudioLayer]
    ln_post_w: torch.Tensor
    ln_post_b: torch.Tensor
    proj1_w: torch.Tensor; proj1_b: torch.Tensor; proj2_w: torch.Tensor; proj2_b: torch.Tensor


def _act(name):
    return {"gelu": F.gelu, "relu": F.relu, "silu": F.silu}[name]


def sinusoid_position(seq: int, dim: int, device) -> torch.Tensor:
    half = dim // 2
    inc = math.log(10000.0) / max(1, half - 1)
    t = torch.arange(seq, dtype=torch.float32, device=device)[:, None] * torch.exp(-inc * torch.arange(half, dtype=torch.float32, device=device))[None]
    return torch.cat([torch.sin(t), torch.cos(t)], 1)


def build_chunk_lengths(cfg: AudioEncoderConfig, feature_lens: Sequence[int]) -> List[int]:
    step, out = 2 * cfg.n_window, []
    for n in feature_lens:
        if n == 0:
            continue
        chunks = (n + step - 1) // step
        out += [step] * (chunks - 1) + [n % step or step]
    return out


def audio_token_count(cfg: AudioEncoderConfig, frames: int) -> int:
    """Tokens the encoder emits for ``frames`` mel frames: the per-chunk counts summed.  With chunks that are multiples of
    100 frames (every released model) this equals ``feat_extract_output_length(frames)``."""
    return sum(feat_extract_output_length(c) for c in build_chunk_lengths(cfg, [frames]))


def attention_window_lengths(cfg: AudioEncoderConfig, total_after_cnn: int, chunk_after_cnn: int) -> List[int]:
    """Attention runs inside windows of ``chunk_after_cnn * n_window_infer / (2 n_window)`` audio tokens."""
    win = max(1, chunk_after_cnn * (cfg.n_window_infer // (2 * cfg.n_window)))
    return [win] * (total_after_cnn // win) + ([total_after_cnn % win] if total_after_cnn % win else [])


def _audio_layer(cfg, l: AudioLayer, x):
    B, S, C = x.shape
    H, D = cfg.encoder_attention_heads, cfg.head_dim
    h = F.layer_norm(x, (C,), l.ln1_w, l.ln1_b, 1e-5)
    q, k, v = (F.linear(h, w, b).reshape(B, S, H, D).transpose(1, 2) for w, b in ((l.q_w, l.q_b), (l.k_w, l.k_b), (l.v_w, l.v_b)))
    a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, S, C)
    x = x + F.linear(a, l.o_w, l.o_b)
    h = F.layer_norm(x, (C,), l.ln2_w, l.ln2_b, 1e-5)
    return x + F.linear(_act(cfg.activation_function)(F.linear(h, l.fc1_w, l.fc1_b)), l.fc2_w, l.fc2_b)


def _conv_stack(m: AudioEncoder, chunks: torch.Tensor) -> torch.Tensor:
    """[N, mel, T] -> [N, T/8, d_model]: three 3x3 stride-2 convolutions with GELU, then a linear over (channel, mel)."""
    x = chunks.unsqueeze(1)
    for w, b in zip(m.conv_w, m.conv_b):
        x = F.gelu(F.conv2d(x, w, b, stride=2, padding=1))
    N, Cc, Mm, T = x.shape
    return F.linear(x.permute(0, 3, 1, 2).reshape(N, T, Cc * Mm), m.conv_out)


@torch.no_grad()
def encode_audio(m: AudioEncoder, features: torch.Tensor, feature_lens: Optional[Sequence[int]] = None) -> List[torch.Tensor]:
    """features: [B, mel, frames] log-mel.  Returns per sample ``[audio_tokens, output_dim]`` where the token count is
    ``feat_extract_output_length(feature_len)``.  Each sample is cut into chunks of ``2 n_window`` frames that pass the
    convolutions independently (all chunks of the batch in one padded call), positions restart per chunk, and attention
    is confined to windows of several chunks (AudioEncoder.lean:231-470)."""
    cfg = m.cfg
    B, _, frames = features.shape
    lens = [min(int(n), frames) for n in (feature_lens if feature_lens is not None else [frames] * B)]
    features = features.to(m.conv_out.dtype)
    outs: List[torch.Tensor] = []
    for b in range(B):
        n = lens[b]
        if n == 0:
            outs.append(torch.zeros(0, cfg.output_dim, dtype=features.dtype, device=features.device))
            continue
        cl = build_chunk_lengths(cfg, [n])
        width = max(cl)
        padded = torch.zeros(len(cl), cfg.num_mel_bins, width, dtype=features.dtype, device=features.device)
        s = 0
        for i, c in enumerate(cl):
            padded[i, :, :c] = features[b, :, s:s + c]
            s += c
        emb = _conv_stack(m, padded)                                                      # [chunks, t_chunk, d_model]
        emb = emb + sinusoid_position(emb.shape[1], cfg.d_model, emb.device).to(emb.dtype)[None]
        after = [feat_extract_output_length(c) for c in cl]
        # a chunk owes ``feat_extract_output_length(frames)`` tokens; where the convolutions yield fewer the tail is zero rows
        hidden = torch.cat([F.pad(emb[i, :min(a, emb.shape[1])], (0, 0, 0, max(0, a - emb.shape[1]))) for i, a in enumerate(after)], 0).unsqueeze(0)
        total = hidden.shape[1]
        parts, s = [], 0
        for wlen in attention_window_lengths(cfg, total, max(max(after), 1)):
            seg = hidden[:, s:s + wlen]
            for l in m.layers:
                seg = _audio_layer(cfg, l, seg)
            parts.append(seg)
            s += wlen
        h = F.layer_norm(torch.cat(parts, 1), (cfg.d_model,), m.ln_post_w, m.ln_post_b, 1e-5)
        h = F.linear(_act(cfg.activation_function)(F.linear(h, m.proj1_w, m.proj1_b)), m.proj2_w, m.proj2_b)
        outs.append(h[0])
    return outs


def init_audio_encoder(cfg: AudioEncoderConfig, device="cpu", dtype=torch.float32, seed=0) -> AudioEncoder:
    g = torch.Generator().manual_seed(seed)
    w = lambda *s, fan=None: (torch.randn(*s, generator=g) * (fan or s[-1]) ** -0.5).to(device=device, dtype=dtype)
    z = lambda n: torch.zeros(n, device=device, dtype=dtype)
    o = lambda n: torch.ones(n, device=device, dtype=dtype)
    C, Fd, Hd = cfg.d_model, cfg.encoder_ffn_dim, cfg.downsample_hidden_size
    layers = [AudioLayer(w(C, C), z(C), w(C, C), z(C), w(C, C), z(C), w(C, C), z(C), o(C), z(C), w(Fd, C), z(Fd), w(C, Fd), z(C), o(C), z(C))
              for _ in range(cfg.encoder_layers)]
    return AudioEncoder(cfg, [w(Hd, 1, 3, 3, fan=9), w(Hd, Hd, 3, 3, fan=9 * Hd), w(Hd, Hd, 3, 3, fan=9 * Hd)], [z(Hd), z(Hd), z(Hd)],
                        w(C, cfg.conv_out_in_dim), layers, o(C), z(C), w(C, C), z(C), w(cfg.output_dim, C), z(cfg.output_dim))


# ---- processor ------------------------------------------------------------------------------------------------------------------
@dataclass
class Processor:
    audio_token: str = "<|audio_pad|>"
    audio_bos_token: str = "<|audio_start|>"
    audio_eos_token: str = "<|audio_end|>"
    im_start: str = "<|im_start|>"
    im_end: str = "<|im_end|>"
    sampling_rate: int = 16000

    def apply_chat_template(self, system: str, user: str, add_generation_prompt: bool = True) -> str:
        blk = lambda role, c: f"{self.im_start}{role}\n{c}{self.im_end}\n"
        return blk("system", system) + blk("user", user) + (f"{self.im_start}assistant\n" if add_generation_prompt else "")

    def audio_user_placeholder(self) -> str:
        return self.audio_bos_token + self.audio_token + self.audio_eos_token

    def build_asr_prompt(self, context: str = "", force_language: Optional[str] = None) -> str:
        base = self.apply_chat_template(context, self.audio_user_placeholder(), True)
        return base + (f"language {force_language}<asr_text>" if force_language else "")

    def replace_multimodal_special_tokens(self, texts: Sequence[str], audio_lengths: Sequence[int]) -> List[str]:
        out, idx = [], 0
        for s in texts:
            parts = s.split(self.audio_token)
            if len(parts) - 1 > len(audio_lengths) - idx:
                raise ValueError(f"Not enough audio lengths while replacing `{self.audio_token}` placeholders")
            acc = parts[0]
            for p in parts[1:]:
                acc += self.audio_token * audio_lengths[idx] + p
                idx += 1
            out.append(acc)
        return out

    def encode_with_expanded_audio_token_ids(self, encode: Callable[[str], List[int]], text: str, audio_lengths: Sequence[int], audio_token_id: int) -> List[int]:
        """Text pieces are tokenised separately and joined by exact runs of the placeholder id, so that tokenizer merges
        cannot change the number of placeholders."""
        parts = text.split(self.audio_token)
        if len(parts) - 1 > len(audio_lengths):
            raise ValueError(f"Not enough audio lengths while encoding `{self.audio_token}` placeholders")
        out: List[int] = []
        for i, p in enumerate(parts):
            out += encode(p)
            if i + 1 < len(parts):
                out += [audio_token_id] * audio_lengths[i]
        return out

    @staticmethod
    def get_chunked_index(token_indices: Sequence[int], tokens_per_chunk: int) -> List[Tuple[int, int]]:
        if tokens_per_chunk == 0:
            return [(0, len(token_indices))]
        out, start, cur = [], 0, 1
        for i, t in enumerate(token_indices):
            if t >= cur * tokens_per_chunk:
                out.append((start, i))
                start, cur = i, cur + 1
        return out + [(start, len(token_indices))]


# ---- thinker --------------------------------------------------------------------------------------------------------------------
@dataclass
class Qwen3ASR:
    cfg: Qwen3ASRConfig
    audio_tower: AudioEncoder
    lm: Q.Qwen3ForCausalLM            # lm_head has ``classify_num`` rows for a forced aligner

    @property
    def device(self): return self.lm.model.embed_tokens.device

    def get_supported_languages(self): return list(self.cfg.support_languages)


def init(cfg: Qwen3ASRConfig, device="cpu", dtype=torch.float32, seed=0) -> Qwen3ASR:
    th = cfg.thinker
    lm = Q.Qwen3ForCausalLM.init(th.text, tie_word_embeddings=False, device=device, dtype=dtype, seed=seed)
    if th.is_forced_aligner:
        g = torch.Generator().manual_seed(seed + 1)
        lm.lm_head = (torch.randn(th.classify_num, th.text.hidden_size, generator=g) * th.text.hidden_size ** -0.5).to(device=device, dtype=dtype)
    return Qwen3ASR(cfg, init_audio_encoder(th.audio, device, dtype, seed + 2), lm)


def build_inputs_embeds(m: Qwen3ASR, input_ids: torch.Tensor, audio_feats: Sequence[torch.Tensor]) -> torch.Tensor:
    """Token embeddings with the placeholder positions of row b replaced, in order, by ``audio_feats[b]``."""
    emb = m.lm.embed_tokens(input_ids).clone()
    for b in range(input_ids.shape[0]):
        pos = torch.nonzero(input_ids[b] == m.cfg.thinker.audio_token_id).reshape(-1)
        if pos.numel() != audio_feats[b].shape[0]:
            raise ValueError(f"Qwen3-ASR: row {b} has {pos.numel()} audio placeholders for {audio_feats[b].shape[0]} audio features")
        emb[b, pos] = audio_feats[b].to(emb.dtype)
    return emb


@torch.no_grad()
def forward(m: Qwen3ASR, input_ids: torch.Tensor, features: Optional[torch.Tensor] = None, feature_lens=None) -> torch.Tensor:
    """Logits [B, S, lm_head_out_dim] (uncached; the forced aligner reads every position)."""
    if features is None:
        return m.lm.forward(input_ids)
    return m.lm.forward_embeds(build_inputs_embeds(m, input_ids, encode_audio(m.audio_tower, features.to(m.device), feature_lens)))


@dataclass
class PromptCache:
    """Decoder state after a prompt, reusable while later prompts extend it (streaming re-decodes the same audio prefix
    with more audio appended: the common prefix of the embedded prompt is not recomputed)."""
    ids: List[int]
    session: Q.Qwen3Session


@torch.no_grad()
def generate_greedy(m: Qwen3ASR, input_ids: torch.Tensor, features: torch.Tensor, feature_lens=None, max_new_tokens: int = 256,
                    eos_token_ids: Sequence[int] = DEFAULT_EOS) -> List[List[int]]:
    """Batch rows must have equal prompt length (bucket by length, Transcribe.lean:503-547).  Returns new tokens per row."""
    emb = build_inputs_embeds(m, input_ids, encode_audio(m.audio_tower, features.to(m.device), feature_lens))
    B, S = input_ids.shape
    sess = Q.Qwen3Session(m.lm, B, S + max_new_tokens)
    logits = sess.run_embeds(emb)
    done = torch.zeros(B, dtype=torch.bool, device=emb.device)
    eos = torch.tensor(list(eos_token_ids), device=emb.device)
    out: List[List[int]] = [[] for _ in range(B)]
    for _ in range(max_new_tokens):
        tok = logits.argmax(-1)
        done |= torch.isin(tok, eos)
        if bool(done.all()):
            break
        for b, t in enumerate(tok.tolist()):
            if not done[b]:
                out[b].append(t)
        logits = sess.step(tok)
    return out


# ---- forced alignment ----------------------------------------------------------------------------------------------------------------
@dataclass
class ForcedAlignItem:
    text: str
    start_time: float
    end_time: float


def _kept(ch: str) -> bool:
    return ch == "'" or ch.isalnum()


def _is_cjk(ch: str) -> bool:
    c = ord(ch)
    return (0x4E00 <= c <= 0x9FFF or 0x3400 <= c <= 0x4DBF or 0x20000 <= c <= 0x2A6DF or 0x2A700 <= c <= 0x2B73F or 0x2B740 <= c <= 0x2B81F
            or 0x2B820 <= c <= 0x2CEAF or 0xF900 <= c <= 0xFAFF)


def _is_japanese(ch: str) -> bool:
    c = ord(ch)
    return _is_cjk(ch) or 0x3040 <= c <= 0x30FF or 0x31F0 <= c <= 0x31FF or 0xFF66 <= c <= 0xFF9D


def _is_korean(ch: str) -> bool:
    c = ord(ch)
    return 0xAC00 <= c <= 0xD7AF or 0x1100 <= c <= 0x11FF or 0x3130 <= c <= 0x318F or 0xA960 <= c <= 0xA97F or 0xD7B0 <= c <= 0xD7FF


def tokenize_space_lang(text: str) -> List[str]:
    out = []
    for seg in text.split(" "):
        cleaned = "".join(c for c in seg if _kept(c))
        buf = ""
        for ch in cleaned:
            if _is_cjk(ch):
                if buf:
                    out.append(buf)
                    buf = ""
                out.append(ch)
            else:
                buf += ch
        if buf:
            out.append(buf)
    return out


def tokenize_script_mixed(text: str, is_script: Callable[[str], bool]) -> List[str]:
    out, buf = [], ""
    for ch in text:
        if is_script(ch):
            if buf:
                out.append(buf)
                buf = ""
            out.append(ch)
        elif _kept(ch):
            buf += ch
        elif buf:
            out.append(buf)
            buf = ""
    return out + ([buf] if buf else [])


def encode_timestamp_text(text: str, language: str) -> Tuple[List[str], str]:
    lang = language.strip().lower()
    words = tokenize_script_mixed(text, _is_japanese) if lang == "japanese" else tokenize_script_mixed(text, _is_korean) if lang == "korean" else tokenize_space_lang(text)
    body = "<timestamp><timestamp>".join(words) + "<timestamp><timestamp>" if words else "<timestamp><timestamp>"
    return words, "<|audio_start|><|audio_pad|><|audio_end|>" + body


def fix_timestamp(data: Sequence[int]) -> List[int]:
    """Keep a longest non-decreasing subsequence; short outlier runs snap to the nearer kept neighbour, longer runs are
    interpolated between their kept neighbours (ForcedAligner.lean:148-246)."""
    n = len(data)
    if n == 0:
        return []
    dp, parent = [1] * n, [-1] * n
    for i in range(1, n):
        for j in range(i):
            if data[j] <= data[i] and dp[j] + 1 > dp[i]:
                dp[i], parent[i] = dp[j] + 1, j
    idx = max(range(n), key=lambda i: (dp[i], -i))
    normal = [False] * n
    while idx != -1:
        normal[idx] = True
        idx = parent[idx]
    res = list(data)
    i = 0
    while i < n:
        if normal[i]:
            i += 1
            continue
        j = i
        while j < n and not normal[j]:
            j += 1
        left = next((res[k] for k in range(i - 1, -1, -1) if normal[k]), None)
        right = next((res[k] for k in range(j, n) if normal[k]), None)
        if j - i <= 2:
            for k in range(i, j):
                if left is not None and right is not None:
                    res[k] = left if k - (i - 1) <= j - k else right
                elif left is not None or right is not None:
                    res[k] = left if left is not None else right
        elif left is not None and right is not None:
            for k in range(i, j):
                res[k] = left + (right - left) * (k - i + 1) // (j - i + 1)
        elif left is not None or right is not None:
            for k in range(i, j):
                res[k] = left if left is not None else right
        i = j
    return res


def parse_timestamp(words: Sequence[str], timestamp_ms: Sequence[int]) -> List[ForcedAlignItem]:
    need = 2 * len(words)
    fixed = fix_timestamp(list(timestamp_ms)[:need])
    fixed += [fixed[-1] if fixed else 0] * (need - len(fixed))
    return [ForcedAlignItem(w, fixed[2 * i] / 1000.0, fixed[2 * i + 1] / 1000.0) for i, w in enumerate(words)]


def align_from_logits(cfg: Qwen3ASRConfig, input_ids: torch.Tensor, logits: torch.Tensor, word_lists: Sequence[Sequence[str]]) -> List[List[ForcedAlignItem]]:
    """The class predicted at every timestamp slot, times the bin width, is that slot's time in milliseconds."""
    pred = logits.argmax(-1)
    out = []
    for b, words in enumerate(word_lists):
        slots = input_ids[b] == cfg.timestamp_token_id
        ms = (pred[b][slots].double() * cfg.timestamp_segment_time).long().tolist()
        out.append(parse_timestamp(words, ms))
    return out


# ---- transcription ------------------------------------------------------------------------------------------------------------------
@dataclass
class ASRTranscription:
    language: str
    text: str
    time_stamps: Optional[List[ForcedAlignItem]] = None


MIN_INPUT_SECONDS, MAX_INPUT_SECONDS, MAX_ALIGN_SECONDS = 0.5, 1200.0, 180.0


def split_audio_into_chunks(wave: torch.Tensor, sample_rate: int, max_seconds: float, search_seconds: float = 5.0) -> List[Tuple[torch.Tensor, float]]:
    """Cut at the quietest 100 ms window within ``search_seconds`` of each boundary; returns (chunk, offset seconds)."""
    n, limit = wave.numel(), int(max_seconds * sample_rate)
    if n <= limit:
        return [(wave, 0.0)]
    out, start = [], 0
    win, search = max(1, sample_rate // 10), int(search_seconds * sample_rate)
    while n - start > limit:
        lo, hi = start + limit - search, start + limit
        energy = F.avg_pool1d(wave[lo:hi].abs()[None, None], win, 1)[0, 0]
        cut = lo + int(energy.argmin()) + win // 2
        out.append((wave[start:cut], start / sample_rate))
        start = cut
    return out + [(wave[start:], start / sample_rate)]


def parse_asr_output(text: str, forced_language: Optional[str] = None) -> Tuple[str, str]:
    """``language X<asr_text>...`` -> (language, text); with a forced language the model emits the text only."""
    if forced_language:
        return forced_language, text.strip()
    if "<asr_text>" in text:
        head, body = text.split("<asr_text>", 1)
        lang = head.replace("language", "").strip()
        return lang, body.strip()
    return "", text.strip()


def mel_features(wave: torch.Tensor, n_mels: int = 128) -> torch.Tensor:
    """[mel, frames] log-mel of a 16 kHz waveform without padding to 30 s."""
    return fe.log_mel_spectrogram(wave, n_mels=n_mels, n_frames=None)


@torch.no_grad()
def transcribe_waveform(m: Qwen3ASR, encode: Callable[[str], List[int]], decode: Callable[[List[int]], str], wave: torch.Tensor, sample_rate: int = 16000,
                        context: str = "", language: Optional[str] = None, max_new_tokens: int = 256, processor: Optional[Processor] = None,
                        aligner: Optional["Qwen3ASR"] = None) -> ASRTranscription:
    proc = processor or Processor()
    if language is not None:
        match = [l for l in m.cfg.support_languages if l.lower() == language.strip().lower()]
        if not match:
            raise ValueError(f"Unsupported language: {language}")
        language = match[0]
    if sample_rate != proc.sampling_rate:
        wave = fe.resample_linear(wave, sample_rate, proc.sampling_rate)
    if wave.numel() < MIN_INPUT_SECONDS * proc.sampling_rate:
        wave = F.pad(wave, (0, int(MIN_INPUT_SECONDS * proc.sampling_rate) - wave.numel()))
    texts, lang_out, stamps = [], "", []
    limit = MAX_ALIGN_SECONDS if aligner is not None else MAX_INPUT_SECONDS
    for chunk, offset in split_audio_into_chunks(wave, proc.sampling_rate, limit):
        feats = mel_features(chunk, m.cfg.thinker.audio.num_mel_bins)
        n_audio = audio_token_count(m.cfg.thinker.audio, feats.shape[1])
        ids = proc.encode_with_expanded_audio_token_ids(encode, proc.build_asr_prompt(context, language), [n_audio], m.cfg.thinker.audio_token_id)
        new = generate_greedy(m, torch.tensor([ids], device=m.device), feats[None], [feats.shape[1]], max_new_tokens)[0]
        lang, text = parse_asr_output(decode(new), language)
        lang_out = lang_out or lang
        texts.append(text)
        if aligner is not None and text:
            stamps += [ForcedAlignItem(i.text, i.start_time + offset, i.end_time + offset)
                       for i in align_waveform(aligner, encode, chunk, text, lang or "English", proc)]
    return ASRTranscription(lang_out, " ".join(t for t in texts if t), stamps if aligner is not None else None)


@torch.no_grad()
def align_waveform(aligner: Qwen3ASR, encode, wave: torch.Tensor, text: str, language: str, processor: Optional[Processor] = None) -> List[ForcedAlignItem]:
    proc = processor or Processor()
    words, prompt = encode_timestamp_text(text, language)
    feats = mel_features(wave, aligner.cfg.thinker.audio.num_mel_bins)
    ids = proc.encode_with_expanded_audio_token_ids(encode, prompt, [audio_token_count(aligner.cfg.thinker.audio, feats.shape[1])], aligner.cfg.thinker.audio_token_id)
    t = torch.tensor([ids], device=aligner.device)
    return align_from_logits(aligner.cfg, t, forward(aligner, t, feats[None], [feats.shape[1]]), [words])[0]


# ---- streaming ----------------------------------------------------------------------------------------------------------------------
class StreamingTranscriber:
    """Feed audio as it arrives; every ``chunk_seconds`` the whole buffered audio is re-decoded and the hypothesis passes
    through a stable-prefix consensus, so ``text`` only ever grows (Streaming.lean, Realtime.lean)."""

    def __init__(self, m: Qwen3ASR, encode, decode, chunk_seconds: float = 2.0, language: Optional[str] = None, context: str = "",
                 max_new_tokens: int = 128, confirm_windows: int = 2, rollback_tokens: int = 2):
        self.m, self.encode, self.decode = m, encode, decode
        self.language, self.context, self.max_new_tokens = language, context, max_new_tokens
        self.chunk = int(chunk_seconds * 16000)
        self.buffer = torch.zeros(0)
        self.pending = 0
        self.consensus = ConsensusState(ConsensusConfig(confirm_windows=confirm_windows, rollback_tokens=rollback_tokens))
        self._word_ids: Dict[str, int] = {}
        self._words: List[str] = []
        self.stable_text = ""
        self.unstable_text = ""
        self.decodes = 0

    @property
    def text(self) -> str:
        return self.stable_text

    def push(self, samples: torch.Tensor) -> str:
        self.buffer = torch.cat([self.buffer, samples.reshape(-1).float().cpu()])
        self.pending += samples.numel()
        while self.pending >= self.chunk:
            self.pending -= self.chunk
            self._decode(final=False)
        return self.text

    def finish(self) -> str:
        """Decodes what is buffered once more and commits the whole hypothesis."""
        if self.buffer.numel():
            self._decode(final=True)
        return self.text

    def _decode(self, final: bool):
        r = transcribe_waveform(self.m, self.encode, self.decode, self.buffer, 16000, self.context, self.language, self.max_new_tokens)
        self.decodes += 1
        ids = []
        for w in r.text.split():                                   # consensus over words: ids are assigned on first sight
            if w not in self._word_ids:
                self._word_ids[w] = len(self._words)
                self._words.append(w)
            ids.append(self._word_ids[w])
        join = lambda xs: " ".join(self._words[i] for i in xs)
        d = self.consensus.update_with_signals(ids, join, speech_active=not final, boundary=final)
        if d.stable_append:
            self.stable_text = (self.stable_text + " " + d.stable_append).strip()
        if final and self.consensus.unstable_ids:                  # the rollback margin no longer applies at the end
            self.stable_text = (self.stable_text + " " + join(self.consensus.unstable_ids)).strip()
            self.consensus.stable_ids += self.consensus.unstable_ids
            self.consensus.unstable_ids = []
        self.unstable_text = join(self.consensus.unstable_ids)


# ---- weights --------------------------------------------------------------------------------------------------------------------------
def load(cfg: Qwen3ASRConfig, source, device="cpu", dtype=torch.bfloat16) -> Qwen3ASR:
    """Checkpoint names: ``thinker.audio_tower.*``, ``thinker.model.*`` (Qwen3 decoder), ``thinker.lm_head.weight``."""
    src = source if isinstance(source, st.Source) else st.Source.open(source)
    a = cfg.thinker.audio
    g = lambda n: src.load("thinker.audio_tower." + n).to(device=device, dtype=dtype)
    layers = []
    for i in range(a.encoder_layers):
        p = f"layers.{i}."
        layers.append(AudioLayer(*(g(p + f"self_attn.{x}_proj.{y}") for x in ("q", "k", "v", "out") for y in ("weight", "bias")),
                                 g(p + "self_attn_layer_norm.weight"), g(p + "self_attn_layer_norm.bias"), g(p + "fc1.weight"), g(p + "fc1.bias"),
                                 g(p + "fc2.weight"), g(p + "fc2.bias"), g(p + "final_layer_norm.weight"), g(p + "final_layer_norm.bias")))
    tower = AudioEncoder(a, [g(f"conv2d{i}.weight") for i in (1, 2, 3)], [g(f"conv2d{i}.bias") for i in (1, 2, 3)], g("conv_out.weight"), layers,
                         g("ln_post.weight"), g("ln_post.bias"), g("proj1.weight"), g("proj1.bias"), g("proj2.weight"), g("proj2.bias"))
    lm = Q.load_qwen3_causal_lm(cfg.thinker.text, src, device, dtype, name_map=lambda n: "thinker." + n)
    return Qwen3ASR(cfg, tower, lm)


def state_dict(m: Qwen3ASR) -> Dict[str, torch.Tensor]:
    out = {"thinker." + k: v for k, v in Q.state_dict(m.lm).items()}
    t = m.audio_tower
    P = "thinker.audio_tower."
    for i in (1, 2, 3):
        out[f"{P}conv2d{i}.weight"], out[f"{P}conv2d{i}.bias"] = t.conv_w[i - 1], t.conv_b[i - 1]
    out[P + "conv_out.weight"] = t.conv_out
    for n in ("ln_post_w", "ln_post_b", "proj1_w", "proj1_b", "proj2_w", "proj2_b"):
        base, kind = n.rsplit("_", 1)
        out[f"{P}{base}.{'weight' if kind == 'w' else 'bias'}"] = getattr(t, n)
    for i, l in enumerate(t.layers):
        p = f"{P}layers.{i}."
        for x, nm in (("q", "q"), ("k", "k"), ("v", "v"), ("o", "out")):
            out[p + f"self_attn.{nm}_proj.weight"], out[p + f"self_attn.{nm}_proj.bias"] = getattr(l, x + "_w"), getattr(l, x + "_b")
        out[p + "self_attn_layer_norm.weight"], out[p + "self_attn_layer_norm.bias"] = l.ln1_w, l.ln1_b
        out[p + "fc1.weight"], out[p + "fc1.bias"], out[p + "fc2.weight"], out[p + "fc2.bias"] = l.fc1_w, l.fc1_b, l.fc2_w, l.fc2_b
        out[p + "final_layer_norm.weight"], out[p + "final_layer_norm.bias"] = l.ln2_w, l.ln2_b
    return out
