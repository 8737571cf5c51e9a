"""Silero VAD (tiny): STFT-as-convolution front end, four 1-D convolutions, one LSTM cell, sigmoid speech probability
per 512-sample chunk at 16 kHz; stateful streaming runtime, speech-timestamp segmentation, iterator
(Tyr/Model/SileroVAD/{Model,Utils}.lean)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..io import safetensors as st

SAMPLE_RATE, CHUNK, CONTEXT, RIGHT_PAD = 16000, 512, 64, 64
COMBINED, PREPARED = CHUNK + CONTEXT, CHUNK + CONTEXT + RIGHT_PAD

SHAPES = {"stft_conv.weight": (258, 1, 256), "conv1.weight": (128, 129, 3), "conv1.bias": (128,), "conv2.weight": (64, 128, 3),
          "conv2.bias": (64,), "conv3.weight": (64, 64, 3), "conv3.bias": (64,), "conv4.weight": (128, 64, 3), "conv4.bias": (128,),
          "lstm_cell.weight_ih": (512, 128), "lstm_cell.weight_hh": (512, 128), "lstm_cell.bias_ih": (512,), "lstm_cell.bias_hh": (512,),
          "final_conv.weight": (1, 128, 1), "final_conv.bias": (1,)}


def reflect_pad_right(x: torch.Tensor, pad: int) -> torch.Tensor:
    """``F.pad(x, (0, pad), mode="reflect")`` for a 1-D signal, defined for every length."""
    n = x.numel()
    if pad == 0:
        return x
    if n == 0:
        return torch.zeros(pad, dtype=x.dtype)
    if n == 1:
        return torch.cat([x, x.expand(pad)])
    idx = []
    for k in range(pad):
        i = n + k
        while i < 0 or i >= n:
            i = -i if i < 0 else 2 * n - 2 - i
        idx.append(i)
    return torch.cat([x, x[idx]])


@dataclass
class LstmState:
    h: torch.Tensor
    c: torch.Tensor

    @staticmethod
    def zero(device="cpu") -> "LstmState":
        return LstmState(torch.zeros(1, 128, device=device), torch.zeros(1, 128, device=device))


@dataclass
class SileroVAD:
    w: Dict[str, torch.Tensor]

    @staticmethod
    def init(device="cpu", seed=0) -> "SileroVAD":
        g = torch.Generator().manual_seed(seed)
        w = {}
        for n, s in SHAPES.items():
            fan = 1
            for d in s[1:]:
                fan *= d
            w[n] = ((torch.randn(s, generator=g) * fan ** -0.5) if n.endswith("weight") or "weight_" in n else torch.zeros(s)).to(device)
        return SileroVAD(w)

    @staticmethod
    def load(path: str, device="cpu") -> "SileroVAD":
        src = st.Source.open(path)
        w = {}
        for n, s in SHAPES.items():
            try:
                t = src.load(n)
            except Exception as e:
                raise IOError(f"SileroVAD tensor '{n}': {e}")
            if tuple(t.shape) != s:
                raise IOError(f"SileroVAD tensor '{n}': expected shape {list(s)}, got {list(t.shape)}")
            w[n] = t.float().to(device).requires_grad_(False)
        return SileroVAD(w)

    def lstm_cell(self, x, s: LstmState) -> LstmState:
        w = self.w
        gates = F.linear(x, w["lstm_cell.weight_ih"], w["lstm_cell.bias_ih"]) + F.linear(s.h, w["lstm_cell.weight_hh"], w["lstm_cell.bias_hh"])
        i, f, g, o = gates.chunk(4, dim=1)
        c = torch.sigmoid(f) * s.c + torch.sigmoid(i) * torch.tanh(g)
        return LstmState(torch.sigmoid(o) * torch.tanh(c), c)

    @torch.no_grad()
    def forward_prepared(self, x_prepared: torch.Tensor, state: LstmState) -> Tuple[torch.Tensor, LstmState]:
        """x_prepared [1, 640] = 64 context + 512 chunk + 64 reflect pad -> (probability [1, 1], new state)."""
        w = self.w
        if tuple(x_prepared.shape) != (1, PREPARED):
            raise ValueError(f"SileroVAD prepared input size mismatch: expected {PREPARED}, got {x_prepared.shape[-1]}")
        stft = F.conv1d(x_prepared.reshape(1, 1, PREPARED), w["stft_conv.weight"], stride=128)          # [1, 258, 4]
        mag = torch.sqrt(stft[:, :129] ** 2 + stft[:, 129:] ** 2)
        h = F.relu(F.conv1d(mag, w["conv1.weight"], w["conv1.bias"], stride=1, padding=1))
        h = F.relu(F.conv1d(h, w["conv2.weight"], w["conv2.bias"], stride=2, padding=1))
        h = F.relu(F.conv1d(h, w["conv3.weight"], w["conv3.bias"], stride=2, padding=1))
        h = F.relu(F.conv1d(h, w["conv4.weight"], w["conv4.bias"], stride=1, padding=1))
        s2 = self.lstm_cell(h.reshape(1, 128), state)
        y = torch.sigmoid(F.conv1d(F.relu(s2.h).reshape(1, 128, 1), w["final_conv.weight"], w["final_conv.bias"]))
        return y.reshape(1, 1), s2


class SileroVADRuntime:
    """Keeps the LSTM state and the 64-sample context between chunks."""

    def __init__(self, model: SileroVAD):
        self.model = model
        self.device = model.w["conv1.bias"].device
        self.reset()

    def reset(self):
        self.state = LstmState.zero(self.device)
        self.context = torch.zeros(CONTEXT)

    def step_chunk(self, chunk: torch.Tensor) -> float:
        if chunk.numel() != CHUNK:
            raise ValueError(f"SileroVAD chunk size mismatch: expected {CHUNK}, got {chunk.numel()}")
        combined = torch.cat([self.context, chunk.float().cpu()])
        x = reflect_pad_right(combined, RIGHT_PAD).reshape(1, PREPARED).to(self.device)
        y, self.state = self.model.forward_prepared(x, self.state)
        self.context = combined[-CONTEXT:]
        return float(y)

    def probabilities(self, wave: torch.Tensor) -> List[float]:
        """Per-chunk speech probabilities of a whole waveform (the last chunk is zero padded)."""
        self.reset()
        out = []
        for i in range(0, wave.numel(), CHUNK):
            c = wave[i:i + CHUNK]
            out.append(self.step_chunk(F.pad(c, (0, CHUNK - c.numel()))))
        return out


@dataclass
class SpeechTimestamp:
    start: int
    end: int


@dataclass
class TimestampConfig:
    threshold: float = 0.5
    sampling_rate: int = 16000
    min_speech_duration_ms: int = 250
    max_speech_duration_s: float = 1.0e9
    min_silence_duration_ms: int = 100
    speech_pad_ms: int = 30
    neg_threshold: Optional[float] = None
    min_silence_at_max_speech_ms: int = 98
    use_max_possible_silence_at_max_speech: bool = True


def timestamps_from_probabilities(probs: Sequence[float], audio_length_samples: int, cfg: Optional[TimestampConfig] = None) -> List[SpeechTimestamp]:
    """Silero ``get_speech_timestamps`` segmentation over chunk probabilities (hysteresis thresholds, minimum
    speech / silence, optional maximum speech length with a split at the longest recent silence, padding)."""
    cfg = cfg or TimestampConfig()
    if cfg.sampling_rate not in (8000, 16000):
        raise ValueError("SileroVAD supports 8000 and 16000 Hz")
    sr = cfg.sampling_rate
    win = 512 if sr == 16000 else 256
    ms = lambda v: sr * v // 1000
    min_speech, min_silence, pad = ms(cfg.min_speech_duration_ms), ms(cfg.min_silence_duration_ms), ms(cfg.speech_pad_ms)
    max_speech = sr * cfg.max_speech_duration_s - win - 2 * pad
    min_sil_at_max = ms(cfg.min_silence_at_max_speech_ms)
    neg = cfg.neg_threshold if cfg.neg_threshold is not None else max(cfg.threshold - 0.15, 0.01)
    triggered, speeches, cur = False, [], {}
    temp_end = prev_end = next_start = 0
    possible: List[Tuple[int, int]] = []
    for i, p in enumerate(probs):
        pos = win * i
        if p >= cfg.threshold and temp_end:
            sil = pos - temp_end
            if sil > min_sil_at_max:
                possible.append((temp_end, sil))
            temp_end = 0
            if next_start < prev_end:
                next_start = pos
        if p >= cfg.threshold and not triggered:
            triggered, cur = True, {"start": pos}
            continue
        if triggered and pos - cur["start"] > max_speech:
            if cfg.use_max_possible_silence_at_max_speech and possible:
                prev_end, dur = max(possible, key=lambda x: x[1])
                cur["end"] = prev_end
                speeches.append(cur)
                cur = {}
                next_start = prev_end + dur
                if next_start < prev_end + pos:
                    cur = {"start": next_start}
                else:
                    triggered = False
                prev_end = next_start = temp_end = 0
                possible = []
            elif prev_end:
                cur["end"] = prev_end
                speeches.append(cur)
                cur = {}
                if next_start < prev_end:
                    triggered = False
                else:
                    cur = {"start": next_start}
                prev_end = next_start = temp_end = 0
                possible = []
            else:
                cur["end"] = pos
                speeches.append(cur)
                cur, triggered = {}, False
                prev_end = next_start = temp_end = 0
                possible = []
                continue
        if p < neg and triggered:
            if not temp_end:
                temp_end = pos
            if pos - temp_end > min_sil_at_max:
                prev_end = temp_end
            if pos - temp_end < min_silence:
                continue
            cur["end"] = temp_end
            if cur["end"] - cur["start"] > min_speech:
                speeches.append(cur)
            cur, triggered = {}, False
            prev_end = next_start = temp_end = 0
            possible = []
    if cur and audio_length_samples - cur["start"] > min_speech:
        cur["end"] = audio_length_samples
        speeches.append(cur)
    for i, s in enumerate(speeches):
        if i == 0:
            s["start"] = max(0, s["start"] - pad)
        if i != len(speeches) - 1:
            gap = speeches[i + 1]["start"] - s["end"]
            if gap < 2 * pad:
                s["end"] += gap // 2
                speeches[i + 1]["start"] = max(0, speeches[i + 1]["start"] - gap // 2)
            else:
                s["end"] = min(audio_length_samples, s["end"] + pad)
                speeches[i + 1]["start"] = max(0, speeches[i + 1]["start"] - pad)
        else:
            s["end"] = min(audio_length_samples, s["end"] + pad)
    return [SpeechTimestamp(int(s["start"]), int(s["end"])) for s in speeches]


def timestamps_to_seconds(tss: Sequence[SpeechTimestamp], sampling_rate: int = 16000, digits: int = 1) -> List[Tuple[float, float]]:
    r = lambda x: int(x * 10 ** digits + 0.5) / 10 ** digits
    return [(r(t.start / sampling_rate), r(t.end / sampling_rate)) for t in tss]


def get_speech_timestamps(rt: SileroVADRuntime, wave: torch.Tensor, cfg: Optional[TimestampConfig] = None) -> List[SpeechTimestamp]:
    return timestamps_from_probabilities(rt.probabilities(wave), wave.numel(), cfg)


def collect_chunks(tss: Sequence[SpeechTimestamp], wav: torch.Tensor) -> torch.Tensor:
    return torch.cat([wav[t.start:t.end] for t in tss]) if tss else wav[:0]


def drop_chunks(tss: Sequence[SpeechTimestamp], wav: torch.Tensor) -> torch.Tensor:
    out, cur = [], 0
    for t in tss:
        out.append(wav[cur:t.start])
        cur = t.end
    out.append(wav[cur:])
    return torch.cat(out)


def read_audio(path: str, sampling_rate: int = 16000) -> torch.Tensor:
    from ..audio import frontend as fe
    w, r = fe.load_mono_pcm16_wav(path)
    return fe.resample_linear(w, r, sampling_rate)


@dataclass
class VADBoundary:
    kind: str          # "start" | "end"
    sample: int


class VADIterator:
    """Streaming boundaries: emits ``start`` when speech begins and ``end`` after ``min_silence`` of non-speech."""

    def __init__(self, runtime: SileroVADRuntime, threshold: float = 0.5, sampling_rate: int = 16000, min_silence_duration_ms: int = 100,
                 speech_pad_ms: int = 30):
        if sampling_rate != 16000:
            raise ValueError("VADIterator runs at 16 kHz")
        self.rt, self.threshold = runtime, threshold
        self.min_silence = sampling_rate * min_silence_duration_ms // 1000
        self.pad = sampling_rate * speech_pad_ms // 1000
        self.reset()

    def reset(self):
        self.rt.reset()
        self.triggered, self.temp_end, self.current_sample = False, 0, 0

    def step(self, chunk: torch.Tensor) -> Optional[VADBoundary]:
        self.current_sample += chunk.numel()
        p = self.rt.step_chunk(chunk)
        if p >= self.threshold and self.temp_end:
            self.temp_end = 0
        if p >= self.threshold and not self.triggered:
            self.triggered = True
            return VADBoundary("start", max(0, self.current_sample - self.pad - chunk.numel()))
        if p < self.threshold - 0.15 and self.triggered:
            if not self.temp_end:
                self.temp_end = self.current_sample
            if self.current_sample - self.temp_end < self.min_silence:
                return None
            end = self.temp_end + self.pad - chunk.numel()
            self.temp_end, self.triggered = 0, False
            return VADBoundary("end", end)
        return None
