"""Audio front ends shared by Whisper, Qwen3-ASR and Silero VAD: PCM16 WAV reading, resampling,
Whisper-style log-mel spectrograms (Tyr/Model/Qwen3ASR/Frontend.lean, Tyr/Model/Whisper/Transcribe.lean)."""
from __future__ import annotations

import math
import struct
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

SAMPLE_RATE = 16000
N_FFT = 400
HOP = 160


def load_mono_pcm16_wav(path: str) -> Tuple[torch.Tensor, int]:
    """Returns (float32 samples in [-1, 1], sample rate); multi-channel files are averaged."""
    with open(path, "rb") as f:
        data = f.read()
    if data[:4] != b"RIFF" or data[8:12] != b"WAVE":
        raise ValueError(f"{path}: not a RIFF/WAVE file")
    pos, fmt, pcm = 12, None, None
    while pos + 8 <= len(data):
        cid, size = data[pos:pos + 4], struct.unpack("<I", data[pos + 4:pos + 8])[0]
        body = data[pos + 8:pos + 8 + size]
        if cid == b"fmt ":
            fmt = struct.unpack("<HHIIHH", body[:16])
        elif cid == b"data":
            pcm = body
        pos += 8 + size + (size & 1)
    if fmt is None or pcm is None:
        raise ValueError(f"{path}: missing fmt or data chunk")
    tag, channels, rate, _, _, bits = fmt
    if tag != 1 or bits != 16:
        raise ValueError(f"{path}: only 16-bit PCM is supported (format {tag}, {bits} bits)")
    x = torch.frombuffer(bytearray(pcm[:len(pcm) // 2 * 2]), dtype=torch.int16).float() / 32768.0
    if channels > 1:
        x = x[:x.numel() // channels * channels].reshape(-1, channels).mean(1)
    return x, rate


def resample_linear(x: torch.Tensor, src_rate: int, dst_rate: int) -> torch.Tensor:
    if src_rate == dst_rate or x.numel() == 0:
        return x
    n = int(round(x.numel() * dst_rate / src_rate))
    return torch.nn.functional.interpolate(x[None, None], size=n, mode="linear", align_corners=False)[0, 0]


def hz_to_mel(f):
    """Slaney scale (linear below 1 kHz, logarithmic above), as used by Whisper's filter bank."""
    f = torch.as_tensor(f, dtype=torch.float64)
    lin = f / (200.0 / 3)
    log = 15.0 + torch.log(f.clamp_min(1e-9) / 1000.0) / (math.log(6.4) / 27.0)
    return torch.where(f >= 1000.0, log, lin)


def mel_to_hz(m):
    m = torch.as_tensor(m, dtype=torch.float64)
    lin = m * (200.0 / 3)
    log = 1000.0 * torch.exp((math.log(6.4) / 27.0) * (m - 15.0))
    return torch.where(m >= 15.0, log, lin)


def mel_filter_bank(n_mels: int = 80, n_fft: int = N_FFT, sample_rate: int = SAMPLE_RATE) -> torch.Tensor:
    """[n_mels, n_fft/2 + 1] triangular filters with Slaney area normalisation."""
    n_freq = n_fft // 2 + 1
    freqs = torch.linspace(0, sample_rate / 2, n_freq, dtype=torch.float64)
    pts = mel_to_hz(torch.linspace(float(hz_to_mel(0.0)), float(hz_to_mel(sample_rate / 2)), n_mels + 2, dtype=torch.float64))
    fb = torch.zeros(n_mels, n_freq, dtype=torch.float64)
    for i in range(n_mels):
        lo, c, hi = pts[i], pts[i + 1], pts[i + 2]
        up, down = (freqs - lo) / (c - lo), (hi - freqs) / (hi - c)
        fb[i] = torch.clamp(torch.minimum(up, down), min=0.0) * (2.0 / (hi - lo))
    return fb.float()


def log_mel_spectrogram(wave: torch.Tensor, n_mels: int = 80, n_frames: Optional[int] = 3000) -> torch.Tensor:
    """Whisper features [n_mels, frames]: Hann STFT (400 / 160), power, mel, log10 clamp to max-8, (x + 4) / 4.
    ``n_frames`` pads or trims the waveform to ``n_frames * 160`` samples first (30 s = 3000 frames)."""
    if n_frames is not None:
        need = n_frames * HOP
        wave = torch.nn.functional.pad(wave, (0, max(0, need - wave.numel())))[:need]
    win = torch.hann_window(N_FFT, periodic=True, device=wave.device)
    spec = torch.stft(wave.float(), N_FFT, HOP, window=win, center=True, pad_mode="reflect", return_complex=True)
    power = spec[:, :-1].abs() ** 2
    mel = mel_filter_bank(n_mels).to(wave.device) @ power
    log = torch.log10(mel.clamp_min(1e-10))
    log = torch.maximum(log, log.max() - 8.0)
    return (log + 4.0) / 4.0


@dataclass
class FrontendOutput:
    """Features ``[mels, frames]`` plus the number of frames that carry real audio."""
    input_features: torch.Tensor
    feature_length: int


def whisper_frontend(wave: torch.Tensor, sample_rate: int = SAMPLE_RATE, n_mels: int = 80, pad_to_30s: bool = True) -> FrontendOutput:
    wave = resample_linear(wave, sample_rate, SAMPLE_RATE)
    frames = (wave.numel() + HOP - 1) // HOP
    feats = log_mel_spectrogram(wave, n_mels, 3000 if pad_to_30s else max(1, frames))
    return FrontendOutput(feats, min(frames, feats.shape[1]))
