"""File-level glue around the Qwen3-TTS speech tokenizer: audio file -> codec id rows, codec id rows -> wav, reference audio ->
speaker mel / speaker embedding.  Everything runs in-process on the encoders and decoder of this package (the reference still
shells out to a Python script for decoding; encoding and the speaker mel are native there as well).

Contract: Tyr/Model/Qwen3TTS/SpeechTokenizerBridge.lean (speaker mel :178-228, code rows :236-245, decode :247-275,
encode :278-341, speaker embedding :345-392).
"""
from __future__ import annotations

import os
from typing import List, Optional, Tuple

import torch

from ..audio import frontend as FE
from ..io import media
from ..io import safetensors as st
from . import qwen3_tts as T
from . import qwen3_tts_encoder as E


def resolve_speech_tokenizer_dir(model_dir: str, speech_tokenizer_dir: Optional[str] = None) -> str:
    return os.path.expanduser(speech_tokenizer_dir) if speech_tokenizer_dir else os.path.join(model_dir, "speech_tokenizer")


def is_tokenizer_25hz(speech_tokenizer_dir: str) -> bool:
    with open(os.path.join(speech_tokenizer_dir, "config.json"), encoding="utf-8") as f:
        return '"qwen3_tts_tokenizer_25hz"' in f.read()


def load_resampled_mono_wav(path: str, target_rate: int) -> torch.Tensor:
    wave, rate = FE.load_mono_pcm16_wav(os.path.expanduser(path))
    return wave if rate == target_rate else FE.resample_linear(wave, rate, target_rate)


def slaney_mel_filter_bank(freq_bins: int, n_mels: int, sample_rate: int, fmin: float, fmax: float) -> torch.Tensor:
    """[freq_bins, n_mels] triangles on the Slaney mel scale between fmin and min(fmax, Nyquist), area-normalised."""
    if freq_bins < 2 or n_mels == 0:
        return torch.zeros(freq_bins, n_mels)
    nyq = float(sample_rate // 2)
    lo = max(0.0, fmin)
    hi = min(nyq, max(lo, fmax))
    pts = FE.mel_to_hz(torch.linspace(float(FE.hz_to_mel(torch.tensor(lo, dtype=torch.float64))), float(FE.hz_to_mel(torch.tensor(hi, dtype=torch.float64))),
                                      n_mels + 2, dtype=torch.float64))
    fft = torch.linspace(0.0, nyq, freq_bins, dtype=torch.float64)[:, None]
    f0, f1, f2 = pts[None, :-2], pts[None, 1:-1], pts[None, 2:]
    down = torch.where(f1 - f0 == 0, torch.zeros_like(fft - f0), (fft - f0) / (f1 - f0))
    up = torch.where(f2 - f1 == 0, torch.zeros_like(f2 - fft), (f2 - fft) / (f2 - f1))
    norm = torch.where(f2 - f0 == 0, torch.zeros_like(f2 - f0), 2.0 / (f2 - f0))
    return (torch.clamp(torch.minimum(down, up), min=0.0) * norm).float()


def compute_speaker_mel(wave: torch.Tensor, sample_rate: int, n_mels: int, n_fft: int = 1024, hop: int = 256, win: int = 1024, fmin: float = 0.0,
                        fmax: Optional[float] = None) -> torch.Tensor:
    """[1, frames, n_mels] log-magnitude mel: reflect-pad (n_fft - hop) / 2, Hann STFT without centring, sqrt(re^2 + im^2 + 1e-9),
    Slaney filter bank, log of the clamp to [1e-5, 1e10]."""
    if wave.numel() == 0:
        raise ValueError("Reference audio is empty after loading/resampling.")
    if min(n_fft, hop, win) <= 0:
        raise ValueError("Invalid STFT config for speaker mel (n_fft/hop_size/win_size must be > 0).")
    pad = (n_fft - hop) // 2 if n_fft > hop else 0
    x = wave.reshape(-1).float()
    if pad:
        if x.numel() == 1:
            x = x.repeat(1 + 2 * pad)
        else:
            idx = torch.arange(-pad, x.numel() + pad)
            period = 2 * x.numel() - 2
            idx = idx.abs() % period
            idx = torch.where(idx >= x.numel(), period - idx, idx)
            x = x[idx]
    if x.numel() < n_fft:
        raise ValueError(f"STFT parameters n_fft={n_fft} hop={hop} win={win} do not fit {x.numel()} samples")
    spec = torch.stft(x, n_fft, hop, win, torch.hann_window(win, periodic=True), center=False, return_complex=True)
    mag = torch.sqrt(spec.real ** 2 + spec.imag ** 2 + 1e-9)
    bank = slaney_mel_filter_bank(n_fft // 2 + 1, n_mels, sample_rate, fmin, fmax if fmax is not None else sample_rate / 2.0)
    return torch.log((bank.t() @ mag).clamp(1e-5, 1e10)).t()[None]


def format_code_rows(flat: List[int], groups: int) -> str:
    if groups == 0 or not flat:
        return ""
    rows = len(flat) // groups
    return "".join(" ".join(str(v) for v in flat[r * groups:(r + 1) * groups]) + "\n" for r in range(rows))


def parse_code_rows(text: str) -> torch.Tensor:
    """[frames, groups] int64 from whitespace-separated rows."""
    rows = [[int(t) for t in line.split()] for line in text.splitlines() if line.strip()]
    if rows and any(len(r) != len(rows[0]) for r in rows):
        raise ValueError("codec rows have different lengths")
    return torch.tensor(rows, dtype=torch.long).reshape(len(rows), len(rows[0]) if rows else 0)


def encode_audio_to_codes(model_dir: str, audio_path: str, codes_path: str, device="cpu", speech_tokenizer_dir: Optional[str] = None,
                          chunk_seconds: int = 10, left_context_seconds: int = 12) -> Tuple[int, int]:
    """Writes one row of codec ids per frame and returns (rows, groups).  The 12 Hz family streams inputs longer than
    ``chunk_seconds`` through :func:`push_encode_stream` so that the attention window stays bounded."""
    tok_dir = resolve_speech_tokenizer_dir(model_dir, speech_tokenizer_dir)
    codes_path = os.path.expanduser(codes_path)
    os.makedirs(os.path.dirname(codes_path) or ".", exist_ok=True)
    if is_tokenizer_25hz(tok_dir):
        enc = E.load_encoder_25hz(tok_dir, device)
        wave = load_resampled_mono_wav(audio_path, enc.cfg.input_sample_rate)
        if wave.numel() == 0:
            raise ValueError(f"Audio encode input is empty: {audio_path}")
        groups, vals = enc.encode_wave_to_codes(wave)
        with open(codes_path, "w", encoding="utf-8") as f:
            f.write(format_code_rows(vals, groups))
        return len(vals) // groups, groups
    enc = E.load_encoder_12hz(tok_dir, device)
    wave = load_resampled_mono_wav(audio_path, enc.cfg.input_sample_rate)
    if wave.numel() == 0:
        raise ValueError(f"Audio encode input is empty: {audio_path}")
    return encode_wave_12hz(enc, wave, codes_path, chunk_seconds, left_context_seconds)


def encode_wave_12hz(enc: E.SpeechTokenizer12HzEncoder, wave: torch.Tensor, codes_path: str, chunk_seconds: int = 10, left_context_seconds: int = 12) -> Tuple[int, int]:
    rate, groups = enc.cfg.input_sample_rate, enc.num_code_groups
    chunk = rate * chunk_seconds
    expected = E.encoded_frames(wave.numel())
    with open(codes_path, "w", encoding="utf-8") as f:
        if wave.numel() <= chunk:
            dev = enc.p["encoder.downsample.conv.weight"].device
            vals = enc.encode_mono_frame_major(wave.to(dev)).reshape(-1).tolist()
            f.write(format_code_rows(vals, groups))
            return len(vals) // groups, groups
        state, written, samples = E.EncodeStreamState(chunk, rate * left_context_seconds), 0, wave.tolist()
        for off in range(0, len(samples), chunk):
            if written >= expected:
                break
            state, vals = E.push_encode_stream(enc, state, samples[off:off + chunk])
            rows = min(len(vals) // groups, expected - written)
            f.write(format_code_rows(vals[:rows * groups], groups))
            written += rows
        return written, groups


def decode_codes_to_wav(dec: T.SpeechDecoder, codes_path: str, wav_path: str, num_code_groups: Optional[int] = None, sample_rate: int = 24000) -> int:
    """Reads codec rows, decodes them in chunks with left context and writes 16-bit PCM; returns the number of samples."""
    with open(os.path.expanduser(codes_path), encoding="utf-8") as f:
        codes = parse_code_rows(f.read())
    nq = dec.cfg.num_quantizers
    if num_code_groups is not None and codes.shape[1] != num_code_groups:
        raise ValueError(f"codec rows have {codes.shape[1]} groups, expected {num_code_groups}")
    if codes.shape[1] < nq:
        raise ValueError(f"codec rows have {codes.shape[1]} groups, the decoder needs {nq}")
    wave = dec.decode_chunked(codes[:, :nq].t()[None].to(dec.device))[0, 0].float().cpu()
    wav_path = os.path.expanduser(wav_path)
    os.makedirs(os.path.dirname(wav_path) or ".", exist_ok=True)
    media.save_wav(wav_path, wave, sample_rate)
    return wave.numel()


def prepare_speaker_mel(audio_path: str, mel_out_path: str, mel_frames_path: str, sample_rate: int = 24000, mel_dim: int = 128) -> int:
    """Speaker-encoder input for a reference recording: tensor ``mel`` [1, frames, mel_dim] as safetensors plus the frame count."""
    wave = load_resampled_mono_wav(audio_path, sample_rate)
    mel = compute_speaker_mel(wave, sample_rate, mel_dim, 1024, 256, 1024, 0.0, sample_rate / 2.0)
    for p in (mel_out_path, mel_frames_path):
        os.makedirs(os.path.dirname(os.path.expanduser(p)) or ".", exist_ok=True)
    st.save_file({"mel": mel.contiguous()}, os.path.expanduser(mel_out_path))
    with open(os.path.expanduser(mel_frames_path), "w", encoding="utf-8") as f:
        f.write(f"{mel.shape[1]}\n")
    return mel.shape[1]


def extract_speaker_embedding_from_audio(model: T.Qwen3TTS, audio_path: str, mel_out_path: str = "", mel_frames_path: str = "") -> torch.Tensor:
    """[1, 1, talker hidden] speaker embedding of a reference recording; optionally also stores the mel and its frame count."""
    sc = model.cfg.speaker_encoder
    if sc.enc_dim != model.cfg.talker.hidden_size:
        raise ValueError(f"speaker embedding dim mismatch: speaker enc_dim={sc.enc_dim}, talker hidden={model.cfg.talker.hidden_size}")
    wave = load_resampled_mono_wav(audio_path, sc.sample_rate)
    mel = compute_speaker_mel(wave, sc.sample_rate, sc.mel_dim, 1024, 256, 1024, 0.0, sc.sample_rate / 2.0)
    if mel_out_path.strip():
        os.makedirs(os.path.dirname(os.path.expanduser(mel_out_path.strip())) or ".", exist_ok=True)
        st.save_file({"mel": mel.contiguous()}, os.path.expanduser(mel_out_path.strip()))
    if mel_frames_path.strip():
        os.makedirs(os.path.dirname(os.path.expanduser(mel_frames_path.strip())) or ".", exist_ok=True)
        with open(os.path.expanduser(mel_frames_path.strip()), "w", encoding="utf-8") as f:
            f.write(f"{mel.shape[1]}\n")
    return model.extract_speaker_embedding(mel).reshape(1, 1, model.cfg.talker.hidden_size)
