"""VAD signals for the streaming consensus: feeds 16 kHz PCM through the Silero iterator in 512-sample chunks,
carrying the residue between calls (Tyr/Text/VADProvider.lean)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..models import silero_vad as sv


@dataclass
class VADSignal:
    speech_active: bool = True
    boundary: bool = False


class SileroProvider:
    def __init__(self, model: sv.SileroVAD, threshold: float = 0.5, min_silence_duration_ms: int = 100, speech_pad_ms: int = 30):
        self.iterator = sv.VADIterator(sv.SileroVADRuntime(model), threshold, 16000, min_silence_duration_ms, speech_pad_ms)
        self.residue = torch.zeros(0)
        self.speech_active = False

    @staticmethod
    def from_weights(path: str, device="cpu", **kw) -> "SileroProvider":
        return SileroProvider(sv.SileroVAD.load(path, device), **kw)

    def step(self, pcm16k: torch.Tensor) -> VADSignal:
        allx = torch.cat([self.residue, pcm16k.float().cpu()])
        n_full = allx.numel() // sv.CHUNK * sv.CHUNK
        boundary = False
        for i in range(0, n_full, sv.CHUNK):
            b = self.iterator.step(allx[i:i + sv.CHUNK])
            self.speech_active = self.iterator.triggered
            if b is not None and b.kind == "end":
                boundary = True
        self.residue = allx[n_full:]
        return VADSignal(self.speech_active, boundary)
