"""Apple-only device services (Metal probe, microphone capture, beep playback): on Linux the native library exports
the same entry points as error stubs, as the reference does for its non-Apple builds (cc/src/apple_audio_input.mm:275-310,
cc/src/apple_audio_output.mm:198-216, Tyr/Audio/{AppleInput,AppleOutput}.lean)."""
from __future__ import annotations

import ctypes

from .._native import host, register_host_signatures


@register_host_signatures
def _sigs(lib):
    lib.tyr_audio_input_start.restype = ctypes.c_char_p
    lib.tyr_audio_output_beep.restype = ctypes.c_char_p
    lib.tyr_apple_mps_is_available.restype = ctypes.c_int


def mps_is_available() -> bool:
    return bool(host().tyr_apple_mps_is_available())


def start_microphone():
    """Raises IOError off macOS (there is no capture queue to start)."""
    raise IOError(host().tyr_audio_input_start().decode())


def beep():
    raise IOError(host().tyr_audio_output_beep().decode())
