"""WAV / PPM writers, streaming WAV, float ring buffer (csrc/host/io.cpp, float_buffer.cpp)."""
from __future__ import annotations

import ctypes

import torch

from .._native import host, register_host_signatures


@register_host_signatures
def _sigs(lib):
    P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    lib.tyr_save_ppm.argtypes = [ctypes.c_char_p, P, I, I]
    lib.tyr_save_wav.argtypes = [ctypes.c_char_p, P, L, I, I]
    lib.tyr_wav_begin.argtypes = [ctypes.c_char_p, I, I]
    lib.tyr_wav_append.argtypes = [ctypes.c_char_p, P, L]
    lib.tyr_wav_finalize.argtypes = [ctypes.c_char_p, I, I]
    lib.tyr_float_buffer_new.restype = P
    lib.tyr_float_buffer_free.argtypes = [P]
    lib.tyr_float_buffer_size.argtypes = [P]
    lib.tyr_float_buffer_size.restype = L
    lib.tyr_float_buffer_rms.argtypes = [P]
    lib.tyr_float_buffer_rms.restype = ctypes.c_double
    lib.tyr_float_buffer_get.argtypes = [P, L, ctypes.POINTER(F)]
    lib.tyr_float_buffer_push.argtypes = [P, F]
    lib.tyr_float_buffer_append.argtypes = [P, P, L]
    lib.tyr_float_buffer_append_buffer.argtypes = [P, P]
    lib.tyr_float_buffer_clear.argtypes = [P]
    lib.tyr_float_buffer_copy_out.argtypes = [P, P]
    lib.tyr_float_buffer_keep_last.argtypes = [P, L]
    for n in ("tyr_media_load_image_patchified", "tyr_media_load_video_patchified",
              "tyr_media_load_image_patch_grid_gemma4"):
        getattr(lib, n).argtypes = [ctypes.c_char_p]
        getattr(lib, n).restype = ctypes.c_char_p


def _err(lib):
    return lib.tyr_host_last_error().decode()


def save_ppm(path: str, image: torch.Tensor) -> None:
    """image: float [3, H, W] in [0, 1]."""
    if image.dim() != 3 or image.shape[0] != 3:
        raise ValueError(f"save_ppm expects [3, H, W], got {list(image.shape)}")
    img = image.detach().float().cpu().contiguous()
    lib = host()
    if lib.tyr_save_ppm(path.encode(), ctypes.c_void_p(img.data_ptr()), img.shape[1], img.shape[2]) != 0:
        raise IOError(_err(lib))


def save_wav(path: str, samples: torch.Tensor, sample_rate: int, channels: int = 1) -> None:
    s = samples.detach().float().cpu().contiguous().reshape(-1)
    lib = host()
    if lib.tyr_save_wav(path.encode(), ctypes.c_void_p(s.data_ptr()), s.numel(), sample_rate, channels) != 0:
        raise IOError(_err(lib))


class WavStream:
    """wav_begin / wav_append / wav_finalize."""

    def __init__(self, path: str, sample_rate: int, channels: int = 1):
        self.path, self.sr, self.ch = path, sample_rate, channels
        lib = host()
        if lib.tyr_wav_begin(path.encode(), sample_rate, channels) != 0:
            raise IOError(_err(lib))

    def append(self, samples: torch.Tensor):
        s = samples.detach().float().cpu().contiguous().reshape(-1)
        lib = host()
        if lib.tyr_wav_append(self.path.encode(), ctypes.c_void_p(s.data_ptr()), s.numel()) != 0:
            raise IOError(_err(lib))

    def finalize(self):
        lib = host()
        if lib.tyr_wav_finalize(self.path.encode(), self.sr, self.ch) != 0:
            raise IOError(_err(lib))


class FloatBuffer:
    """Growable float buffer used by the streaming audio paths."""

    def __init__(self):
        self._lib = host()
        self._h = self._lib.tyr_float_buffer_new()

    def __del__(self):
        try:
            self._lib.tyr_float_buffer_free(self._h)
        except Exception:
            pass

    def __len__(self):
        return int(self._lib.tyr_float_buffer_size(self._h))

    size = __len__

    def rms(self) -> float:
        return float(self._lib.tyr_float_buffer_rms(self._h))

    def get(self, i: int) -> float:
        out = ctypes.c_float()
        if self._lib.tyr_float_buffer_get(self._h, i, ctypes.byref(out)) != 0:
            raise IndexError(i)
        return out.value

    def push(self, v: float):
        self._lib.tyr_float_buffer_push(self._h, v)

    def append(self, values):
        if isinstance(values, FloatBuffer):
            self._lib.tyr_float_buffer_append_buffer(self._h, values._h)
            return
        t = torch.as_tensor(values, dtype=torch.float32).contiguous()
        self._lib.tyr_float_buffer_append(self._h, ctypes.c_void_p(t.data_ptr()), t.numel())

    def clear(self):
        self._lib.tyr_float_buffer_clear(self._h)

    def to_tensor(self) -> torch.Tensor:
        t = torch.empty(len(self), dtype=torch.float32)
        self._lib.tyr_float_buffer_copy_out(self._h, ctypes.c_void_p(t.data_ptr()))
        return t

    def keep_last(self, n: int):
        self._lib.tyr_float_buffer_keep_last(self._h, n)


def load_image_patchified(path: str):
    """Apple-only in the reference; on Linux it reports the same error."""
    raise IOError(host().tyr_media_load_image_patchified(path.encode()).decode())


def load_video_patchified(path: str):
    raise IOError(host().tyr_media_load_video_patchified(path.encode()).decode())
