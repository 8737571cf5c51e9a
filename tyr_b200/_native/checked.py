"""Access to ``libtyr_kernels_checked.so``: the index-consuming kernels compiled with ``-DTYR_BOUNDS_CHECK``.  Used to hunt
a bad index without a sanitizer: run the suspect op through ``checked()`` and read ``bounds_status(unit)``, which returns
``(code, tag, index, limit)`` of the first violation since the last read (code 0 = none) and clears the record."""
from __future__ import annotations

import ctypes
from pathlib import Path
from typing import Tuple

_lib = None
STATUS_FNS = {"moe": "tyr_bounds_status_moe", "rope": "tyr_bounds_status_rope"}
UNITS = tuple(STATUS_FNS)


def checked():
    global _lib
    if _lib is None:
        path = Path(__file__).resolve().parent / "libtyr_kernels_checked.so"
        if not path.exists():
            from . import build as b
            b.build_kernels(checked=True)
        _lib = ctypes.CDLL(str(path))
        P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        _lib.tyr_rope_norm.argtypes = [P, P, P, P, P, P, L, L, I, I, I, I, I, F, I, P]
        _lib.tyr_moe_gather_rows.argtypes = [P, P, P, I, I, I, P]
        for u in UNITS:
            getattr(_lib, STATUS_FNS[u]).argtypes = [ctypes.POINTER(ctypes.c_int)]
    return _lib


def bounds_status(unit: str) -> Tuple[int, int, int, int]:
    out = (ctypes.c_int * 4)()
    rc = getattr(checked(), STATUS_FNS[unit])(out)
    if rc != 0:
        raise RuntimeError(f"{STATUS_FNS[unit]} failed with CUDA error {rc}")
    return tuple(out)
