"""ctypes bindings to the in-tree native libraries.

``kernels()`` returns ``libtyr_kernels.so`` (CUDA, sm_100a) and ``host()`` returns
``libtyr_host.so`` (C++ runtime pieces).  Both are built by :mod:`tyr_b200._native.build`.
A missing kernel library is a hard error whenever a CUDA tensor reaches an op: there is no
silent eager fallback on a GPU machine.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

_HERE = Path(__file__).resolve().parent
_lock = threading.Lock()
_kernels = None
_host = None


class NativeLibraryMissing(RuntimeError):
    pass


def _load(name: str):
    path = _HERE / name
    if not path.exists():
        if os.environ.get("TYR_B200_AUTOBUILD", "1") != "0":
            from . import build as _b
            try:
                if name == "libtyr_kernels.so":
                    _b.build_kernels()
                elif name == "libtyr_parquet.so":
                    _b.build_parquet()
                else:
                    _b.build_host()
            except Exception as e:  # pragma: no cover - build environment specific
                raise NativeLibraryMissing(f"{name} is not built and building it failed: {e}") from e
        if not path.exists():
            raise NativeLibraryMissing(
                f"{path} not found; run `python -m tyr_b200._native.build` (or __graft_entry__.build())")
    return ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)


def kernels():
    global _kernels
    if _kernels is None:
        with _lock:
            if _kernels is None:
                lib = _load("libtyr_kernels.so")
                _declare_kernels(lib)
                _kernels = lib
    return _kernels


def host():
    global _host
    if _host is None:
        with _lock:
            if _host is None:
                lib = _load("libtyr_host.so")
                _declare_host(lib)
                _host = lib
    return _host


_parquet = None


def parquet():
    """``libtyr_parquet.so`` (native parquet reader) or None when it was not built (no pyarrow at build time)."""
    global _parquet
    if _parquet is None:
        with _lock:
            if _parquet is None:
                try:
                    lib = _load("libtyr_parquet.so")
                except Exception:
                    _parquet = False
                    return None
                P, I, L, C = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_char_p
                PP, PL = ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_longlong)
                lib.tyr_parquet_open.argtypes, lib.tyr_parquet_open.restype = [C, PP, C, I], I
                lib.tyr_parquet_close.argtypes, lib.tyr_parquet_close.restype = [P], None
                lib.tyr_parquet_info.argtypes, lib.tyr_parquet_info.restype = [P, PL], I
                lib.tyr_parquet_row_group_rows.argtypes, lib.tyr_parquet_row_group_rows.restype = [P, I], L
                lib.tyr_parquet_column.argtypes, lib.tyr_parquet_column.restype = [P, I, C, I], I
                lib.tyr_parquet_read_text.argtypes, lib.tyr_parquet_read_text.restype = [P, I, C, PP, PP, PP, PL, C, I], I
                lib.tyr_parquet_to_json_lines.argtypes, lib.tyr_parquet_to_json_lines.restype = [P, I, PP, PL, C, I], I
                lib.tyr_parquet_free.argtypes, lib.tyr_parquet_free.restype = [P], None
                _parquet = lib
    return _parquet or None


def kernels_available() -> bool:
    try:
        kernels()
        return True
    except Exception:
        return False


c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float
c_double = ctypes.c_double


class GemmArgs(ctypes.Structure):
    _fields_ = [
        ("A", c_void_p), ("B", c_void_p), ("C", c_void_p), ("aux", c_void_p),
        ("M", c_int), ("N", c_int), ("K", c_int), ("batch", c_int),
        ("lda", c_ll), ("ldb", c_ll), ("ldc", c_ll), ("ldaux", c_ll),
        ("sA", c_ll), ("sB", c_ll), ("sC", c_ll), ("sAux", c_ll),
        ("a_mn", c_int), ("b_mn", c_int), ("out_mode", c_int), ("act", c_int),
        ("alpha", c_float), ("beta", c_float),
        ("bn", c_int), ("sm_count", c_int),
        ("err", c_void_p), ("stream", c_void_p), ("group_offsets", c_void_p), ("group_tiles", c_void_p),
    ]


def _sig(lib, name, argtypes, restype=c_int):
    fn = getattr(lib, name, None)
    if fn is None:
        return
    fn.argtypes = argtypes
    fn.restype = restype


def _declare_kernels(lib):
    P = c_void_p
    _sig(lib, "tyr_gemm_bf16", [ctypes.POINTER(GemmArgs)])
    _sig(lib, "tyr_bind_device", [c_int])
    _sig(lib, "tyr_newton_schulz_scratch_bytes", [c_int, c_int, c_int], c_ll)
    _sig(lib, "tyr_newton_schulz_bf16", [P, P, c_ll, c_int, c_int, c_int, c_int, c_float, c_float, c_float, P, P])
    _sig(lib, "tyr_lincomb_rmsnorm_fwd", [P, P, P, P, P, c_int, c_int, c_int, P, P, c_float, P])
    _sig(lib, "tyr_lincomb_rmsnorm_bwd",
         [ctypes.POINTER(P), ctypes.POINTER(P), P, P, P, P, P, c_int, c_int, c_int, c_float, P])
    _sig(lib, "tyr_rmsnorm_weighted", [P, P, P, P, P, P, c_int, c_int, c_float, c_int, P])
    _sig(lib, "tyr_qkv_post_fwd", [P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_float, P])
    _sig(lib, "tyr_qkv_post_bwd",
         [P, P, P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_float, P])
    _sig(lib, "tyr_rope_norm",
         [P, P, P, P, P, P, c_ll, c_ll, c_int, c_int, c_int, c_int, c_int, c_float, c_int, P])
    _sig(lib, "tyr_softcap_ce", [P, P, P, P, c_int, c_int, c_ll, c_float, c_float, P, c_ll, c_int, P])
    _sig(lib, "tyr_adamw_step",
         [P, P, P, P, P, c_ll, c_float, c_float, c_float, c_float, c_float, c_float, c_float,
          c_float, c_int, P])
    _sig(lib, "tyr_muon_momentum", [P, P, P, P, c_ll, c_int, c_float, c_float, c_int, P])
    _sig(lib, "tyr_scale_by_inv_norm", [P, P, c_ll, c_int, c_float, P])
    _sig(lib, "tyr_muon_apply", [P, P, P, c_ll, c_float, c_float, P])
    # later files declare themselves through register_signatures()
    for fn in _extra_kernel_sigs:
        fn(lib)


_extra_kernel_sigs = []


def register_signatures(fn):
    """Let an ops module declare argtypes for the symbols it uses (applied at load time)."""
    _extra_kernel_sigs.append(fn)
    if _kernels is not None:
        fn(_kernels)
    return fn


def _declare_host(lib):
    if hasattr(lib, "tyr_host_last_error"):
        lib.tyr_host_last_error.restype = ctypes.c_char_p
    for fn in _extra_host_sigs:
        fn(lib)


_extra_host_sigs = []


def register_host_signatures(fn):
    _extra_host_sigs.append(fn)
    if _host is not None:
        fn(_host)
    return fn
