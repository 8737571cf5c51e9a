"""SafeTensors reader/writer with the reference's validation rules.

Header parsing and validation happen here (8-byte LE size, JSON object, <= 100 MiB, per-entry
dtype tag / shape / data_offsets / range / size checks: Tyr/SafeTensors/File.lean:16-111); sharded
``model.safetensors.index.json`` weight maps reject absolute paths, drive prefixes, ``.``/``..``
segments and non-``.safetensors`` names (:135-160); ``Source`` resolves names over a file or a model
directory (Source.lean:20-74).  Byte movement is native (csrc/host/io.cpp: parallel pread into the
destination tensor, fsync'ed writer).
"""
from __future__ import annotations

import ctypes
import json
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .._native import host, register_host_signatures
from ..typed.dtype import DType

MAX_HEADER_BYTES = 100 * 1024 * 1024


@register_host_signatures
def _sigs(lib):
    P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    lib.tyr_host_last_error.restype = ctypes.c_char_p
    lib.tyr_file_size.argtypes = [ctypes.c_char_p]
    lib.tyr_file_size.restype = L
    lib.tyr_file_read_range.argtypes = [ctypes.c_char_p, L, L, P, I]
    lib.tyr_safetensors_write.argtypes = [ctypes.c_char_p, ctypes.c_char_p, L, I, ctypes.POINTER(P), ctypes.POINTER(L)]


class SafeTensorsError(IOError):
    pass


@dataclass(frozen=True)
class Entry:
    dtype: DType
    shape: Tuple[int, ...]
    data_start: int
    data_end: int


@dataclass
class Handle:
    path: str
    data_offset: int
    entries: Dict[str, Entry]
    metadata: Dict[str, str]


def _parse_entry(name: str, j, data_size: int) -> Entry:
    if not isinstance(j, dict):
        raise SafeTensorsError(f"SafeTensors entry '{name}' is not an object")
    if "dtype" not in j:
        raise SafeTensorsError(f"SafeTensors entry '{name}' is missing 'dtype'")
    tag = j["dtype"]
    if not isinstance(tag, str):
        raise SafeTensorsError(f"SafeTensors entry '{name}' has non-string 'dtype'")
    dtype = DType.of_safetensor_tag(tag)
    if dtype is None:
        raise SafeTensorsError(f"SafeTensors entry '{name}' has unsupported dtype '{tag}'")
    width = dtype.safetensor_format[1]
    if "shape" not in j:
        raise SafeTensorsError(f"SafeTensors entry '{name}' is missing 'shape'")
    dims = j["shape"]
    if not isinstance(dims, list) or not all(isinstance(d, int) and not isinstance(d, bool) and d >= 0 for d in dims):
        raise SafeTensorsError(f"SafeTensors entry '{name}' has a malformed 'shape'")
    if "data_offsets" not in j:
        raise SafeTensorsError(f"SafeTensors entry '{name}' is missing 'data_offsets'")
    offs = j["data_offsets"]
    if not (isinstance(offs, list) and len(offs) == 2 and all(isinstance(o, int) and o >= 0 for o in offs)):
        raise SafeTensorsError(f"SafeTensors entry '{name}' has malformed 'data_offsets'")
    start, end = offs
    if start > end:
        raise SafeTensorsError(f"SafeTensors entry '{name}' has an invalid data_offsets range")
    if end > data_size:
        raise SafeTensorsError(f"SafeTensors entry '{name}' exceeds the file's data section (truncated file)")
    n = 1
    for d in dims:
        n *= d
    if end - start != n * width:
        raise SafeTensorsError(f"SafeTensors entry '{name}': data size mismatch (offset range {end - start} bytes)")
    return Entry(dtype, tuple(dims), start, end)


def read_header(path: str) -> Handle:
    def invalid(msg):
        return SafeTensorsError(f"Invalid SafeTensors file '{path}': {msg}")
    try:
        size = os.path.getsize(path)
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) < 8:
                raise invalid("missing 8-byte header size")
            (hsize,) = struct.unpack("<Q", head)
            if hsize > MAX_HEADER_BYTES:
                raise invalid(f"header exceeds {MAX_HEADER_BYTES}-byte limit")
            if 8 + hsize > size:
                raise invalid(f"header exceeds file size ({hsize} bytes)")
            raw = f.read(hsize)
    except OSError as e:
        raise SafeTensorsError(f"Failed to open: {path} ({e})") from None
    if len(raw) != hsize:
        raise invalid("truncated header")
    try:
        text = raw.decode("utf-8")
    except UnicodeDecodeError:
        raise invalid("header is not UTF-8") from None
    try:
        j = json.loads(text)
    except json.JSONDecodeError as e:
        raise invalid(f"failed to parse header JSON: {e}") from None
    if not isinstance(j, dict):
        raise invalid("header is not a JSON object")
    data_offset = 8 + hsize
    entries: Dict[str, Entry] = {}
    meta = {}
    for name, ej in j.items():
        if name == "__metadata__":
            meta = ej if isinstance(ej, dict) else {}
            continue
        try:
            entries[name] = _parse_entry(name, ej, size - data_offset)
        except SafeTensorsError as e:
            raise invalid(str(e)) from None
    return Handle(path, data_offset, entries, meta)


_handle_cache: Dict[str, Handle] = {}


def open_handle(path: str) -> Handle:
    h = _handle_cache.get(path)
    if h is None:
        h = read_header(path)
        _handle_cache[path] = h
    return h


def clear_caches():
    _handle_cache.clear()
    _model_dir_cache.clear()


def read_tensor(handle: Handle, name: str, pin: bool = False, threads: int = 8) -> torch.Tensor:
    e = handle.entries.get(name)
    if e is None:
        raise KeyError(f"tensor '{name}' not found in {handle.path}")
    t = torch.empty(e.shape, dtype=e.dtype.torch, pin_memory=pin and torch.cuda.is_available())
    length = e.data_end - e.data_start
    if t.numel() * t.element_size() != length:
        raise SafeTensorsError(f"SafeTensors load error: data size mismatch (offset range {length} bytes, "
                               f"dtype/shape require {t.numel() * t.element_size()}).")
    if length:
        lib = host()
        rc = lib.tyr_file_read_range(handle.path.encode(), handle.data_offset + e.data_start, length,
                                     ctypes.c_void_p(t.data_ptr()), threads)
        if rc != 0:
            raise SafeTensorsError(lib.tyr_host_last_error().decode())
    return t


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None) -> None:
    """Write several tensors into one file (entries in insertion order, offsets contiguous)."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    cpu: List[torch.Tensor] = []
    off = 0
    for name, t in tensors.items():
        if not name:
            raise SafeTensorsError("SafeTensors save error: tensor name cannot be empty.")
        fmt = DType.of_torch(t.dtype).safetensor_format
        if fmt is None:
            raise SafeTensorsError(f"SafeTensors save error: unsupported dtype for tensor '{name}'.")
        c = t.detach().to("cpu").contiguous()
        n = c.numel() * c.element_size()
        header[name] = {"dtype": fmt[0], "shape": list(c.shape), "data_offsets": [off, off + n]}
        off += n
        cpu.append(c)
    hb = json.dumps(header, separators=(",", ":")).encode()
    hb += b" " * ((8 - len(hb) % 8) % 8)
    lib = host()
    P = ctypes.c_void_p
    ptrs = (P * len(cpu))(*[c.data_ptr() for c in cpu])
    lens = (ctypes.c_longlong * len(cpu))(*[c.numel() * c.element_size() for c in cpu])
    if lib.tyr_safetensors_write(path.encode(), hb, len(hb), len(cpu), ptrs, lens) != 0:
        raise SafeTensorsError(lib.tyr_host_last_error().decode())
    _handle_cache.pop(path, None)


def save_safe_tensor(path: str, name: str, tensor: torch.Tensor) -> None:
    """Single-tensor file (``RawTensor.saveSafeTensor``, File.lean:213)."""
    save_file({name: tensor}, path)


# ---- sharded model directories ----------------------------------------------------------------------
def _unsafe_shard(file: str) -> bool:
    if file.startswith("/") or file.startswith("\\"):
        return True
    if len(file) >= 2 and file[1] == ":" and file[0].isalpha():
        return True
    segs = set(file.split("/")) | set(file.split("\\"))
    return ".." in segs or "." in segs


def read_weight_map(index_path: str) -> List[Tuple[str, str]]:
    def invalid(msg):
        return SafeTensorsError(f"Invalid SafeTensors index '{index_path}': {msg}")
    try:
        with open(index_path, "r", encoding="utf-8") as f:
            j = json.load(f)
    except json.JSONDecodeError as e:
        raise invalid(f"failed to parse JSON: {e}") from None
    if not isinstance(j, dict) or "weight_map" not in j:
        raise invalid("missing 'weight_map'")
    wm = j["weight_map"]
    if not isinstance(wm, dict):
        raise invalid("'weight_map' must be a JSON object")
    if not wm:
        raise invalid("'weight_map' is empty")
    out = []
    for name, file in wm.items():
        if not isinstance(file, str):
            raise invalid(f"tensor '{name}' has non-string shard filename")
        if not file:
            raise invalid(f"tensor '{name}' maps to an empty shard filename")
        if _unsafe_shard(file):
            raise invalid(f"unsafe shard path '{file}' (must be relative and stay within the directory)")
        if not file.endswith(".safetensors"):
            raise invalid(f"shard '{file}' must use '.safetensors' extension")
        out.append((name, file))
    return out


@dataclass
class Stored:
    file: str
    handle: Handle
    entry: Entry


_model_dir_cache: Dict[str, Dict[str, Stored]] = {}


def open_model_dir(directory: str) -> Dict[str, Stored]:
    cached = _model_dir_cache.get(directory)
    if cached is not None:
        return cached
    index = os.path.join(directory, "model.safetensors.index.json")
    single = os.path.join(directory, "model.safetensors")
    tensors: Dict[str, Stored] = {}
    if os.path.exists(index):
        for name, file in read_weight_map(index):
            path = os.path.join(directory, file)
            if not os.path.exists(path):
                raise SafeTensorsError(f"Invalid SafeTensors index '{index}': referenced shard does not exist: '{file}'")
            if os.path.isdir(path):
                raise SafeTensorsError(f"Invalid SafeTensors index '{index}': referenced shard is a directory: '{file}'")
            h = open_handle(path)
            if name not in h.entries:
                raise SafeTensorsError(f"Invalid SafeTensors index '{index}': tensor '{name}' not found in shard '{file}'")
            tensors[name] = Stored(file, h, h.entries[name])
    elif os.path.exists(single):
        h = open_handle(single)
        tensors = {n: Stored("model.safetensors", h, e) for n, e in h.entries.items()}
    else:
        raise SafeTensorsError(f"No model.safetensors.index.json or model.safetensors in {directory}")
    _model_dir_cache[directory] = tensors
    return tensors


class Source:
    """Name -> tensor over a single file or a model directory (Source.lean:20-74)."""

    def __init__(self, tensors: Dict[str, Stored], origin: str):
        self._t = tensors
        self.origin = origin

    @staticmethod
    def open(path: str) -> "Source":
        if os.path.isdir(path):
            return Source(open_model_dir(path), path)
        h = open_handle(path)
        return Source({n: Stored("", h, e) for n, e in h.entries.items()}, path)

    def names(self) -> List[str]:
        return sorted(self._t)

    def find(self, name: str) -> Optional[Stored]:
        return self._t.get(name)

    def resolve(self, *candidates: str) -> str:
        """First candidate name that exists (weight-name aliases)."""
        for c in candidates:
            if c in self._t:
                return c
        raise KeyError(f"none of {candidates} found in {self.origin}")

    def spec(self, name: str) -> Tuple[Tuple[int, ...], DType]:
        s = self._t[name]
        return s.entry.shape, s.entry.dtype

    def load(self, name: str, pin: bool = False) -> torch.Tensor:
        s = self._t.get(name)
        if s is None:
            raise KeyError(f"tensor '{name}' not found in {self.origin}")
        return read_tensor(s.handle, name, pin=pin)

    def load_as(self, name: str, shape: Sequence[int], dtype: DType, device=None) -> torch.Tensor:
        """Typed load: the stored shape and dtype must match the expectation exactly."""
        st_shape, st_dtype = self.spec(name)
        if tuple(shape) != st_shape:
            raise ValueError(f"{name}: stored shape {list(st_shape)} != expected {list(shape)}")
        if st_dtype is not dtype:
            raise TypeError(f"{name}: stored dtype {st_dtype} != expected {dtype}")
        t = self.load(name)
        return t.to(device) if device is not None else t

    def load_all(self, device=None, dtype: Optional[torch.dtype] = None) -> Dict[str, torch.Tensor]:
        out = {}
        for n in self.names():
            t = self.load(n)
            if dtype is not None and t.dtype.is_floating_point:
                t = t.to(dtype)
            out[n] = t.to(device) if device is not None else t
        return out


def schema_snapshot(src: Source) -> Dict[str, dict]:
    """name -> {shape, dtype} (Schema.lean:85-111): what the type provider generates loaders from."""
    return {n: {"shape": list(src.spec(n)[0]), "dtype": src.spec(n)[1].name} for n in src.names()}


def safetensors_type_provider(path: str, class_name: str = "Weights"):
    """Run-time type provider (TypeProvider.lean:25,737): returns a class with one typed loader per
    tensor (``load_<sanitised name>(device=None)``) and a nested ``tree()`` mirroring the dotted
    hierarchy.  The generated loaders validate shape and dtype against the snapshot taken here, so
    a later file with a different layout fails loudly."""
    src = Source.open(path)
    snap = schema_snapshot(src)

    def sanitise(n):
        return "".join(c if c.isalnum() else "_" for c in n)

    ns = {"__doc__": f"Typed loaders generated from {path}", "SCHEMA": snap, "_path": path}

    def make(name, shape, dtype):
        def loader(device=None, _name=name, _shape=shape, _dtype=dtype):
            return Source.open(path).load_as(_name, _shape, DType[_dtype], device)
        loader.__name__ = f"load_{sanitise(name)}"
        loader.__doc__ = f"{name}: {dtype}{shape}"
        return staticmethod(loader)

    for name, info in snap.items():
        ns[f"load_{sanitise(name)}"] = make(name, tuple(info["shape"]), info["dtype"])

    def tree():
        root: dict = {}
        for name in snap:
            cur = root
            parts = name.split(".")
            for p in parts[:-1]:
                cur = cur.setdefault(p, {})
            cur[parts[-1]] = name
        return root
    ns["tree"] = staticmethod(tree)
    return type(class_name, (), ns)
