"""Parquet reading (Tyr/Parquet.lean + cc/src/tyr_parquet.cpp use Arrow C++; here pyarrow): whole file to JSON rows,
row-group streaming of one text column with a resumable cursor."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterator, List, Optional


import ctypes
import json
import os


def _pq():
    import pyarrow.parquet as pq
    return pq


def _native():
    """The native reader (csrc/parquet/parquet_reader.cpp), or None when it is not built or TYR_PARQUET_NATIVE=0."""
    if os.environ.get("TYR_PARQUET_NATIVE", "1") == "0":
        return None
    from .._native import parquet
    return parquet()


class ParquetError(RuntimeError):
    pass


class NativeParquetFile:
    """One open parquet file on the native reader: metadata, a string column of a row group, JSON lines."""

    def __init__(self, path: str):
        self.lib = _native()
        if self.lib is None:
            raise ParquetError("the native parquet reader is not available")
        self.handle = ctypes.c_void_p()
        self._err = ctypes.create_string_buffer(512)
        if self.lib.tyr_parquet_open(os.fsencode(path), ctypes.byref(self.handle), self._err, 512) != 0:
            raise ParquetError(f"{path}: {self._err.value.decode(errors='replace')}")
        info = (ctypes.c_longlong * 3)()
        self.lib.tyr_parquet_info(self.handle, info)
        self.num_rows, self.num_row_groups, self.num_columns = int(info[0]), int(info[1]), int(info[2])

    def close(self):
        if self.handle:
            self.lib.tyr_parquet_close(self.handle)
            self.handle = ctypes.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def row_group_rows(self, g: int) -> int:
        return int(self.lib.tyr_parquet_row_group_rows(self.handle, g))

    def columns(self) -> List[tuple]:
        """(dotted name, parquet physical type tag) of every leaf column."""
        buf, out = ctypes.create_string_buffer(512), []
        for i in range(self.num_columns):
            t = self.lib.tyr_parquet_column(self.handle, i, buf, 512)
            out.append((buf.value.decode(), t))
        return out

    def read_text(self, row_group: int, column: str = "text") -> List[Optional[str]]:
        data, off, valid, n = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_longlong()
        rc = self.lib.tyr_parquet_read_text(self.handle, row_group, column.encode(), ctypes.byref(data), ctypes.byref(off),
                                            ctypes.byref(valid), ctypes.byref(n), self._err, 512)
        if rc != 0:
            raise ParquetError(self._err.value.decode(errors="replace"))
        try:
            rows = n.value
            offs = (ctypes.c_longlong * (rows + 1)).from_address(off.value)
            ok = (ctypes.c_ubyte * max(rows, 1)).from_address(valid.value)
            blob = ctypes.string_at(data.value, offs[rows])
            return [blob[offs[i]:offs[i + 1]].decode("utf-8", errors="replace") if ok[i] else None for i in range(rows)]
        finally:
            for q in (data, off, valid):
                self.lib.tyr_parquet_free(q)

    def json_lines(self, row_group: int = -1) -> str:
        out, n = ctypes.c_void_p(), ctypes.c_longlong()
        rc = self.lib.tyr_parquet_to_json_lines(self.handle, row_group, ctypes.byref(out), ctypes.byref(n), self._err, 512)
        if rc != 0:
            raise ParquetError(self._err.value.decode(errors="replace"))
        try:
            return ctypes.string_at(out.value, n.value).decode("utf-8", errors="replace")
        finally:
            self.lib.tyr_parquet_free(out)


def read_parquet_to_json(path: str) -> List[dict]:
    """Every row as a dict.  Flat schemas go through the native reader's JSON lines; nested ones through pyarrow."""
    if _native() is not None:
        try:
            with NativeParquetFile(path) as f:
                return [json.loads(l) for l in f.json_lines().splitlines()]
        except ParquetError:
            pass
    return _pq().read_table(path).to_pylist()


def read_parquet_to_json_streaming(path: str) -> Iterator[dict]:
    if _native() is not None:
        try:
            f = NativeParquetFile(path)
            first = f.json_lines(0) if f.num_row_groups else ""
        except ParquetError:
            f = None
        if f is not None:
            with f:
                for g in range(f.num_row_groups):
                    for l in (first if g == 0 else f.json_lines(g)).splitlines():
                        yield json.loads(l)
            return
    f = _pq().ParquetFile(path)
    for g in range(f.num_row_groups):
        yield from f.read_row_group(g).to_pylist()


_groups_cache: dict = {}


def num_row_groups(path: str) -> int:
    key = (path, os.path.getmtime(path) if os.path.exists(path) else 0)
    if key not in _groups_cache:
        if _native() is not None:
            with NativeParquetFile(path) as f:
                _groups_cache[key] = f.num_row_groups
        else:
            _groups_cache[key] = _pq().ParquetFile(path).num_row_groups
    return _groups_cache[key]


def read_text_column(path: str, row_group: int, column: str = "text") -> List[str]:
    if _native() is not None:
        try:
            with NativeParquetFile(path) as f:
                return f.read_text(row_group, column)
        except ParquetError:
            pass
    return _pq().ParquetFile(path).read_row_group(row_group, columns=[column]).column(column).to_pylist()


@dataclass
class ParquetCursor:
    """Position of a document stream over a list of parquet shards (file, row group, row); JSON-serialisable."""
    file_idx: int = 0
    row_group: int = 0
    row: int = 0
    epoch: int = 0

    def to_json(self) -> dict:
        return {"file_idx": self.file_idx, "row_group": self.row_group, "row": self.row, "epoch": self.epoch}

    @staticmethod
    def from_json(j: dict) -> "ParquetCursor":
        return ParquetCursor(j.get("file_idx", 0), j.get("row_group", 0), j.get("row", 0), j.get("epoch", 0))


class ParquetDocumentStream:
    """Documents of ``column`` from ``paths`` in order, rank-strided by row group, endlessly (epochs); ``cursor`` always
    points at the next unread document so a checkpointed cursor resumes exactly (Examples/NanoChat/Pipeline.lean:815-973)."""

    def __init__(self, paths: List[str], column: str = "text", rank: int = 0, world_size: int = 1,
                 cursor: Optional[ParquetCursor] = None):
        if not paths:
            raise ValueError("no parquet files")
        self.paths, self.column, self.rank, self.world = list(paths), column, rank, max(1, world_size)
        self.cursor = cursor or ParquetCursor(row_group=rank)
        self._rows: Optional[List[str]] = None

    def _advance_group(self):
        c = self.cursor
        c.row_group += self.world
        c.row = 0
        self._rows = None
        while c.row_group >= num_row_groups(self.paths[c.file_idx]):
            c.row_group -= num_row_groups(self.paths[c.file_idx])
            c.file_idx += 1
            if c.file_idx >= len(self.paths):
                c.file_idx, c.epoch = 0, c.epoch + 1
                c.row_group = self.rank

    def __iter__(self):
        return self

    def __next__(self) -> str:
        for _ in range(1 << 20):
            c = self.cursor
            if c.row_group >= num_row_groups(self.paths[c.file_idx]):
                c.row_group -= self.world
                self._advance_group()
                continue
            if self._rows is None:
                self._rows = read_text_column(self.paths[c.file_idx], c.row_group, self.column)
            if c.row < len(self._rows):
                doc = self._rows[c.row]
                c.row += 1
                return doc
            self._advance_group()
        raise RuntimeError("parquet stream made no progress (all shards empty?)")
