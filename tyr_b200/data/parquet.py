"""Parquet reading (Tyr/Parquet.lean + cc/src/tyr_parquet.cpp use Arrow C++; here pyarrow): whole file to JSON rows,
row-group streaming of one text column with a resumable cursor."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterator, List, Optional


def _pq():
    import pyarrow.parquet as pq
    return pq


def read_parquet_to_json(path: str) -> List[dict]:
    return _pq().read_table(path).to_pylist()


def read_parquet_to_json_streaming(path: str) -> Iterator[dict]:
    f = _pq().ParquetFile(path)
    for g in range(f.num_row_groups):
        yield from f.read_row_group(g).to_pylist()


def num_row_groups(path: str) -> int:
    return _pq().ParquetFile(path).num_row_groups


def read_text_column(path: str, row_group: int, column: str = "text") -> List[str]:
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
