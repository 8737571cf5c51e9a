"""Native parquet reader (csrc/parquet/parquet_reader.cpp over the Arrow C++ inside pyarrow) against pyarrow itself."""
import json

import pytest

pa = pytest.importorskip("pyarrow")
import pyarrow.parquet as pq

from tyr_b200.data import parquet as PQ


@pytest.fixture()
def shard(tmp_path):
    t = pa.table({"text": ["hello", None, "wörld \"q\"\n\t\\", "", "x" * 5000], "n": [1, 2, None, 4, -5],
                  "f": [0.5, 1.25, 3.0, None, 1e-9], "b": [True, False, None, True, False]})
    p = str(tmp_path / "t.parquet")
    pq.write_table(t, p, row_group_size=2)
    return p, t


def test_native_reader_is_built_and_loaded():
    assert PQ._native() is not None, "libtyr_parquet.so was not built although pyarrow is installed"


def test_metadata_text_column_and_json_lines_match_pyarrow(shard):
    p, t = shard
    with PQ.NativeParquetFile(p) as f:
        assert (f.num_rows, f.num_row_groups, f.num_columns) == (5, 3, 4)
        assert [f.row_group_rows(g) for g in range(3)] == [2, 2, 1] and f.row_group_rows(7) == -1
        assert [c[0] for c in f.columns()] == ["text", "n", "f", "b"]
        got = [r for g in range(3) for r in f.read_text(g, "text")]
        assert got == t.column("text").to_pylist()
        assert [json.loads(l) for l in f.json_lines().splitlines()] == t.to_pylist()
        assert [json.loads(l) for l in f.json_lines(1).splitlines()] == t.to_pylist()[2:4]
        with pytest.raises(PQ.ParquetError, match="no column named"):
            f.read_text(0, "missing")
        with pytest.raises(PQ.ParquetError, match="not a flat string"):
            f.read_text(0, "n")
        with pytest.raises(PQ.ParquetError, match="out of range"):
            f.read_text(9, "text")
    with pytest.raises(PQ.ParquetError):
        PQ.NativeParquetFile(p + ".missing")


def test_module_functions_use_native_and_fall_back_for_nested(shard, tmp_path, monkeypatch):
    p, t = shard
    assert PQ.read_parquet_to_json(p) == t.to_pylist() and list(PQ.read_parquet_to_json_streaming(p)) == t.to_pylist()
    assert PQ.num_row_groups(p) == 3 and PQ.read_text_column(p, 2) == ["x" * 5000]
    nested = pa.table({"text": ["a", "b"], "tags": [["x", "y"], []]})
    q = str(tmp_path / "n.parquet")
    pq.write_table(nested, q)
    assert PQ.read_parquet_to_json(q) == nested.to_pylist() and list(PQ.read_parquet_to_json_streaming(q)) == nested.to_pylist()
    assert PQ.read_text_column(q, 0) == ["a", "b"]
    monkeypatch.setenv("TYR_PARQUET_NATIVE", "0")
    assert PQ._native() is None and PQ.read_parquet_to_json(p) == t.to_pylist()
