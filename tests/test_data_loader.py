"""Token shards, BOS windows, resumable stream cursors (the reference's data-loader cursor tests)."""
import os

import pytest
import torch

from tyr_b200.data import loader as dl


def _make(tmp_path, name, docs, header=True):
    toks = []
    for i, n in enumerate(docs):
        toks += [999] + [(i * 7 + j) % 500 for j in range(n - 1)]
    p = str(tmp_path / name)
    dl.write_u16_bin(p, torch.tensor(toks), with_header=header)
    return p, torch.tensor(toks)


def test_native_loader_header_and_ranges(tmp_path):
    p, toks = _make(tmp_path, "a.bin", [10, 20, 5])
    assert dl.bin_file_token_count(p) == 35
    assert torch.equal(dl.load_u16_bin(p), toks) and torch.equal(dl.load_u16_bin(p, 3, 4), toks[3:7])
    q, toks2 = _make(tmp_path, "raw.bin", [6], header=False)
    assert dl.bin_file_token_count(q) == 6 and torch.equal(dl.load_u16_bin(q), toks2)
    with pytest.raises(IOError):
        dl.load_u16_bin(p, 30, 10)
    assert dl.find_bos_positions(toks, 999) == [0, 10, 30]


def test_bos_finder_packs_documents_and_shuffles(tmp_path):
    _, toks = _make(tmp_path, "a.bin", [4, 6, 3, 7])
    f = dl.BOSFinder(toks, 999)
    b = f.get_batch(2, 5)
    assert torch.equal(b.reshape(-1), toks[:10]) and f.current_pos == 10
    assert f.get_batch(3, 5) is None
    f.shuffle(123)
    out = f.take(20)
    assert sorted(out.tolist()) == sorted(toks.tolist()) and not torch.equal(out, toks)
    assert (out == 999).sum() == 4 and out[0] == 999


def test_data_shard_splits_by_rank(tmp_path):
    p, toks = _make(tmp_path, "a.bin", [8] * 5)
    parts = [dl.DataShard.load(p, r, 3, 999).tokens for r in range(3)]
    assert [t.numel() for t in parts] == [13, 13, 14] and torch.equal(torch.cat(parts), toks)
    with pytest.raises(ValueError):
        dl.DataShard.load(p, 3, 3, 999)


def test_generator_cursor_resume(tmp_path):
    d = tmp_path / "shards"
    d.mkdir()
    for i in range(3):
        _make(d, f"train_{i}.bin", [5 + i, 9, 4, 11])
    cfg = dl.LoaderConfig(str(d), bos_token=999, seed=7, shuffle=True)
    g = dl.DistributedDataGenerator(cfg, 0, 2)
    seq = [g.next_tokens(7) for _ in range(3)]
    cur = dl.StreamCursor.from_json(g.cursor().to_json())
    after = [g.next_tokens(7) for _ in range(6)]        # crosses files and an epoch
    g2 = dl.DistributedDataGenerator(cfg, 0, 2).restore_cursor(cur)
    again = [g2.next_tokens(7) for _ in range(6)]
    assert all(torch.equal(a, b) for a, b in zip(after, again))
    assert g2.global_step == g.global_step and g.iterator.epoch >= 1
    with pytest.raises(ValueError, match="mismatch"):
        dl.DistributedDataGenerator(cfg, 0, 3).restore_cursor(cur)       # world size is pinned
    with pytest.raises(ValueError, match="mismatch"):
        dl.DistributedDataGenerator(dl.LoaderConfig(str(d), bos_token=999, seed=8), 0, 2).restore_cursor(cur)
    x, y = g.next_batch(2, 4)
    assert x.shape == (2, 4) and torch.equal(x.reshape(-1)[1:], y.reshape(-1)[:-1])


def test_resolve_paths(tmp_path):
    _make(tmp_path, "tr_0.bin", [4])
    _make(tmp_path, "tr_1.bin", [4])
    assert len(dl.resolve_shard_paths(str(tmp_path))) == 2
    assert len(dl.resolve_shard_paths(str(tmp_path / "tr_"))) == 2
    with pytest.raises(IOError):
        dl.resolve_shard_paths(str(tmp_path / "nothing"))
    z = dl.synthetic_zipf_tokens(1000, 65536)
    assert z.min() >= 0 and z.max() < 65536 and (z == 0).float().mean() > 0.05
