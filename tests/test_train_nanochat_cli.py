"""TrainNanoChat CLI on CPU: a run interrupted by a checkpoint and resumed reproduces the uninterrupted run."""
import json
import os

import torch

from tyr_b200.cli import train_nanochat as T
from tyr_b200.data import loader as dl
from tyr_b200.io import checkpoint as ckpt
from tyr_b200.train import run_ledger as rl


def _shards(tmp_path, n=2, tokens=40000):
    d = tmp_path / "data"
    d.mkdir()
    g = torch.Generator().manual_seed(0)
    for i in range(n):
        t = torch.randint(1, 4000, (tokens,), generator=g)
        t[::97] = 50256 % 4096
        dl.write_u16_bin(str(d / f"shard_{i:03d}.bin"), t)
    return str(d)


def test_resume_matches_uninterrupted_run(tmp_path, monkeypatch):
    monkeypatch.setenv("TYR_DEVICE", "cpu")
    data = _shards(tmp_path)
    common = ["--data", data, "--debug", "--seq-len", "64", "--device-batch-size", "2", "--total-batch-tokens", "128", "--log-every", "1"]
    a_dir, b_dir = str(tmp_path / "a"), str(tmp_path / "b")
    assert T.main(common + ["--checkpoint-dir", a_dir, "--iterations", "6"]) == 0
    assert T.main(common + ["--checkpoint-dir", b_dir, "--iterations", "3"]) == 0
    assert T.main(common + ["--checkpoint-dir", b_dir, "--iterations", "6", "--resume", b_dir]) == 0
    la = [r["metrics"]["loss"] for r in rl.read_events(os.path.join(a_dir, "metrics.jsonl")) if r["scope"] == "train"]
    lb = [r["metrics"]["loss"] for r in rl.read_events(os.path.join(b_dir, "metrics.jsonl")) if r["scope"] == "train"]
    assert len(la) == 6 and len(lb) == 6
    assert all(abs(x - y) < 1e-4 for x, y in zip(la, lb)), (la, lb)
    snap = ckpt.resolve_snapshot(os.path.join(b_dir, "checkpoints"))
    meta = json.load(open(os.path.join(snap, "meta.json")))
    assert meta["step"] == 6 and os.path.exists(os.path.join(snap, "optimizer.rank0.safetensors")) and os.path.exists(os.path.join(snap, "cursor.rank0.json"))
    cps = rl.read_events(os.path.join(b_dir, "checkpoints.jsonl"))
    assert [c["name"] for c in cps] == ["final", "final"]


def test_synthetic_mode_runs(tmp_path, monkeypatch):
    monkeypatch.setenv("TYR_DEVICE", "cpu")
    assert T.main(["--synthetic", "--debug", "--seq-len", "32", "--device-batch-size", "2", "--total-batch-tokens", "64", "--iterations", "2",
                   "--checkpoint-dir", str(tmp_path / "s"), "--eval-every", "1", "--eval-batches", "1"]) == 0
