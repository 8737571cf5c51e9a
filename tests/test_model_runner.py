"""Shared runner helpers: device selection, prompt files, batching, padding, and a Gemma 4 round trip from a local directory."""
import json
import os

import pytest
import torch

from tyr_b200.cli import model_runner as R


def test_device_selection_falls_back_with_warnings():
    assert R.resolve_device("cpu") == (torch.device("cpu"), None)
    d, w = R.resolve_device("tpu")
    assert d.type == "cpu" and "invalid device selector" in w
    d, w = R.resolve_device("cuda:x")
    assert d.type == "cpu" and "invalid" in w
    if not torch.cuda.is_available():
        d, w = R.resolve_device("cuda:1")
        assert d.type == "cpu" and "CUDA is unavailable" in w
        assert R.resolve_device("auto")[0].type == "cpu"


def test_prompts_batches_and_padding(tmp_path):
    f = tmp_path / "p.txt"
    f.write_text("one\n\n two \nthree\n")
    assert R.load_prompts(str(f), "x") == ["one", "two", "three"] and R.load_prompts(None, "x") == ["x"]
    (tmp_path / "e.txt").write_text("\n\n")
    with pytest.raises(ValueError, match="no non-empty"):
        R.load_prompts(str(tmp_path / "e.txt"), "x")
    assert list(R.batches([1, 2, 3, 4, 5], 2)) == [[1, 2], [3, 4], [5]]
    assert R.left_pad([[1, 2, 3], [4]], 9).tolist() == [[1, 2, 3], [9, 9, 4]]


def test_speech_family_requires_audio(capsys):
    assert R.main(["--family", "whisper", "--source", "/nonexistent", "--device", "cpu"]) == 2
