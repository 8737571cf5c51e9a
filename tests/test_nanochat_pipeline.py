"""NanoChat recipe on CPU: environment parsing, parquet token stream cursors, and a whole quick pipeline on synthetic shards."""
import json
import os

import pyarrow as pa
import pyarrow.parquet as papq
import pytest
import torch

from tyr_b200 import pipeline as pl
from tyr_b200.nanochat import pipeline as np_
from tyr_b200.tokenizer.bpe import BPETokenizer


def _write_shards(d, n_files=3, docs=24):
    os.makedirs(d, exist_ok=True)
    words = ["tensor", "core", "memory", "bandwidth", "kernel", "stream", "graph", "token", "loss", "the", "a", "of", "and", "runs", "fast", "on"]
    g = torch.Generator().manual_seed(0)
    for f in range(n_files):
        texts = [" ".join(words[int(i)] for i in torch.randint(0, len(words), (40,), generator=g)) + "." for _ in range(docs)]
        papq.write_table(pa.table({"text": texts}), os.path.join(d, np_.shard_name(f)), row_group_size=8)


def test_env_defaults_overrides_and_validation():
    e = np_.load_env({})
    assert e.model.depth == 20 and e.pretrain.num_iterations == 21400 and e.pretrain.checkpoint_interval == 21400 and e.midtrain.val_interval == 150
    assert e.pipeline.wandb_enabled is False and e.pipeline.enable_rl is False and e.sft.target_examples_per_step == 32
    e = np_.load_env({"MODEL_DEPTH": "12", "PRETRAIN_VAL_INTERVAL": "0", "ENABLE_RL": "1", "WANDB_RUN": "exp7", "QUICK_MODE": "maybe", "GRPO_MAX_PROMPTS": "5"})
    assert e.model.depth == 12 and e.pretrain.val_interval is None and e.pipeline.enable_rl and e.pipeline.wandb_enabled and e.pipeline.quick_mode
    assert e.rl.max_prompts == 5
    with pytest.raises(ValueError, match="SFT_EPOCHS"):
        np_.load_env({"SFT_EPOCHS": "0"})
    cfg = np_.NanoChatConfig.from_env({"NANOCHAT_DIR": "/tmp/x", "MODEL_DEPTH": "20"})
    mc = cfg.to_model_config()
    assert (mc.n_layer, mc.n_head, mc.head_dim, mc.vocab_size) == (20, 10, 128, 65536)
    assert cfg.checkpoint_dir("base") == "/tmp/x/checkpoints/base" and cfg.tokenizer_path() == "/tmp/x/tokenizer"


def test_parquet_token_stream_cursor_resumes_exactly(tmp_path):
    d = str(tmp_path / "data")
    _write_shards(d)
    tok = BPETokenizer.byte_level()
    files = np_.parquet_files(d, "train")
    assert len(files) == 2 and len(np_.parquet_files(d, "val")) == 1
    a = np_.ParquetTokenStream(files, tok, 0, 2, 32, tokenizer_batch=5)
    for _ in range(3):
        a.next_batch()
    cur = np_.ParquetTokenStreamCursor.from_json(json.loads(json.dumps(a.capture_cursor().to_json())))
    want = [a.next_batch() for _ in range(260)]                       # runs through both files and wraps into a second epoch
    b = np_.ParquetTokenStream(files, tok, 0, 2, 32, tokenizer_batch=5)
    b.restore_cursor(cur)
    for x, y in want:
        bx, by = b.next_batch()
        assert torch.equal(x, bx) and torch.equal(y, by) and torch.equal(x.reshape(-1)[1:], y.reshape(-1)[:-1])
    assert a.cur.epoch >= 1
    r0 = np_.ParquetTokenStream(files, tok, 0, 2, 32, rank=0, world=2)
    r1 = np_.ParquetTokenStream(files, tok, 0, 2, 32, rank=1, world=2)
    assert r0.files != r1.files


def test_download_uses_injected_fetch_and_skips_present_shards(tmp_path):
    cfg = np_.NanoChatConfig(base_dir=str(tmp_path))
    os.makedirs(cfg.data_dir())
    open(os.path.join(cfg.data_dir(), np_.shard_name(0)), "w").close()
    asked = []

    def fetch(url, dest):
        asked.append(url)
        open(dest, "w").close()
        return True
    assert np_.download_data_shards(cfg, 3, fetch=fetch) == 3
    assert [u.rsplit("/", 1)[1] for u in asked] == [np_.shard_name(1), np_.shard_name(2)]


def test_quick_pipeline_runs_every_stage_and_resumes(tmp_path):
    base = str(tmp_path / "run")
    env = {"NANOCHAT_DIR": base, "MODEL_ASPECT_RATIO": "16", "MODEL_HEAD_DIM": "32", "MAX_SEQ_LEN": "64", "VOCAB_SIZE": "300", "PRETRAIN_ITERS": "2",
           "PRETRAIN_DEVICE_BATCH_SIZE": "2", "PRETRAIN_TOTAL_BATCH_SIZE": "128", "PRETRAIN_VAL_INTERVAL": "1", "PRETRAIN_LOG_INTERVAL": "1", "MIDTRAIN_ITERS": "2",
           "MIDTRAIN_DEVICE_BATCH_SIZE": "2", "MIDTRAIN_TOTAL_BATCH_SIZE": "128", "SFT_DEVICE_BATCH_SIZE": "2", "SFT_TARGET_EXAMPLES_PER_STEP": "2",
           "SFT_MAX_EXAMPLES": "6", "QUICK_MODE": "1"}
    cfg = np_.NanoChatConfig.from_env(env)
    cfg.device = "cpu"
    _write_shards(cfg.data_dir())
    lines = []
    from tyr_b200.utils.log import Handlers
    log = Handlers(on_info=lines.append, on_warn=lines.append, on_error=lines.append)
    pl.run_pipeline(cfg, lambda p: np_.run_quick_pipeline(p, cfg), log=log)
    assert cfg.env.model.depth == 4
    for stage in ("base", "mid", "sft"):
        assert os.path.exists(os.path.join(cfg.checkpoint_dir(stage), "CURRENT")), stage
    tok = np_.load_tokenizer(cfg)
    assert tok.vocab_size == 300 and tok.decode(tok.encode_ordinary("tensor core")) == "tensor core"
    assert any("[base] step 2/2" in l for l in lines) and any("Quick pipeline complete" in l for l in lines)
    # a second run finds every stage completed and skips the work
    lines.clear()
    pl.run_pipeline(cfg, lambda p: np_.run_quick_pipeline(p, cfg), log=log)
    assert not any("[base] step" in l for l in lines)
    # the evaluation stages work from the checkpoints that were written
    p = pl.Pipeline(cfg, log=log)
    ratios = np_.eval_tokenizer(p, cfg)
    assert ratios["fineweb"] > 1.5 and ratios["korean"] >= 1.0
    assert np_.eval_base_model(p, cfg) > 0.0
    acc = np_.eval_chat(p, cfg, "sft", max_problems=2)
    assert 0.0 <= acc <= 1.0
    # the chat CLI answers from the SFT checkpoint with the trained tokenizer
    from tyr_b200.cli import run_chat
    import io, contextlib
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        rc = run_chat.main(["--base-dir", base, "--stage", "sft", "--prompt", "2+2?", "--chat-markers", "--max-new-tokens", "6", "--temperature", "0",
                            "--show-tokens", "--device", "cpu"])
    assert rc == 0 and "[tokens]" in buf.getvalue()
    assert run_chat.main(["--base-dir", base, "--stage", "rl", "--prompt", "x", "--device", "cpu"]) == 1        # no such checkpoint yet
    # one GRPO update from the SFT checkpoint
    cfg.env.rl = np_.RLEnv(num_samples=2, max_new_tokens=4, examples_per_step_global=1, max_prompts=2)
    reward = np_.reinforcement_learning(p, cfg)
    assert 0.0 <= reward <= 1.0 and os.path.exists(os.path.join(cfg.checkpoint_dir("rl"), "CURRENT"))
