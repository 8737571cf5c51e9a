"""NanoChat end-to-end recipe: environment -> typed configuration, then the stages tokenizer training / evaluation,
data download, base pretraining, CORE evaluation, midtraining, chat evaluation, supervised fine-tuning and (optional)
GRPO, run through the pipeline orchestrator with per-stage checkpoints (Examples/NanoChat/Pipeline.lean).

Every stage works offline when its inputs are already on disk: parquet shards under ``<base>/<DATA_PATH>``, the CORE bundle
under ``<base>/eval_bundle``; network fetches go through an injectable ``fetch`` so tests run without a network.
"""
from __future__ import annotations

import glob
import json
import math
import os
import sys
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .. import pipeline as pl
from ..data import download as dl
from ..data import parquet as pq
from ..data import task as tk
from ..data import tasks as tks
from ..models import nanochat as nc
from ..rl import grpo
from ..tokenizer.bpe import BPETokenizer, train_bpe
from ..train import chat_sft
from ..train import nanochat_checkpoint as ckpt
from ..train.nanochat_engine import Hyperparameters, NanoChatTrainer
from ..train import run_ledger as rl_ledger
from ..utils.log import Handlers
from . import core_eval
from .generator import EngineConfig, SamplingConfig, SpecialTokens, session_runner
from .inference import NanoChatSession

SPECIAL_TOKENS = ["<|bos|>", "<|user_start|>", "<|user_end|>", "<|assistant_start|>", "<|assistant_end|>", "<|python_start|>",
                  "<|python_end|>", "<|output_start|>", "<|output_end|>"]
DATA_URL = "https://huggingface.co/datasets/karpathy/fineweb-edu-100b-shuffle/resolve/main"


# ---- environment -------------------------------------------------------------------------------------------------------
@dataclass
class ModelEnv:
    depth: int = 20
    aspect_ratio: int = 64
    target_head_dim: int = 128
    max_seq_len: int = 2048
    rope_base: float = 500000.0
    param_data_ratio: int = 20
    vocab_size: int = 65536
    tokenizer_max_chars: int = 2_000_000_000
    tokenizer_doc_cap: int = 10000


@dataclass
class PipelineEnv:
    base_dir: str = "~/.cache/nanochat"
    num_gpus: int = 1
    data_path: str = "base_data"
    num_data_shards: int = 240
    initial_data_shards: int = 8
    quick_mode: bool = False
    enable_rl: bool = False
    wandb_run: str = "dummy"
    wandb_enabled: bool = False


@dataclass
class PretrainEnv:
    data_path_override: Optional[str] = None
    num_iterations: int = 21400
    extension_iterations: int = 0
    val_interval: Optional[int] = 250
    log_interval: Optional[int] = 10
    device_batch_size: int = 32
    total_batch_size_tokens: int = 524288
    checkpoint_interval: Optional[int] = 21400
    text_column: str = "text"
    tokenizer_batch_size: int = 128
    eval_tokens: int = 10485760


@dataclass
class MidtrainEnv:
    num_iterations: int = 811
    extension_iterations: int = 0
    val_interval: Optional[int] = 150
    log_interval: Optional[int] = 10
    device_batch_size: int = 32
    total_batch_size_tokens: int = 524288
    checkpoint_interval: Optional[int] = 811
    eval_tokens: int = 10485760


@dataclass
class SFTEnv:
    num_epochs: int = 1
    device_batch_size: int = 4
    target_examples_per_step: int = 32
    max_examples: Optional[int] = None


@dataclass
class RLEnv:
    num_samples: int = 16
    max_new_tokens: int = 256
    examples_per_step_global: int = 16
    eval_every: int = 60
    log_every: int = 10
    epochs: int = 1
    max_prompts: Optional[int] = None


@dataclass
class EvalEnv:
    core_max_examples: Optional[int] = None
    identity_conversations_path: Optional[str] = None


@dataclass
class NanoChatEnv:
    pipeline: PipelineEnv = field(default_factory=PipelineEnv)
    model: ModelEnv = field(default_factory=ModelEnv)
    pretrain: PretrainEnv = field(default_factory=PretrainEnv)
    midtrain: MidtrainEnv = field(default_factory=MidtrainEnv)
    sft: SFTEnv = field(default_factory=SFTEnv)
    rl: RLEnv = field(default_factory=RLEnv)
    eval: EvalEnv = field(default_factory=EvalEnv)


def parse_bool(raw: str) -> Optional[bool]:
    v = raw.strip().lower()
    if v in ("1", "true", "yes", "on"):
        return True
    if v in ("0", "false", "no", "off"):
        return False
    return None


def load_env(env: Optional[Dict[str, str]] = None) -> NanoChatEnv:
    """Variable names and defaults of ``loadNanoChatEnvState`` (Pipeline.lean:302-426).  Intervals given as 0 disable
    the periodic action; positive-only settings reject 0."""
    env = os.environ if env is None else env

    def nat(name, default=None):
        raw = env.get(name)
        return int(raw) if raw is not None and raw.strip().isdigit() else default

    def pos(name, default):
        v = nat(name, default)
        if v is None or v <= 0:
            raise ValueError(f"{name} must be a positive integer")
        return v

    def interval(name, default):
        v = nat(name)
        return default if v is None else (v if v > 0 else None)

    def flag(name):
        raw = env.get(name)
        if raw is None:
            return None
        b = parse_bool(raw)
        return True if b is None else b            # set but unparsable counts as set

    pre_iters, mid_iters = nat("PRETRAIN_ITERS", 21400), nat("MIDTRAIN_ITERS", 811)
    wandb_run = env.get("WANDB_RUN", "dummy")
    we = flag("WANDB_ENABLED")
    return NanoChatEnv(
        PipelineEnv(env.get("NANOCHAT_DIR", "~/.cache/nanochat"), nat("WORLD_SIZE", 1), env.get("DATA_PATH", "base_data"), nat("NUM_SHARDS", 240),
                    nat("INITIAL_DATA_SHARDS", 8), bool(flag("QUICK_MODE")), bool(flag("ENABLE_RL")), wandb_run, we if we is not None else wandb_run != "dummy"),
        ModelEnv(nat("MODEL_DEPTH", 20), nat("MODEL_ASPECT_RATIO", 64), nat("MODEL_HEAD_DIM", 128), nat("MAX_SEQ_LEN", 2048),
                 float(nat("ROPE_BASE", 500000)), nat("PARAM_DATA_RATIO", 20), nat("VOCAB_SIZE", 65536), nat("TOKENIZER_MAX_CHARS", 2_000_000_000),
                 nat("TOKENIZER_DOC_CAP", 10000)),
        PretrainEnv(env.get("PRETRAIN_DATA_PATH"), pre_iters, nat("PRETRAIN_EXTENSION_ITERS", 0), interval("PRETRAIN_VAL_INTERVAL", 250),
                    interval("PRETRAIN_LOG_INTERVAL", 10), nat("PRETRAIN_DEVICE_BATCH_SIZE", 32), nat("PRETRAIN_TOTAL_BATCH_SIZE", 524288),
                    interval("PRETRAIN_CHECKPOINT_INTERVAL", pre_iters if pre_iters > 0 else None), env.get("PRETRAIN_TEXT_COLUMN", "text"),
                    nat("PRETRAIN_TOKENIZER_BATCH_SIZE", 128), nat("PRETRAIN_EVAL_TOKENS", 10485760)),
        MidtrainEnv(mid_iters, nat("MIDTRAIN_EXTENSION_ITERS", 0), interval("MIDTRAIN_VAL_INTERVAL", 150), interval("MIDTRAIN_LOG_INTERVAL", 10),
                    nat("MIDTRAIN_DEVICE_BATCH_SIZE", 32), nat("MIDTRAIN_TOTAL_BATCH_SIZE", 524288),
                    interval("MIDTRAIN_CHECKPOINT_INTERVAL", mid_iters if mid_iters > 0 else None), nat("MIDTRAIN_EVAL_TOKENS", 10485760)),
        SFTEnv(pos("SFT_EPOCHS", 1), pos("SFT_DEVICE_BATCH_SIZE", 4), pos("SFT_TARGET_EXAMPLES_PER_STEP", 32), nat("SFT_MAX_EXAMPLES")),
        RLEnv(pos("GRPO_NUM_SAMPLES", 16), pos("GRPO_MAX_NEW_TOKENS", 256), pos("GRPO_EXAMPLES_PER_STEP", 16), pos("GRPO_EVAL_EVERY", 60),
              pos("GRPO_LOG_EVERY", 10), pos("GRPO_EPOCHS", 1), nat("GRPO_MAX_PROMPTS")),
        EvalEnv(nat("CORE_MAX_EXAMPLES"), env.get("IDENTITY_CONVERSATIONS_PATH")))


@dataclass
class NanoChatConfig(pl.PipelineConfig):
    env: NanoChatEnv = field(default_factory=NanoChatEnv)
    data_url: str = DATA_URL
    max_download_retries: int = 5
    sft_embedding_lr: float = 0.2
    sft_matrix_lr: float = 0.02
    device: str = "cuda" if torch.cuda.is_available() else "cpu"

    @staticmethod
    def from_env(env: Optional[Dict[str, str]] = None) -> "NanoChatConfig":
        e = load_env(env)
        return NanoChatConfig(base_dir=e.pipeline.base_dir, wandb_enabled=e.pipeline.wandb_enabled, wandb_run=e.pipeline.wandb_run,
                              num_gpus=e.pipeline.num_gpus, env=e)

    def to_model_config(self) -> nc.Config:
        m = self.env.model
        if m.vocab_size <= 0:
            raise ValueError("VOCAB_SIZE must be positive")
        if m.max_seq_len <= 0:
            raise ValueError("MAX_SEQ_LEN must be positive")
        return nc.depth_config(m.depth, m.aspect_ratio, m.target_head_dim, m.vocab_size, m.max_seq_len, m.rope_base)

    def data_dir(self) -> str:
        o = self.env.pretrain.data_path_override
        return os.path.expanduser(o) if o else os.path.join(self.resolved_base_dir(), self.env.pipeline.data_path)

    def tokenizer_path(self) -> str:
        return os.path.join(self.resolved_base_dir(), "tokenizer")

    def checkpoint_dir(self, stage: str) -> str:
        return os.path.join(self.resolved_base_dir(), "checkpoints", stage)


# ---- data ----------------------------------------------------------------------------------------------------------------
def shard_name(index: int) -> str:
    return f"shard_{index:05d}.parquet"


def download_data_shards(cfg: NanoChatConfig, num_shards: int, log: Optional[Handlers] = None, fetch=None) -> int:
    """Fetch shards ``0 .. num_shards-1`` that are not on disk yet; returns how many are present afterwards."""
    d = cfg.data_dir()
    os.makedirs(d, exist_ok=True)
    have = 0
    for i in range(num_shards):
        dest = os.path.join(d, shard_name(i))
        if os.path.exists(dest) or dl.download_with_retry(f"{cfg.data_url}/{shard_name(i)}", dest, cfg.max_download_retries, log=log, fetch=fetch):
            have += 1
    return have


def parquet_files(data_dir: str, split: str = "train") -> List[str]:
    """All shards but the last train; the last one validates (a single shard serves both)."""
    files = sorted(glob.glob(os.path.join(data_dir, "*.parquet")))
    if len(files) <= 1:
        return files
    return files[:-1] if split == "train" else files[-1:]


def load_parquet_texts(data_dir: str, max_chars: int, doc_cap: int = 10000, column: str = "text") -> List[str]:
    out, seen = [], 0
    for f in parquet_files(data_dir, "train"):
        for g in range(pq.num_row_groups(f)):
            for t in pq.read_text_column(f, g, column):
                t = t[:doc_cap]
                out.append(t)
                seen += len(t)
                if seen >= max_chars:
                    return out
    return out


@dataclass
class ParquetTokenStreamCursor:
    file_index: int = 0
    row_group: int = 0
    doc_in_group: int = 0
    buffer: List[int] = field(default_factory=list)
    epoch: int = 0

    def to_json(self) -> dict:
        return {"fileIndex": self.file_index, "rowGroup": self.row_group, "docInGroup": self.doc_in_group, "buffer": self.buffer, "epoch": self.epoch}

    @staticmethod
    def from_json(j: dict) -> "ParquetTokenStreamCursor":
        return ParquetTokenStreamCursor(j["fileIndex"], j["rowGroup"], j["docInGroup"], list(j["buffer"]), j.get("epoch", 0))


class ParquetTokenStream:
    """Documents of the rank's files -> ``bos + tokens`` appended to a buffer -> ``[B, T]`` input / target windows.
    Files are dealt to ranks round-robin; the cursor (file, row group, document, pending tokens) makes a resumed run
    read exactly the tokens the interrupted run would have read next (Pipeline.lean:815-973)."""

    def __init__(self, files: Sequence[str], tokenizer: BPETokenizer, bos: int, batch: int, seq: int, rank: int = 0, world: int = 1,
                 column: str = "text", tokenizer_batch: int = 128):
        self.files = [f for i, f in enumerate(files) if i % max(1, world) == rank] or list(files)
        if not self.files:
            raise ValueError("parquet token stream: no input files")
        self.tok, self.bos, self.batch, self.seq, self.column, self.tok_batch = tokenizer, bos, batch, seq, column, tokenizer_batch
        self.cur = ParquetTokenStreamCursor()
        self._docs: Optional[List[str]] = None

    def capture_cursor(self) -> ParquetTokenStreamCursor:
        c = self.cur
        return ParquetTokenStreamCursor(c.file_index, c.row_group, c.doc_in_group, list(c.buffer), c.epoch)

    def restore_cursor(self, c: ParquetTokenStreamCursor) -> None:
        self.cur = ParquetTokenStreamCursor(c.file_index % len(self.files), c.row_group, c.doc_in_group, list(c.buffer), c.epoch)
        self._docs = None

    def _fill(self, need: int) -> None:
        c = self.cur
        while len(c.buffer) < need:
            if self._docs is None:
                f = self.files[c.file_index]
                if c.row_group >= pq.num_row_groups(f):
                    c.file_index, c.row_group, c.doc_in_group = c.file_index + 1, 0, 0
                    if c.file_index >= len(self.files):
                        c.file_index, c.epoch = 0, c.epoch + 1
                    continue
                self._docs = pq.read_text_column(f, c.row_group, self.column)
            take = self._docs[c.doc_in_group:c.doc_in_group + self.tok_batch]
            if not take:
                c.row_group, c.doc_in_group, self._docs = c.row_group + 1, 0, None
                continue
            for d in take:
                c.buffer.append(self.bos)
                c.buffer.extend(self.tok.encode_ordinary(d))
            c.doc_in_group += len(take)

    def next_batch(self) -> Tuple[torch.Tensor, torch.Tensor]:
        need = self.batch * self.seq + 1
        self._fill(need)
        w = torch.tensor(self.cur.buffer[:need], dtype=torch.int64)
        del self.cur.buffer[:need - 1]
        return w[:-1].reshape(self.batch, self.seq), w[1:].reshape(self.batch, self.seq)


# ---- tokenizer stages --------------------------------------------------------------------------------------------------------
def load_tokenizer(cfg: NanoChatConfig) -> BPETokenizer:
    return BPETokenizer.load(os.path.join(cfg.tokenizer_path(), "tokenizer.bin"))


def chat_tokens(tok: BPETokenizer) -> tk.ChatTokens:
    s = tok.encode_special
    return tk.ChatTokens(s("<|bos|>"), s("<|user_start|>"), s("<|user_end|>"), s("<|assistant_start|>"), s("<|assistant_end|>"),
                         s("<|python_start|>"), s("<|python_end|>"), output_start=s("<|output_start|>"), output_end=s("<|output_end|>"))


def train_tokenizer(p: pl.Pipeline, cfg: NanoChatConfig) -> None:
    if not p.is_master:
        return
    m = cfg.env.model
    texts = load_parquet_texts(cfg.data_dir(), m.tokenizer_max_chars, m.tokenizer_doc_cap, cfg.env.pretrain.text_column)
    if not texts:
        raise RuntimeError(f"no training text under {cfg.data_dir()}")
    tok = train_bpe(texts, m.vocab_size, SPECIAL_TOKENS, doc_cap=m.tokenizer_doc_cap, max_chars=m.tokenizer_max_chars)
    os.makedirs(cfg.tokenizer_path(), exist_ok=True)
    tok.save(os.path.join(cfg.tokenizer_path(), "tokenizer.bin"))
    tb = torch.tensor(tok.token_bytes(), dtype=torch.int32)
    torch.save(tb, os.path.join(cfg.tokenizer_path(), "token_bytes.pt"))
    p.record_metrics([("tokenizer_vocab", str(tok.vocab_size)), ("tokenizer_docs", str(len(texts)))])
    p.log(f"tokenizer: {tok.vocab_size} tokens from {len(texts)} documents")


EVAL_SNIPPETS = {
    "news": "The central bank said on Tuesday that it would keep interest rates unchanged, citing slower growth and easing inflation across the region.",
    "code": "def fib(n):\n    a, b = 0, 1\n    for _ in range(n):\n        a, b = b, a + b\n    return a\n",
    "math": "Let x = 3/4 and y = 5/6. Then x + y = 9/12 + 10/12 = 19/12, so 12(x + y) = 19.",
    "korean": "안녕하세요. 오늘 날씨가 정말 좋네요. 같이 산책하러 갈까요?",
}


def eval_tokenizer(p: pl.Pipeline, cfg: NanoChatConfig) -> Dict[str, float]:
    """Bytes per token on fixed snippets plus held-out training text, against the byte-level floor of 1.0."""
    if not p.is_master:
        return {}
    tok = load_tokenizer(cfg)
    samples = dict(EVAL_SNIPPETS)
    held = load_parquet_texts(cfg.data_dir(), 200_000, cfg.env.model.tokenizer_doc_cap, cfg.env.pretrain.text_column)
    if held:
        samples["fineweb"] = "\n".join(held[-8:])
    ratios = {}
    for name, text in samples.items():
        ids = tok.encode_ordinary(text)
        if tok.decode(ids) != text:
            raise RuntimeError(f"tokenizer round trip failed on the {name} sample")
        ratios[name] = len(text.encode("utf-8")) / max(1, len(ids))
    p.record_metrics([(f"bytes_per_token_{k}", f"{v:.3f}") for k, v in ratios.items()])
    return ratios


# ---- model stages ----------------------------------------------------------------------------------------------------------------
def _hyper(cfg: NanoChatConfig, e, world: int) -> Hyperparameters:
    seq = cfg.env.model.max_seq_len
    total = e.total_batch_size_tokens
    per_pass = e.device_batch_size * seq * world
    if total % per_pass:
        total = max(per_pass, total // per_pass * per_pass)           # keep accumulation whole (ModdedTrain.lean:159-165)
    return Hyperparameters(num_iterations=e.num_iterations, extension_iterations=e.extension_iterations, device_batch_size=e.device_batch_size,
                           total_batch_size_tokens=total, max_seq_len=seq, val_interval=e.val_interval or 0, log_interval=e.log_interval or 0,
                           checkpoint_interval=e.checkpoint_interval or 0)


def _compute_dtype(device: str):
    return torch.bfloat16 if str(device).startswith("cuda") else torch.float32


def _train_on_stream(p: pl.Pipeline, cfg: NanoChatConfig, trainer: NanoChatTrainer, next_batch: Callable[[], Tuple[torch.Tensor, torch.Tensor]],
                     val_batch: Optional[Callable[[], Tuple[torch.Tensor, torch.Tensor]]], stage: str, cursor_json: Callable[[], dict]) -> float:
    """The shared loop of pretraining and midtraining: accumulate, step, log, validate, checkpoint."""
    hp, dev = trainer.hp, trainer.device
    accum = max(1, hp.total_batch_size_tokens // (hp.device_batch_size * hp.max_seq_len * max(1, p.world_size)))
    out_dir = cfg.checkpoint_dir(stage)
    total = hp.num_iterations + hp.extension_iterations
    loss = float("nan")
    while trainer.step_index < total:
        micro = [tuple(t.to(dev) for t in next_batch()) for _ in range(accum)]
        loss = float(trainer.step(micro).loss)
        s = trainer.step_index
        if hp.log_interval and s % hp.log_interval == 0:
            p.log(f"[{stage}] step {s}/{total} loss {loss:.4f}")
        if val_batch is not None and hp.val_interval and s % hp.val_interval == 0:
            p.log(f"[{stage}] step {s} val loss {evaluate_loss(trainer, val_batch, 2):.4f}")
        if (hp.checkpoint_interval and s % hp.checkpoint_interval == 0) or s == total:
            ckpt.save(out_dir, trainer, None, loss, extra={"cursor": cursor_json(), "stage": stage})
    p.record_metrics([(f"{stage}_final_loss", f"{loss:.4f}"), (f"{stage}_steps", str(trainer.step_index))])
    return loss


@torch.no_grad()
def evaluate_loss(trainer: NanoChatTrainer, val_batch, batches: int) -> float:
    cos, sin = nc_tables(trainer)
    tot = 0.0
    params = trainer.params.named_parameters("work")
    for _ in range(batches):
        x, y = (t.to(trainer.device) for t in val_batch())
        tot += float(nc.loss_reference(params, trainer.cfg, x, y, cos, sin))
    return tot / max(1, batches)


def nc_tables(trainer: NanoChatTrainer):
    from ..ops.rope import rotary_freqs
    return rotary_freqs(trainer.cfg.max_seq_len, trainer.cfg.head_dim, trainer.cfg.rope_base, trainer.device)


def _new_trainer(p: pl.Pipeline, cfg: NanoChatConfig, e, init_from: Optional[str]) -> NanoChatTrainer:
    tr = NanoChatTrainer(cfg.to_model_config(), _hyper(cfg, e, p.world_size), device=cfg.device, compute_dtype=_compute_dtype(cfg.device),
                         world_size=1, rank=0)
    if init_from and os.path.isdir(init_from):
        ckpt.load(init_from, tr, None, weights_only=True)
        tr.step_index = 0
    return tr


def pretrain_base_model(p: pl.Pipeline, cfg: NanoChatConfig) -> float:
    e = cfg.env.pretrain
    tok = load_tokenizer(cfg)
    bos = tok.encode_special("<|bos|>")
    seq = cfg.env.model.max_seq_len
    train = ParquetTokenStream(parquet_files(cfg.data_dir(), "train"), tok, bos, e.device_batch_size, seq, p.rank, p.world_size, e.text_column, e.tokenizer_batch_size)
    val = ParquetTokenStream(parquet_files(cfg.data_dir(), "val"), tok, bos, e.device_batch_size, seq, 0, 1, e.text_column, e.tokenizer_batch_size)
    tr = _new_trainer(p, cfg, e, None)
    out = cfg.checkpoint_dir("base")
    if os.path.exists(os.path.join(out, "CURRENT")) or os.path.exists(os.path.join(out, "meta.json")):
        meta = ckpt.load(out, tr, None)
        cur = (meta.get("extra") or {}).get("cursor")
        if cur:
            train.restore_cursor(ParquetTokenStreamCursor.from_json(cur))
        p.log(f"[base] resumed at step {tr.step_index}")
    return _train_on_stream(p, cfg, tr, train.next_batch, val.next_batch, "base", lambda: train.capture_cursor().to_json())


def model_fn(trainer: NanoChatTrainer):
    cos, sin = nc_tables(trainer)
    params = trainer.params.named_parameters("work")
    return lambda ids: nc.forward_reference(params, trainer.cfg, ids, cos, sin)


def eval_base_model(p: pl.Pipeline, cfg: NanoChatConfig) -> Optional[float]:
    """CORE over the bundle under ``<base>/eval_bundle`` when present; held-out loss otherwise."""
    if not p.is_master:
        return None
    tr = _new_trainer(p, cfg, cfg.env.pretrain, cfg.checkpoint_dir("base"))
    tok = load_tokenizer(cfg)
    bundle = os.path.join(cfg.resolved_base_dir(), "eval_bundle")
    if os.path.isdir(bundle):
        ec = core_eval.EvalConfig(max_examples=cfg.env.eval.core_max_examples or 0, bos_token=tok.encode_special("<|bos|>"), max_seq_len=cfg.env.model.max_seq_len)
        with torch.no_grad():
            core, per_task = core_eval.evaluate_core(model_fn(tr), tok.encode_ordinary, bundle, ec, device=tr.device, log=p.log)
        p.record_metrics([(f"core_{n}", f"{a:.4f}") for n, a in per_task])
        p.record_metrics([("core_metric", f"{core:.4f}")])
        return core
    e = cfg.env.pretrain
    val = ParquetTokenStream(parquet_files(cfg.data_dir(), "val"), tok, tok.encode_special("<|bos|>"), e.device_batch_size, cfg.env.model.max_seq_len)
    loss = evaluate_loss(tr, val.next_batch, 2)
    p.record_metrics([("base_val_loss", f"{loss:.4f}")])
    return loss


def _conversation_mixture(cfg: NanoChatConfig, kind: str) -> tk.ConversationMixture:
    mix = tks.create_midtraining_mixture("nanochat") if kind == "mid" else tks.create_sft_mixture("nanochat")
    path = cfg.env.eval.identity_conversations_path
    cm = mix.to_conversation_mixture()
    if path and os.path.exists(path):
        extra = [tk.Conversation([tk.Message(m["role"], m["content"]) for m in row]) for row in tks.load_jsonl_from_file(path) if isinstance(row, list)]
        cm = tk.ConversationMixture(cm.conversations + extra, cm.seed)
    return cm


def midtrain(p: pl.Pipeline, cfg: NanoChatConfig) -> float:
    e = cfg.env.midtrain
    tok = load_tokenizer(cfg)
    stream = tk.TaskTokenStream(_conversation_mixture(cfg, "mid"), e.device_batch_size, cfg.env.model.max_seq_len, chat_tokens(tok), tok.encode_ordinary,
                                p.rank, p.world_size)
    tr = _new_trainer(p, cfg, e, cfg.checkpoint_dir("base"))
    return _train_on_stream(p, cfg, tr, stream.next_gpt_batch, None, "mid", lambda: {"cursor": stream.cursor, "steps": stream.steps})


def _sft_forward(trainer: NanoChatTrainer):
    cos, sin = nc_tables(trainer)
    return lambda params, ids: nc.forward_reference(params, trainer.cfg, ids, cos, sin)


def supervised_fine_tune(p: pl.Pipeline, cfg: NanoChatConfig) -> float:
    e = cfg.env.sft
    tok = load_tokenizer(cfg)
    tr = _new_trainer(p, cfg, cfg.env.midtrain, cfg.checkpoint_dir("mid"))
    cm = _conversation_mixture(cfg, "sft")
    if e.max_examples is not None:
        cm = tk.ConversationMixture(cm.conversations[:e.max_examples], cm.seed)
    it = tk.TaskIterator(cm, e.device_batch_size, cfg.env.model.max_seq_len, chat_tokens(tok), tok.encode_ordinary)
    sc = chat_sft.SFTConfig(num_epochs=e.num_epochs, device_batch_size=e.device_batch_size, target_examples_per_step=e.target_examples_per_step,
                            embedding_lr=cfg.sft_embedding_lr, matrix_lr=cfg.sft_matrix_lr, device=str(tr.device), log_interval=1)
    params = {k: v.detach().float().clone() for k, v in tr.params.named_parameters("master").items()}
    arts = rl_ledger.RunArtifacts.of_base_dir(os.path.join(cfg.resolved_base_dir(), "runs", "sft"))
    rl_ledger.prepare(arts, {"stage": "sft"}, rl_ledger.ExistingRunPolicy.overwrite)
    cb = chat_sft.Callbacks(on_train_step=lambda s, l, m, n: p.log(chat_sft.format_train_update(s, l, m, n))).combine(chat_sft.artifact_callbacks(arts))
    new_params, _, state = chat_sft.train_sft(sc, params, _sft_forward(tr), it, callbacks=cb)
    tr.params.load_named({k: v.detach() for k, v in new_params.items()})
    tr.params.sync_work_from_master()
    ckpt.save(cfg.checkpoint_dir("sft"), tr, None, state.running_loss / max(1, state.step), extra={"stage": "sft"})
    p.record_metrics([("sft_steps", str(state.step)), ("sft_tokens", str(state.total_tokens))])
    return state.running_loss / max(1, state.step)


def make_generate_one(trainer: NanoChatTrainer, tok: BPETokenizer, temperature: Optional[float] = None) -> grpo.GenerateOneFn:
    """``(prompt ids, generation config, seed) -> response ids`` on the row-state engine with the calculator tool."""
    ct = chat_tokens(tok)
    specials = SpecialTokens(eot=ct.assistant_end, bot=ct.bos, tool_start=ct.python_start, tool_end=ct.python_end,
                             output_start=ct.output_start, output_end=ct.output_end, calc_start=ct.python_start, calc_end=ct.python_end)

    def gen(prompt: List[int], gc: grpo.GenerationConfig, seed: int) -> List[int]:
        prompt = list(prompt)
        room = trainer.cfg.max_seq_len - len(prompt) - 1
        if room <= 0:
            return []
        engine = EngineConfig(temperature=gc.temperature if temperature is None else temperature, top_k=gc.top_k,
                              max_tokens=min(gc.max_new_tokens, room)).create(specials)
        params = {k: v.detach() for k, v in trainer.params.named_parameters("work").items()}
        sess = NanoChatSession(params, trainer.cfg, 1, trainer.cfg.max_seq_len)
        if len(prompt) > 1:
            sess.prefill(torch.tensor([prompt[:-1]], device=trainer.device))
        out = engine.generate_one(prompt, session_runner(sess), tok.decode, tok.encode_ordinary, generator=torch.Generator().manual_seed(seed))
        return out[len(prompt):]
    return gen


def _message_text(m: tk.Message) -> str:
    return m.content if m.content else "".join(part.content for part in m.parts)


def eval_chat(p: pl.Pipeline, cfg: NanoChatConfig, checkpoint: str, max_problems: int = 16) -> Optional[float]:
    """Greedy answers to held-out arithmetic prompts, scored with the GSM8K-style ``####`` reward."""
    if not p.is_master:
        return None
    tok = load_tokenizer(cfg)
    tr = _new_trainer(p, cfg, cfg.env.midtrain, cfg.checkpoint_dir(checkpoint))
    gen, gconf = make_generate_one(tr, tok, temperature=0.0), grpo.GenerationConfig(max_new_tokens=48)
    task = tks.create_math_task()
    n = min(max_problems, task.size())
    ct = chat_tokens(tok)
    hits = 0.0
    for i in range(n):
        conv = task.get(i)
        prompt = tk.render_conversation(tk.Conversation(conv.messages[:-1]), ct, tok.encode_ordinary).tokens + [ct.assistant_start]
        expected = tks.extract_hash_answer(_message_text(conv.messages[-1])) or ""
        hits += grpo.math_reward(expected, tok.decode(gen(prompt, gconf, i))).reward
    acc = hits / max(1, n)
    p.record_metrics([(f"chat_{checkpoint}_math_acc", f"{acc:.3f}")])
    return acc


def reinforcement_learning(p: pl.Pipeline, cfg: NanoChatConfig) -> float:
    e = cfg.env.rl
    tok = load_tokenizer(cfg)
    tr = _new_trainer(p, cfg, cfg.env.midtrain, cfg.checkpoint_dir("sft"))
    task = tks.create_math_task()
    n = task.size() if e.max_prompts is None else min(task.size(), e.max_prompts)
    ct = chat_tokens(tok)
    prompts = []
    for i in range(n):
        conv = task.get(i)
        text = tok.decode(tk.render_conversation(tk.Conversation(conv.messages[:-1]), ct, tok.encode_ordinary).tokens + [ct.assistant_start])
        prompts.append((text, tks.extract_hash_answer(_message_text(conv.messages[-1])) or ""))
    gc = grpo.GRPOConfig(num_samples=e.num_samples, max_new_tokens=e.max_new_tokens, examples_per_step=e.examples_per_step_global,
                         eval_every=e.eval_every, log_every=e.log_every, top_k=50, pad_token=ct.assistant_end, eos_token=ct.assistant_end)
    params = {k: v.detach().float().clone() for k, v in tr.params.named_parameters("master").items()}
    fwd = _sft_forward(tr)

    def make_gen(cur_params):
        tr.params.load_named({k: v.detach() for k, v in cur_params.items()})
        tr.params.sync_work_from_master()
        return make_generate_one(tr, tok)
    steps = max(1, (len(prompts) // max(1, gc.examples_per_step)) * e.epochs)
    res = grpo.train_on_prompts_with_updates(gc, params, fwd, make_gen, lambda s: tok.encode(s), tok.decode, prompts, steps, device=str(tr.device),
                                             callbacks=grpo.Callbacks(on_train_step=lambda r, st: p.log(grpo.format_train_update(r, st))))
    tr.params.load_named({k: v.detach() for k, v in res.params.items()})
    tr.params.sync_work_from_master()
    ckpt.save(cfg.checkpoint_dir("rl"), tr, None, 0.0, extra={"stage": "rl"})
    mean_reward = sum(h.mean_reward for h in res.history) / max(1, len(res.history))
    p.record_metrics([("rl_steps", str(steps)), ("rl_mean_reward", f"{mean_reward:.4f}")])
    return mean_reward


# ---- composition ---------------------------------------------------------------------------------------------------------------
BANNER = r"""
   _   _                    ____ _           _
  | \ | | __ _ _ __   ___  / ___| |__   __ _| |_     one-node B200 recipe
  |  \| |/ _` | '_ \ / _ \| |   | '_ \ / _` | __|
  | |\  | (_| | | | | (_) | |___| | | | (_| | |_
  |_| \_|\__,_|_| |_|\___/ \____|_| |_|\__,_|\__|
"""


def estimate_cost(gpu_type: str, num_gpus: int, hours: float) -> float:
    rate = {"H100": 3.0, "A100": 1.8, "B200": 6.0}.get(gpu_type, 3.0)
    return rate * num_gpus * hours


def run_nanochat_pipeline(p: pl.Pipeline, cfg: NanoChatConfig, fetch=None) -> None:
    pe = cfg.env.pipeline
    p.log(BANNER)
    p.log(f"Model: d{cfg.env.model.depth}, vocab: {cfg.env.model.vocab_size}; base directory: {cfg.resolved_base_dir()}")
    p.stage("data-download-initial", lambda: p.master_only(lambda: download_data_shards(cfg, pe.initial_data_shards, fetch=fetch), 0))
    more = p.background("download-remaining-shards", lambda: p.master_only(lambda: download_data_shards(cfg, pe.num_data_shards, fetch=fetch), 0))
    p.stage("tokenizer-training", lambda: train_tokenizer(p, cfg))
    p.stage("tokenizer-eval", lambda: eval_tokenizer(p, cfg))

    def all_data():
        p.await_task(more)
        p.sync_barrier()
        p.log(f"All {pe.num_data_shards} data shards ready")
    p.stage("data-download-complete", all_data)
    p.stage("pretrain", lambda: pretrain_base_model(p, cfg))
    p.stage("pretrain-eval", lambda: eval_base_model(p, cfg))
    p.stage("midtrain", lambda: midtrain(p, cfg))
    p.stage("midtrain-eval", lambda: eval_chat(p, cfg, "mid"))
    p.stage("sft", lambda: supervised_fine_tune(p, cfg))
    p.stage("sft-eval", lambda: eval_chat(p, cfg, "sft"))
    if pe.enable_rl:
        p.stage("rl", lambda: reinforcement_learning(p, cfg))
        p.stage("rl-eval", lambda: eval_chat(p, cfg, "rl"))
    else:
        p.log("RL stage disabled (set ENABLE_RL=1 to enable)")
    p.log("Pipeline complete!")


def run_quick_pipeline(p: pl.Pipeline, cfg: NanoChatConfig) -> None:
    """Depth 4, existing data only (Pipeline.lean:2024-2048)."""
    p.log("Running QUICK pipeline (testing mode)...")
    cfg.env.model.depth = 4
    p.stage("tokenizer-training", lambda: train_tokenizer(p, cfg))
    p.stage("pretrain", lambda: pretrain_base_model(p, cfg))
    p.stage("midtrain", lambda: midtrain(p, cfg))
    p.stage("sft", lambda: supervised_fine_tune(p, cfg))
    p.log("Quick pipeline complete!")


def main(argv=None) -> int:
    cfg = NanoChatConfig.from_env()
    body = (lambda p: run_quick_pipeline(p, cfg)) if cfg.env.pipeline.quick_mode else (lambda p: run_nanochat_pipeline(p, cfg))
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        pl.with_distributed(cfg, body)
    else:
        pl.run_pipeline(cfg, body)
    return 0


if __name__ == "__main__":
    sys.exit(main())
