"""Pipeline orchestrator: named stages with retry, resume from ``.pipeline_checkpoint.json``, background tasks,
a markdown report and rank-aware logging (Tyr/Pipeline.lean).

A stage that completed in an earlier run with the same configuration is skipped; a failed stage is retried.
Ranks agree on health through a barrier plus an all-reduced failure flag, all on the host.
"""
from __future__ import annotations

import concurrent.futures as cf
import json
import os
import time
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple, TypeVar

from . import distributed as tdist
from .utils.log import Handlers
from .utils.timer import mono_ms

T = TypeVar("T")


@dataclass
class RetryPolicy:
    max_attempts: int = 3
    initial_delay_ms: int = 1000
    backoff_multiplier: float = 2.0
    max_delay_ms: int = 60000

    def delay_for_attempt(self, attempt: int) -> int:
        return min(self.max_delay_ms, int(self.initial_delay_ms * (self.backoff_multiplier ** attempt)))


@dataclass
class StageInfo:
    name: str
    status: str = "pending"            # pending | running | completed | failed | skipped
    error: Optional[str] = None
    start_time: Optional[int] = None
    end_time: Optional[int] = None
    metrics: List[Tuple[str, str]] = field(default_factory=list)

    def duration_ms(self) -> Optional[int]:
        return None if self.start_time is None or self.end_time is None else self.end_time - self.start_time

    def to_json(self) -> dict:
        return {"name": self.name, "status": self.status if self.status != "failed" else {"failed": self.error or ""},
                "startTime": self.start_time, "endTime": self.end_time, "metrics": [list(m) for m in self.metrics]}

    @staticmethod
    def from_json(j: dict) -> "StageInfo":
        st = j.get("status", "pending")
        err = None
        if isinstance(st, dict):
            err, st = st.get("failed", ""), "failed"
        return StageInfo(j["name"], st, err, j.get("startTime"), j.get("endTime"), [tuple(m) for m in j.get("metrics", [])])


def format_duration(ms: int) -> str:
    s = ms / 1000.0
    if s < 60:
        return f"{s:.1f}s"
    m, s = divmod(int(s), 60)
    if m < 60:
        return f"{m}m {s}s"
    h, m = divmod(m, 60)
    return f"{h}h {m}m"


class BackgroundTask:
    """An action running on a worker thread (``IO.asTask`` in the reference)."""
    _pool = cf.ThreadPoolExecutor(max_workers=8, thread_name_prefix="tyr-bg")

    def __init__(self, description: str, action: Callable[[], T]):
        self.description = description
        self.start_time = mono_ms()
        self._future = self._pool.submit(action)

    def get(self):
        return self._future.result()

    def done(self) -> bool:
        return self._future.done()


@dataclass
class Report:
    base_dir: str
    sections: List[Tuple[str, str, Any]] = field(default_factory=list)   # (kind, title, payload)
    start_time: int = field(default_factory=mono_ms)

    def log_stage(self, stage_name: str, content: str) -> "Report":
        self.sections.append(("stage", stage_name, content))
        return self

    def log_metrics(self, name: str, values: List[Tuple[str, str]]) -> "Report":
        self.sections.append(("metrics", name, list(values)))
        return self

    def to_markdown(self) -> str:
        out = ["# Pipeline report", "", f"Generated: {time.strftime('%Y-%m-%d %H:%M:%S')}", ""]
        for kind, title, payload in self.sections:
            out.append(f"## {title}")
            if kind == "stage":
                out += [str(payload), ""]
            else:
                out += [f"- **{k}**: {v}" for k, v in payload] + [""]
        out.append(f"Total: {format_duration(mono_ms() - self.start_time)}")
        return "\n".join(out)

    def write(self, filename: str = "report.md") -> str:
        os.makedirs(self.base_dir, exist_ok=True)
        p = os.path.join(self.base_dir, filename)
        with open(p, "w", encoding="utf-8") as f:
            f.write(self.to_markdown())
        return p


def checkpoint_path(base_dir: str) -> str:
    return os.path.join(base_dir, ".pipeline_checkpoint.json")


def save_checkpoint(base_dir: str, stages: List[StageInfo], run_id: str, config_repr: str = "") -> None:
    os.makedirs(base_dir, exist_ok=True)
    tmp = checkpoint_path(base_dir) + ".tmp"
    with open(tmp, "w", encoding="utf-8") as f:
        json.dump({"stages": [s.to_json() for s in stages], "timestamp": mono_ms(), "runId": run_id, "configRepr": config_repr}, f)
    os.replace(tmp, checkpoint_path(base_dir))


def load_checkpoint(base_dir: str) -> Optional[dict]:
    p = checkpoint_path(base_dir)
    if not os.path.exists(p):
        return None
    try:
        j = json.load(open(p, encoding="utf-8"))
        return {"stages": [StageInfo.from_json(s) for s in j["stages"]], "timestamp": j["timestamp"], "runId": j.get("runId", ""),
                "configRepr": j.get("configRepr", "")}
    except (ValueError, KeyError):
        return None


def clear_checkpoint(base_dir: str) -> None:
    if os.path.exists(checkpoint_path(base_dir)):
        os.remove(checkpoint_path(base_dir))


def current_distributed_rank() -> int:
    return int(os.environ.get("RANK", "0"))


def get_local_rank_from_env() -> int:
    return int(os.environ.get("LOCAL_RANK", "0"))


def rank_artifact_file(base_path: str, stem: str, ext: str, rank: int) -> str:
    return os.path.join(base_path, f"{stem}.rank{rank}.{ext}")


def resolve_training_device(rank: int, local_rank: int, is_distributed: bool):
    """``TYR_DEVICE`` = cpu | cuda | cuda:N | auto; distributed runs use ``cuda:<local_rank>`` (Pipeline.lean:305-321)."""
    import torch
    req = os.environ.get("TYR_DEVICE", "auto").lower()
    if req == "cpu":
        return torch.device("cpu")
    if req.startswith("cuda:") and not is_distributed:
        return torch.device(req)
    if req in ("auto", "cuda") or is_distributed or req.startswith("cuda"):
        if torch.cuda.is_available():
            return torch.device("cuda", local_rank if is_distributed else 0)
        if req == "auto":
            return torch.device("cpu")
        raise RuntimeError("TYR_DEVICE requests CUDA but no GPU is visible")
    raise ValueError(f"unknown TYR_DEVICE value {req!r}")


@dataclass
class PipelineConfig:
    base_dir: str = "~/.cache/tyr"
    wandb_enabled: bool = False
    wandb_run: str = "dummy"
    num_gpus: int = 1
    resume_from_checkpoint: bool = True
    retry_policy: RetryPolicy = field(default_factory=RetryPolicy)
    checkpoint_after_stage: bool = True
    fail_fast: bool = True
    run_id: str = ""

    def resolved_base_dir(self) -> str:
        return os.path.expanduser(self.base_dir)


class Pipeline:
    """State of one pipeline execution (``PipelineState`` + the ``PipelineM`` operations)."""

    def __init__(self, config: PipelineConfig, log: Optional[Handlers] = None, rank: int = 0, world_size: int = 1,
                 sleep: Callable[[float], None] = time.sleep):
        self.config, self.rank, self.world_size = config, rank, world_size
        self.log_handlers = (log or Handlers()).master_only(rank)
        self.base_dir = config.resolved_base_dir()
        self.stages: List[StageInfo] = []
        self.report = Report(self.base_dir)
        self.ledger = None
        self._sleep = sleep
        if config.resume_from_checkpoint:
            cp = load_checkpoint(self.base_dir)
            if cp is not None:
                if cp["configRepr"] == repr(config):
                    self.stages = cp["stages"]
                    self.log(f"[RESUME] Loaded {len(self.stages)} stage records from {checkpoint_path(self.base_dir)}")
                else:
                    self.log("[RESUME] Checkpoint belongs to a different configuration; ignoring it")

    # -- logging ----------------------------------------------------------------------------------------
    @property
    def is_master(self) -> bool:
        return self.rank == 0

    def log(self, msg: str) -> None:
        self.log_handlers.on_info(msg)

    def log_error(self, msg: str) -> None:
        self.log_handlers.on_error(msg)

    def master_only(self, action: Callable[[], T], default: T) -> T:
        return action() if self.is_master else default

    # -- stages ---------------------------------------------------------------------------------------------
    def _find(self, name: str) -> Optional[StageInfo]:
        return next((s for s in self.stages if s.name == name), None)

    def _checkpoint(self) -> None:
        if self.config.checkpoint_after_stage and self.is_master:
            save_checkpoint(self.base_dir, self.stages, self.config.run_id, repr(self.config))

    def _run_stage(self, name: str, action: Callable[[], None], propagate: bool) -> bool:
        prev = self._find(name)
        if prev is not None:
            if prev.status == "completed":
                self.log(f"[SKIP] Already completed: {name}")
                return True
            if prev.status == "failed":
                self.log(f"[RESUME] Retrying previously failed stage: {name} (was: {prev.error})")
            self.stages.remove(prev)
        info = StageInfo(name, "running", start_time=mono_ms())
        self.stages.append(info)
        self.log(f"[STAGE] {name}")
        try:
            action()
        except Exception as e:                      # a stage failure is data, not control flow, unless fail_fast
            info.status, info.error, info.end_time = "failed", str(e), mono_ms()
            self.report.log_stage(name, f"FAILED: {e}")
            self._checkpoint()
            self.log_error(f"[FAILED] {name}: {e}")
            if propagate:
                raise
            return False
        info.status, info.end_time = "completed", mono_ms()
        self.report.log_stage(name, f"Duration: {format_duration(info.duration_ms())}")
        self._checkpoint()
        self.log(f"[DONE] {name} ({format_duration(info.duration_ms())})")
        return True

    def stage(self, name: str, action: Callable[[], None]) -> bool:
        return self._run_stage(name, action, self.config.fail_fast)

    def stage_with_retry(self, name: str, action: Callable[[], None], policy: Optional[RetryPolicy] = None) -> bool:
        policy = policy or self.config.retry_policy
        last: Optional[Exception] = None
        for attempt in range(policy.max_attempts):
            try:
                if self._run_stage(name, action, True):
                    return True
            except Exception as e:
                last = e
                if attempt + 1 < policy.max_attempts:
                    delay = policy.delay_for_attempt(attempt)
                    self.log(f"[RETRY] {name}: attempt {attempt + 1}/{policy.max_attempts} failed, retrying in {delay} ms")
                    self._sleep(delay / 1000.0)
        if self.config.fail_fast and last is not None:
            raise last
        return False

    def pretrain_stage(self, name: str, train_fn: Callable[[], None], eval_fn: Callable[[], None]) -> None:
        self.stage(f"{name}-train", train_fn)
        self.stage(f"{name}-eval", eval_fn)

    finetune_stage = pretrain_stage

    # -- background work ----------------------------------------------------------------------------------------
    def background(self, description: str, action: Callable[[], T]) -> BackgroundTask:
        self.log(f"[BACKGROUND] {description}")
        return BackgroundTask(description, action)

    def await_task(self, task: BackgroundTask, on_error: Optional[Callable[[str], T]] = None):
        try:
            v = task.get()
            self.log(f"[BACKGROUND DONE] {task.description} ({format_duration(mono_ms() - task.start_time)})")
            return v
        except Exception as e:
            self.log_error(f"[BACKGROUND FAILED] {task.description}: {e}")
            if on_error is None:
                raise
            return on_error(str(e))

    # -- distributed health -----------------------------------------------------------------------------------------
    def has_local_failure(self) -> bool:
        return any(s.status == "failed" for s in self.stages)

    def sync_barrier(self) -> None:
        if self.world_size > 1:
            tdist.barrier()

    def check_all_ranks_healthy(self) -> bool:
        ok = not self.has_local_failure()
        if self.world_size == 1:
            return ok
        healthy = tdist.check_all_ranks_healthy(ok)
        if not ok and self.is_master:
            self.log_error("[DISTRIBUTED] This rank has failures")
        return healthy

    # -- metrics ---------------------------------------------------------------------------------------------------------
    def record_metrics(self, metrics: List[Tuple[str, str]]) -> None:
        running = next((s for s in reversed(self.stages) if s.status == "running"), None)
        name = running.name if running else "pipeline"
        if running:
            running.metrics += list(metrics)
        self.report.log_metrics(name, metrics)
        if self.ledger is not None and self.is_master:
            from .train import run_ledger as rl
            rl.append_metric_event(self.ledger, rl.MetricEvent(scope=name, metrics=list(metrics)))

    def finalize(self) -> Optional[str]:
        failed = [s for s in self.stages if s.status == "failed"]
        self.log(f"Pipeline finished: {sum(s.status == 'completed' for s in self.stages)} completed, {len(failed)} failed")
        if self.is_master:
            path = self.report.write()
            if not failed:
                clear_checkpoint(self.base_dir)
            return path
        return None


def run_pipeline(config: PipelineConfig, action: Callable[[Pipeline], T], log: Optional[Handlers] = None) -> T:
    p = Pipeline(config, log)
    try:
        return action(p)
    finally:
        p.finalize()


def with_distributed(config: PipelineConfig, action: Callable[[Pipeline], T], log: Optional[Handlers] = None,
                     backend: Optional[str] = None) -> T:
    """torchrun environment -> process group -> pipeline (Pipeline.lean:803-822).  Single-process when WORLD_SIZE is unset."""
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = current_distributed_rank()
    if world <= 1:
        return run_pipeline(config, action, log)
    local = get_local_rank_from_env()
    backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
    if backend == "nccl":
        tdist.set_cuda_device(local)
    tdist.init_process_group(backend, os.environ.get("MASTER_ADDR", "127.0.0.1"), int(os.environ.get("MASTER_PORT", "29500")), rank, world)
    p = Pipeline(config, log, rank, world)
    try:
        return action(p)
    finally:
        p.finalize()
        tdist.destroy_process_group()
