"""Run ledger: the standard artifact layout of a training run (Tyr/Train/RunLedger.lean).

``<base>/config.json``, ``metrics.jsonl``, ``checkpoints.jsonl``, ``checkpoints/``, ``report.md``; JSONL rows are
``{"scope", "step", "timestampMs", "metrics"}`` and ``{"name", "path", "kind", "step", "timestampMs", "metadata"}``.
"""
from __future__ import annotations

import enum
import json
import os
from dataclasses import asdict, dataclass, field, is_dataclass
from typing import Any, Callable, Dict, Generic, List, Optional, Sequence, Tuple, TypeVar

from ..utils.timer import mono_ms


class ExistingRunPolicy(enum.Enum):
    resume = "resume"
    overwrite = "overwrite"
    fail_if_exists = "failIfExists"


@dataclass
class RunArtifacts:
    base_dir: str
    config_path: str
    metrics_path: str
    checkpoints_path: str
    checkpoints_dir: str
    report_path: str

    @staticmethod
    def of_base_dir(base_dir: str) -> "RunArtifacts":
        j = lambda n: os.path.join(base_dir, n)
        return RunArtifacts(base_dir, j("config.json"), j("metrics.jsonl"), j("checkpoints.jsonl"), j("checkpoints"), j("report.md"))


def _to_json(config: Any):
    if is_dataclass(config):
        return asdict(config)
    if hasattr(config, "to_json"):
        return config.to_json()
    return config


def write_config(artifacts: RunArtifacts, config: Any) -> None:
    with open(artifacts.config_path, "w", encoding="utf-8") as f:
        json.dump(_to_json(config), f, indent=2, default=str)


def _has_existing(a: RunArtifacts) -> bool:
    return any(os.path.exists(p) for p in (a.config_path, a.metrics_path, a.checkpoints_path, a.report_path))


def prepare(artifacts: RunArtifacts, config: Any, policy: ExistingRunPolicy = ExistingRunPolicy.resume) -> None:
    os.makedirs(artifacts.base_dir, exist_ok=True)
    os.makedirs(artifacts.checkpoints_dir, exist_ok=True)
    if policy is ExistingRunPolicy.fail_if_exists and _has_existing(artifacts):
        raise IOError(f"Run directory already contains artifacts: {artifacts.base_dir}")
    if policy is ExistingRunPolicy.resume:
        if not os.path.exists(artifacts.config_path):
            write_config(artifacts, config)
        for p in (artifacts.metrics_path, artifacts.checkpoints_path):
            if not os.path.exists(p):
                open(p, "w").close()
        return
    write_config(artifacts, config)
    for p in (artifacts.metrics_path, artifacts.checkpoints_path):
        open(p, "w").close()


MetricFields = List[Tuple[str, Any]]


@dataclass
class MetricEvent:
    scope: str
    step: Optional[int] = None
    metrics: MetricFields = field(default_factory=list)
    timestamp_ms: int = 0

    def to_json(self) -> dict:
        return {"scope": self.scope, "step": self.step, "timestampMs": self.timestamp_ms, "metrics": dict(self.metrics)}


@dataclass
class CheckpointEvent:
    name: str
    path: str
    kind: str
    step: Optional[int] = None
    metadata: MetricFields = field(default_factory=list)
    timestamp_ms: int = 0

    def to_json(self) -> dict:
        return {"name": self.name, "path": self.path, "kind": self.kind, "step": self.step, "timestampMs": self.timestamp_ms,
                "metadata": dict(self.metadata)}


def _append_line(path: str, line: str) -> None:
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with open(path, "a", encoding="utf-8") as f:
        f.write(line + "\n")


def append_metric_event(artifacts: RunArtifacts, event: MetricEvent) -> None:
    if event.timestamp_ms == 0:
        event.timestamp_ms = mono_ms()
    _append_line(artifacts.metrics_path, json.dumps(event.to_json(), separators=(",", ":")))


def append_checkpoint_event(artifacts: RunArtifacts, event: CheckpointEvent) -> None:
    if event.timestamp_ms == 0:
        event.timestamp_ms = mono_ms()
    _append_line(artifacts.checkpoints_path, json.dumps(event.to_json(), separators=(",", ":")))


def read_events(path: str) -> List[dict]:
    if not os.path.exists(path):
        return []
    with open(path, encoding="utf-8") as f:
        return [json.loads(l) for l in f if l.strip()]


@dataclass
class EvalSchedule:
    every: int = 0
    run_at_start: bool = False
    run_at_end: bool = True

    def should_run(self, step: int, is_last_step: bool = False) -> bool:
        return ((self.run_at_start and step == 0) or (self.every > 0 and step > 0 and step % self.every == 0)
                or (self.run_at_end and is_last_step))


C = TypeVar("C")


@dataclass
class Evaluator(Generic[C]):
    name: str
    run: Callable[[C], MetricFields]
    schedule: EvalSchedule = field(default_factory=EvalSchedule)


def run_due_evaluators(evaluators: Sequence[Evaluator], ctx, step: int, is_last_step: bool = False) -> MetricFields:
    out: MetricFields = []
    for ev in evaluators:
        if ev.schedule.should_run(step, is_last_step):
            out += [(f"{ev.name}/{k}", v) for k, v in ev.run(ctx)]
    return out
