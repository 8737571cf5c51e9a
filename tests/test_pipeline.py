"""Run ledger and pipeline orchestrator (Tests: ledger layout, resume/skip, retry back-off, config guard)."""
import json
import os

import pytest

from tyr_b200 import pipeline as P
from tyr_b200.train import run_ledger as RL
from tyr_b200.utils.log import Handlers
from tyr_b200.utils.timer import Timer


def test_ledger_layout_policies_and_events(tmp_path):
    a = RL.RunArtifacts.of_base_dir(str(tmp_path / "run"))
    RL.prepare(a, {"lr": 0.1})
    assert json.load(open(a.config_path)) == {"lr": 0.1} and os.path.isdir(a.checkpoints_dir)
    RL.append_metric_event(a, RL.MetricEvent("train", 3, [("loss", 1.5), ("ok", True)]))
    RL.append_checkpoint_event(a, RL.CheckpointEvent("step3", "checkpoints/3", "model", 3, [("loss", 1.5)]))
    m, c = RL.read_events(a.metrics_path), RL.read_events(a.checkpoints_path)
    assert m[0]["scope"] == "train" and m[0]["step"] == 3 and m[0]["metrics"] == {"loss": 1.5, "ok": True} and m[0]["timestampMs"] > 0
    assert c[0]["kind"] == "model" and c[0]["metadata"] == {"loss": 1.5}
    RL.prepare(a, {"lr": 0.2})                                        # resume keeps the first config and the rows
    assert json.load(open(a.config_path)) == {"lr": 0.1} and len(RL.read_events(a.metrics_path)) == 1
    with pytest.raises(IOError, match="already contains artifacts"):
        RL.prepare(a, {}, RL.ExistingRunPolicy.fail_if_exists)
    RL.prepare(a, {"lr": 0.3}, RL.ExistingRunPolicy.overwrite)
    assert json.load(open(a.config_path)) == {"lr": 0.3} and RL.read_events(a.metrics_path) == []


def test_eval_schedule_and_evaluators():
    s = RL.EvalSchedule(every=5, run_at_start=True)
    assert [s.should_run(i) for i in (0, 1, 5, 7)] == [True, False, True, False] and s.should_run(7, True)
    evs = [RL.Evaluator("val", lambda ctx: [("loss", ctx * 2)], RL.EvalSchedule(every=2, run_at_end=False)),
           RL.Evaluator("core", lambda ctx: [("acc", 0.5)])]
    assert RL.run_due_evaluators(evs, 3, 4) == [("val/loss", 6)]
    assert RL.run_due_evaluators(evs, 3, 5, True) == [("core/acc", 0.5)]


def test_retry_policy_backoff():
    p = P.RetryPolicy(max_attempts=4, initial_delay_ms=100, backoff_multiplier=3.0, max_delay_ms=500)
    assert [p.delay_for_attempt(i) for i in range(4)] == [100, 300, 500, 500]


def test_stages_resume_skip_and_config_guard(tmp_path):
    cfg = P.PipelineConfig(base_dir=str(tmp_path), fail_fast=False, run_id="r1")
    logs = []
    calls = []
    p = P.Pipeline(cfg, Handlers(on_info=logs.append, on_error=logs.append))
    assert p.stage("download", lambda: calls.append("download"))
    assert not p.stage("train", lambda: 1 / 0)
    assert p.has_local_failure() and not p.check_all_ranks_healthy()
    cp = P.load_checkpoint(str(tmp_path))
    assert [s.status for s in cp["stages"]] == ["completed", "failed"] and cp["runId"] == "r1"
    # second run with the same config: the finished stage is skipped, the failed one retried
    p2 = P.Pipeline(cfg, Handlers(on_info=logs.append))
    p2.stage("download", lambda: calls.append("download-again"))
    p2.stage("train", lambda: calls.append("train"))
    assert calls == ["download", "train"] and any("[SKIP]" in l for l in logs) and any("[RESUME] Retrying" in l for l in logs)
    p2.record_metrics([("loss", "1.0")])
    path = p2.finalize()
    assert "## train" in open(path).read() and not os.path.exists(P.checkpoint_path(str(tmp_path)))
    # a different config must not skip
    p.stage("x", lambda: None)
    p3 = P.Pipeline(P.PipelineConfig(base_dir=str(tmp_path), num_gpus=8))
    assert p3.stages == []


def test_stage_with_retry_and_background(tmp_path):
    sleeps = []
    p = P.Pipeline(P.PipelineConfig(base_dir=str(tmp_path), retry_policy=P.RetryPolicy(3, 10, 2.0, 1000)), sleep=sleeps.append)
    attempts = []

    def flaky():
        attempts.append(1)
        if len(attempts) < 3:
            raise RuntimeError("transient")
    assert p.stage_with_retry("fetch", flaky) and len(attempts) == 3 and sleeps == [0.01, 0.02]
    with pytest.raises(ZeroDivisionError):
        p.stage_with_retry("always", lambda: 1 / 0, P.RetryPolicy(2, 1, 1.0, 1))
    t = p.background("sum", lambda: sum(range(10)))
    assert p.await_task(t) == 45
    assert p.await_task(p.background("boom", lambda: 1 / 0), on_error=lambda e: -1) == -1
    assert P.format_duration(61000) == "1m 1s" and P.rank_artifact_file("/a", "log", "txt", 3) == "/a/log.rank3.txt"


def test_resolve_device_and_timer(monkeypatch):
    monkeypatch.setenv("TYR_DEVICE", "cpu")
    assert P.resolve_training_device(0, 0, False).type == "cpu"
    monkeypatch.setenv("TYR_DEVICE", "bogus")
    with pytest.raises(ValueError):
        P.resolve_training_device(0, 0, False)
    t = Timer()
    with t.section("a"):
        pass
    assert t.counts["a"] == 1 and "a:" in t.report()
