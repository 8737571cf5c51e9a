"""Launch helpers for one-node runs (counterparts of scripts/nanochat/{run_train_torchrun,run_pipeline_torchrun,bench_distributed,
test_distributed_resume}.sh).

    python -m tyr_b200.cli.launch train --nproc 8 -- --depth 20 --synthetic --iterations 100
    python -m tyr_b200.cli.launch pipeline --nproc 8
    python -m tyr_b200.cli.launch bench-distributed --sizes 1 2 4 8 -- --depth 20 --synthetic --iterations 12 --log-every 4
    python -m tyr_b200.cli.launch test-resume --nproc 2 -- --debug --synthetic

Every run goes through ``python -m torch.distributed.run --nnodes=1 --master-addr 127.0.0.1`` (one process per GPU); a single
process is started directly.
"""
from __future__ import annotations

import argparse
import os
import re
import subprocess
import sys
import tempfile
from typing import Dict, List, Optional, Sequence

STEP_LINE = re.compile(r"Step (\d+) \| loss ([0-9.naninf-]+) \| ([0-9,]+) tok/s")


def torchrun_command(module: str, nproc: int, args: Sequence[str], port: int = 29500) -> List[str]:
    if nproc <= 1:
        return [sys.executable, "-m", module, *args]
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
            "--master-port", str(port), "-m", module, *args]


def run(cmd: Sequence[str], env: Optional[Dict[str, str]] = None, log_file: Optional[str] = None, echo: bool = True) -> str:
    """Runs to completion, tees the output, raises on a non-zero exit."""
    p = subprocess.Popen(list(cmd), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env={**os.environ, **(env or {})})
    lines = []
    for line in p.stdout:
        lines.append(line)
        if echo:
            sys.stdout.write(line)
    rc = p.wait()
    out = "".join(lines)
    if log_file:
        with open(log_file, "w") as f:
            f.write(out)
    if rc != 0:
        raise RuntimeError(f"command failed with exit code {rc}: {' '.join(cmd)}")
    return out


def parse_throughput(log: str) -> Optional[Dict[str, float]]:
    """Last ``Step N | loss L | T tok/s`` line of a training log."""
    last = None
    for m in STEP_LINE.finditer(log):
        last = m
    if last is None:
        return None
    return {"step": int(last.group(1)), "loss": float(last.group(2)), "tok_s": float(last.group(3).replace(",", ""))}


def bench_distributed(sizes: Sequence[int], args: Sequence[str], log_dir: str, echo: bool = True, runner=run) -> List[Dict]:
    """One training run per process count; a table of the last logged tokens/s and the speed-up over the first size."""
    rows = []
    for i, n in enumerate(sizes):
        if n < 1:
            raise ValueError(f"invalid process count '{n}'")
        ck = tempfile.mkdtemp(prefix=f"bench_{n}gpu_")
        log = runner(torchrun_command("tyr_b200.cli.train_nanochat", n, [*args, "--checkpoint-dir", ck], 29540 + i),
                     log_file=os.path.join(log_dir, f"tyr_nanochat_{n}gpu.log"), echo=echo)
        if "Finished at step" not in log:
            raise RuntimeError(f"run did not reach training completion for {n} GPU(s)")
        t = parse_throughput(log)
        if t is None:
            raise RuntimeError(f"failed to extract throughput for {n} GPU(s)")
        rows.append({"gpus": n, **t})
    base = rows[0]["tok_s"]
    print(f"\n{'gpus':<6}{'tok_per_s':>14}{'speedup':>10}{'efficiency':>12}")
    for r in rows:
        r["speedup"] = r["tok_s"] / base if base else float("nan")
        r["efficiency"] = r["speedup"] * rows[0]["gpus"] / r["gpus"]
        print(f"{r['gpus']:<6}{r['tok_s']:>14,.0f}{r['speedup']:>10.3f}{r['efficiency']:>12.3f}")
    return rows


def test_resume(nproc: int, args: Sequence[str], steps: int = 6, echo: bool = True, runner=run) -> bool:
    """Train ``steps`` straight through, then ``steps / 2`` + resume; the final logged losses must agree."""
    half = steps // 2
    a, b = tempfile.mkdtemp(prefix="resume_a_"), tempfile.mkdtemp(prefix="resume_b_")
    common = [*args, "--log-every", "1"]
    full = runner(torchrun_command("tyr_b200.cli.train_nanochat", nproc, [*common, "--iterations", str(steps), "--checkpoint-dir", a], 29560), echo=echo)
    runner(torchrun_command("tyr_b200.cli.train_nanochat", nproc, [*common, "--iterations", str(half), "--checkpoint-dir", b], 29561), echo=echo)
    resumed = runner(torchrun_command("tyr_b200.cli.train_nanochat", nproc, [*common, "--iterations", str(steps), "--checkpoint-dir", b, "--resume", b], 29562), echo=echo)
    x, y = parse_throughput(full), parse_throughput(resumed)
    ok = x is not None and y is not None and x["step"] == y["step"] and abs(x["loss"] - y["loss"]) <= 1e-3 * max(1.0, abs(x["loss"]))
    print(f"resume check: straight loss {x and x['loss']}, resumed loss {y and y['loss']} -> {'OK' if ok else 'MISMATCH'}")
    return ok


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    rest: List[str] = []
    if "--" in argv:
        i = argv.index("--")
        argv, rest = argv[:i], argv[i + 1:]
    p = argparse.ArgumentParser(prog="launch")
    sub = p.add_subparsers(dest="cmd", required=True)
    for name in ("train", "pipeline", "test-resume"):
        s = sub.add_parser(name)
        s.add_argument("--nproc", type=int, default=int(os.environ.get("NPROC_PER_NODE", "1")))
        s.add_argument("--port", type=int, default=29500)
    b = sub.add_parser("bench-distributed")
    b.add_argument("--sizes", type=int, nargs="+", default=[1, 2, 4])
    b.add_argument("--log-dir", default=tempfile.gettempdir())
    a = p.parse_args(argv)
    if a.cmd == "train":
        run(torchrun_command("tyr_b200.cli.train_nanochat", a.nproc, rest, a.port))
    elif a.cmd == "pipeline":
        run(torchrun_command("tyr_b200.nanochat.pipeline", a.nproc, rest, a.port), env={"WORLD_SIZE": str(a.nproc)} if a.nproc <= 1 else None)
    elif a.cmd == "bench-distributed":
        bench_distributed(a.sizes, rest or ["--debug", "--synthetic", "--iterations", "8", "--log-every", "2"], a.log_dir)
    else:
        return 0 if test_resume(a.nproc, rest or ["--debug", "--synthetic"]) else 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
