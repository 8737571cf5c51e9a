"""Launch helpers: command construction, log parsing, the scaling table and the resume check (with a fake runner), plus one
real single-process resume check on CPU."""
import pytest

from tyr_b200.cli import launch as L


def test_torchrun_command_and_log_parsing():
    assert L.torchrun_command("m", 1, ["--x"])[1:] == ["-m", "m", "--x"]
    cmd = L.torchrun_command("m", 4, ["--x"], 29999)
    assert "--nproc-per-node=4" in cmd and cmd[cmd.index("--master-addr") + 1] == "127.0.0.1" and cmd[-3:] == ["-m", "m", "--x"]
    log = "Step 0 | loss 11.0901 | 1,234 tok/s | 5.0 ms/step\nnoise\nStep 4 | loss 9.5000 | 231,456 tok/s | 283.5 ms/step\nFinished at step 6; checkpoint x\n"
    assert L.parse_throughput(log) == {"step": 4, "loss": 9.5, "tok_s": 231456.0} and L.parse_throughput("nothing") is None


def test_bench_table_and_failures(tmp_path, capsys):
    speeds = {1: 100.0, 2: 196.0, 4: 380.0}

    def fake(cmd, env=None, log_file=None, echo=True):
        n = 1
        for c in cmd:
            if c.startswith("--nproc-per-node="):
                n = int(c.split("=")[1])
        return f"Step 2 | loss 5.0 | {speeds[n]:,.0f} tok/s | 1 ms/step\nFinished at step 4; checkpoint c\n"
    rows = L.bench_distributed([1, 2, 4], ["--debug"], str(tmp_path), echo=False, runner=fake)
    assert [round(r["speedup"], 2) for r in rows] == [1.0, 1.96, 3.8] and round(rows[2]["efficiency"], 2) == 0.95
    assert "efficiency" in capsys.readouterr().out
    with pytest.raises(RuntimeError, match="did not reach"):
        L.bench_distributed([1], [], str(tmp_path), echo=False, runner=lambda *a, **k: "Step 1 | loss 1 | 5 tok/s\n")
    with pytest.raises(ValueError):
        L.bench_distributed([0], [], str(tmp_path), echo=False, runner=fake)


def test_resume_check_single_process_cpu():
    assert L.test_resume(1, ["--debug", "--synthetic", "--depth", "2"], steps=4, echo=False)
