"""Tensor-parallel host logic on CPU: two gloo ranks take the collective fallbacks and must agree with
the single-process product."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_tp_fallbacks_two_gloo_ranks():
    env = dict(os.environ, TYR_TEST_BACKEND="gloo", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29671", os.path.join(ROOT, "tests", "workers", "tp_worker.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=240)
    assert "TP_WORKER_RESULT PASS" in r.stdout, (r.stdout[-2000:], r.stderr[-2000:])


def test_world_one_is_a_plain_product():
    import torch
    from tyr_b200.parallel.tp import TensorParallel
    tp = TensorParallel(0, 1, "cpu")
    x, w = torch.randn(4, 8), torch.randn(3, 8)
    assert torch.allclose(tp.gemm_reduce_scatter(x, w), x @ w.T, atol=1e-5)
    assert torch.allclose(tp.allgather_gemm(x, w, act="relu"), torch.relu(x @ w.T), atol=1e-5)


def test_expert_parallel_collective_path_two_gloo_ranks():
    env = dict(os.environ, TYR_TEST_BACKEND="gloo", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29673", os.path.join(ROOT, "tests", "workers", "ep_worker.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=240)
    assert "EP_WORKER_RESULT PASS" in r.stdout, (r.stdout[-2000:], r.stderr[-2000:])
