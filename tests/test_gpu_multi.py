"""Multi-GPU tests (child processes under torchrun, one rank per GPU, NVLS off)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run_torchrun(script, nproc, timeout=300, port=29611):
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = "0"
    env["MASTER_ADDR"] = "127.0.0.1"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), script]
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)


@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_fused_data_parallel_matches_accumulation(nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    r = _run_torchrun(os.path.join(ROOT, "tests", "workers", "dp_worker.py"), nproc, port=29611 + nproc)
    assert "DP_WORKER_RESULT PASS" in r.stdout, (r.stdout[-3000:], r.stderr[-3000:])


@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_tensor_parallel_fused_gemm_collectives(nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    r = _run_torchrun(os.path.join(ROOT, "tests", "workers", "tp_worker.py"), nproc, port=29631 + nproc)
    assert "TP_WORKER_RESULT PASS" in r.stdout, (r.stdout[-3000:], r.stderr[-3000:])


@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_expert_parallel_pull_dispatch_and_combine(nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    r = _run_torchrun(os.path.join(ROOT, "tests", "workers", "ep_worker.py"), nproc, port=29651 + nproc)
    assert "EP_WORKER_RESULT PASS" in r.stdout, (r.stdout[-3000:], r.stderr[-3000:])


@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_peer_memory_collectives_match_transport(nproc):
    """all_reduce / reduce_scatter(_list) / all_gather(_list) and the public DistAdam / NorMuon steps over the symmetric-heap
    kernels against the same calls over NCCL."""
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    r = _run_torchrun(os.path.join(ROOT, "tests", "workers", "peer_coll_worker.py"), nproc, port=29671 + nproc)
    assert "PEER_COLLECTIVES_OK" in r.stdout, (r.stdout[-3000:], r.stderr[-3000:])
