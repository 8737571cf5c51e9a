"""Distributed API: validation before rendezvous, fake backend with injected failures (the
reference's cc/tools/test_distributed_recovery.cpp), two-rank Gloo value test under a deadline
harness (scripts/test_distributed_values.py), sampler and sharding arithmetic."""
import os
import socket
import subprocess
import sys
import time

import pytest
import torch

import tyr_b200.distributed as dist
from tyr_b200.distributed import ReduceOp
from tyr_b200.distributed.sampler import DistributedSampler, DistributedSamplerConfig
from tyr_b200.distributed import sharding as sd

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(autouse=True)
def _clean():
    yield
    if dist.is_initialized():
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.parametrize("args,frag", [
    (("mpi", "127.0.0.1", 29500, 0, 1), "backend"), (("gloo", "127.0.0.1", 0, 0, 1), "port"),
    (("gloo", "127.0.0.1", 70000, 0, 1), "port"), (("gloo", "127.0.0.1", 29500, 0, 0), "world"),
    (("gloo", "127.0.0.1", 29500, 2, 2), "rank"), (("gloo", "", 29500, 0, 1), "address"),
])
def test_validation_happens_before_rendezvous(args, frag):
    t0 = time.time()
    with pytest.raises(ValueError, match=frag):
        dist.init_process_group(*args)
    assert time.time() - t0 < 1.0 and not dist.is_initialized()


class FakeWork:
    def __init__(self, mode="ok"):
        self.mode, self.waited = mode, 0

    def wait(self):
        self.waited += 1
        if self.mode == "raise":
            raise RuntimeError("injected wait failure")
        if self.mode == "unknown":
            raise KeyboardInterrupt() if False else Exception("injected unknown failure")
        return self.mode != "abort"

    def is_completed(self):
        return self.mode != "pending"


class FakeBackend:
    """No sockets, no GPUs: every async collective returns a scripted FakeWork."""

    def __init__(self, world=2, rank=0):
        self.world, self._rank, self.script, self.issued, self.down = world, rank, [], [], False

    def rank(self): return self._rank
    def size(self): return self.world

    def _work(self, async_op):
        w = FakeWork(self.script.pop(0) if self.script else "ok")
        self.issued.append(w)
        return w

    def all_reduce(self, t, op, async_op): t.mul_(self.world); return self._work(async_op)
    def broadcast(self, t, root, async_op): return None
    def reduce_scatter_tensor(self, out, inp, op, async_op): out.copy_(inp[: out.shape[0]] * self.world)
    def reduce_scatter_list(self, out, ins, op, async_op): out.copy_(ins[self._rank] * self.world)
    def all_gather_into_tensor(self, out, inp, async_op): out.copy_(torch.cat([inp] * self.world))
    def all_gather_list(self, outs, inp, async_op): [o.copy_(inp) for o in outs]
    def barrier(self): pass
    def shutdown(self): self.down = True


def test_fake_backend_handles_released_exactly_once():
    fb = FakeBackend()
    dist.init_process_group("gloo", "127.0.0.1", 29500, 0, 2, _inject=fb)
    fb.script = ["ok", "raise", "abort"]
    h_ok = dist.all_reduce_async(torch.ones(2), ReduceOp.avg)
    h_bad = dist.all_reduce_async(torch.ones(2))
    h_abort = dist.all_reduce_async(torch.ones(2))
    assert torch.equal(h_ok.wait(), torch.ones(2))
    with pytest.raises(dist.DistributedError):
        h_ok.wait()                      # consumed
    with pytest.raises(RuntimeError, match="injected"):
        h_bad.wait()
    with pytest.raises(dist.DistributedError):
        h_bad.wait()                     # released even though waiting raised
    with pytest.raises(dist.DistributedError, match="aborted"):
        h_abort.wait()
    assert [w.waited for w in fb.issued] == [1, 1, 1]


def test_destroy_drains_pending_and_rethrows_first_error():
    fb = FakeBackend()
    dist.init_process_group("gloo", "127.0.0.1", 29500, 0, 2, _inject=fb)
    fb.script = ["ok", "raise", "ok"]
    for _ in range(3):
        dist.all_reduce_async(torch.ones(1))
    with pytest.raises(dist.DistributedError, match="injected"):
        dist.destroy_process_group()
    assert [w.waited for w in fb.issued] == [1, 1, 1] and fb.down and not dist.is_initialized()
    # a fresh group can be created afterwards
    dist.init_process_group("gloo", "127.0.0.1", 29500, 0, 2, _inject=FakeBackend())
    assert dist.get_world_size() == 2
    h = dist.all_reduce_async(torch.ones(1))
    assert h.is_completed()
    dist.destroy_process_group()


def test_collectives_need_a_group_and_preserve_inputs():
    with pytest.raises(dist.DistributedError):
        dist.all_reduce(torch.ones(1))
    dist.init_process_group("gloo", "127.0.0.1", 29500, 1, 2, _inject=FakeBackend(rank=1))
    x = torch.arange(4.0)
    y = dist.reduce_scatter(x, ReduceOp.avg)
    assert torch.equal(x, torch.arange(4.0)) and y.shape == (2,)
    with pytest.raises(ValueError):
        dist.reduce_scatter(torch.ones(3))
    with pytest.raises(ValueError):
        dist.reduce_scatter_list([torch.ones(1)])
    with pytest.raises(ValueError):
        dist.broadcast(torch.ones(1), root=5)


def _free_ports(n):
    socks = [socket.socket() for _ in range(n)]
    for s in socks:
        s.bind(("127.0.0.1", 0))
    ports = [s.getsockname()[1] for s in socks]
    for s in socks:
        s.close()
    return ports


def test_two_rank_gloo_values(tmp_path):
    port, restart, _ = _free_ports(3)
    worker = os.path.join(ROOT, "tests", "workers", "dist_values_worker.py")
    procs = []
    for r in range(2):
        log = open(tmp_path / f"rank{r}.log", "w")
        procs.append((subprocess.Popen([sys.executable, worker, str(r), str(port), str(restart)], stdout=log,
                                       stderr=subprocess.STDOUT, cwd=ROOT), log))
    deadline = time.time() + 90
    try:
        for p, _ in procs:
            p.wait(timeout=max(1, deadline - time.time()))
    finally:
        for p, log in procs:
            if p.poll() is None:
                p.kill()
                p.wait()
            log.close()
    outs = [open(tmp_path / f"rank{r}.log").read() for r in range(2)]
    for r, (p, _) in enumerate(procs):
        assert p.returncode == 0 and f"RANK{r} OK" in outs[r], outs[r][-2000:]


def test_sampler_partitions_dataset():
    parts = [DistributedSampler.create(DistributedSamplerConfig(11, r, 3, seed=7)).indices for r in range(3)]
    assert sorted(sum(parts, [])) == list(range(11)) and [len(p) for p in parts] == [4, 4, 3]
    s = DistributedSampler.create(DistributedSamplerConfig(11, 0, 3, seed=7))
    assert s.next_epoch().indices != s.indices and s.next_epoch().epoch == 1
    ns = DistributedSampler.create(DistributedSamplerConfig(6, 1, 2, shuffle=False))
    assert ns.indices == [3, 4, 5] and ns.get_index(9) is None


def test_sharding_arithmetic_and_tensor():
    assert [sd.shard_size(10, 4, i) for i in range(4)] == [3, 3, 2, 2]
    assert [sd.shard_offset(10, 4, i) for i in range(4)] == [0, 3, 6, 8]
    assert sd.sharded_shape((10, 6), sd.ShardSpec(4, 3, sd.ShardDim.last)) == (10, 1)
    assert sd.sharded_shape((10,), sd.ShardSpec(4, 0, sd.ShardDim.dim(3))) == (10,)   # replicated
    full = torch.arange(20.0).reshape(10, 2)
    st = sd.ShardedTensor.from_full(full, 2, 4)
    assert torch.equal(st.shard, full[6:8])
    assert torch.equal(st.gather(), st.shard) and not st.cache_is_stale   # single process: local view
    st.update_shard(st.shard + 1)
    assert st.cache_is_stale
    with pytest.raises(ValueError):
        sd.ShardedTensor(full.shape, 0, 4, torch.zeros(5, 2))


def test_native_registry_and_apple_stubs():
    from tyr_b200 import distributed as D
    from tyr_b200.audio import apple
    init, rank, world = D.registry_state()
    assert isinstance(init, bool) and rank >= 0 and world >= 0
    assert apple.mps_is_available() is False
    import pytest
    with pytest.raises(IOError, match="macOS"):
        apple.start_microphone()
    with pytest.raises(IOError, match="macOS"):
        apple.beep()
