"""One CPU (Gloo) rank of the two-rank collective value test
(the reference's Tests/RunDistributedValues.lean driven by scripts/test_distributed_values.py)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import tyr_b200.distributed as dist  # noqa: E402
from tyr_b200.distributed import ReduceOp  # noqa: E402


def check(cond, msg):
    if not cond:
        raise AssertionError(msg)


def run(rank, world, port):
    dist.init_process_group("gloo", "127.0.0.1", port, rank, world)
    check(dist.is_initialized() and dist.get_rank() == rank and dist.get_world_size() == world, "identity")
    x = torch.tensor([1.0 + rank, 2.0, -3.0 * rank], requires_grad=True)
    keep = x.detach().clone()
    s = dist.all_reduce(x, ReduceOp.sum)
    check(torch.equal(x.detach(), keep), "all_reduce modified its input")
    check(torch.allclose(s, torch.tensor([3.0, 4.0, -3.0])), f"sum {s}")
    check(s.requires_grad, "requires_grad not propagated")
    check(torch.allclose(dist.all_reduce(x, ReduceOp.avg), torch.tensor([1.5, 2.0, -1.5])), "avg")
    check(torch.allclose(dist.all_reduce(x.detach(), ReduceOp.max), torch.tensor([2.0, 2.0, 0.0])), "max")
    check(torch.allclose(dist.all_reduce(x.detach(), ReduceOp.min), torch.tensor([1.0, 2.0, -3.0])), "min")
    check(torch.allclose(dist.all_reduce(x.detach(), ReduceOp.product), torch.tensor([2.0, 4.0, 0.0])), "product")
    xi = torch.tensor([rank + 1, 10], dtype=torch.int64)
    check(torch.equal(dist.all_reduce(xi, ReduceOp.sum), torch.tensor([3, 20])), "int sum")
    check(torch.equal(dist.all_reduce(xi, ReduceOp.avg), torch.tensor([1, 10])), "int avg")
    b = dist.broadcast(torch.tensor([float(rank), 7.0]), root=1)
    check(torch.equal(b, torch.tensor([1.0, 7.0])), "broadcast")
    rs = dist.reduce_scatter(torch.arange(4.0) + rank, ReduceOp.sum)
    check(torch.equal(rs, torch.tensor([1.0, 3.0]) if rank == 0 else torch.tensor([5.0, 7.0])), f"reduce_scatter {rs}")
    rsl = dist.reduce_scatter_list([torch.full((2,), float(rank + r)) for r in range(world)], ReduceOp.avg)
    check(torch.allclose(rsl, torch.full((2,), 0.5 + rank)), f"reduce_scatter_list {rsl}")
    ag = dist.all_gather(torch.tensor([[float(rank), 1.0]]))
    check(torch.equal(ag, torch.tensor([[0.0, 1.0], [1.0, 1.0]])), "all_gather")
    agl = dist.all_gather_list(torch.tensor([rank]))
    check([int(t) for t in agl] == [0, 1], "all_gather_list")
    h = dist.all_reduce_async(torch.ones(3), ReduceOp.sum)
    check(torch.equal(h.wait(), torch.full((3,), 2.0)), "async")
    try:
        h.wait()
        raise AssertionError("a consumed handle was waited twice")
    except dist.DistributedError:
        pass
    dist.barrier()
    # a pending handle is drained by teardown
    dist.all_reduce_async(torch.ones(2))
    dist.destroy_process_group()
    check(not dist.is_initialized(), "teardown")


def main():
    rank, port, restart_port = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    run(rank, 2, port)
    # teardown + re-init on a second port
    run(rank, 2, restart_port)
    # teardown after an action error
    try:
        with dist.with_distributed("gloo", "127.0.0.1", restart_port + 2, rank, 2):
            raise RuntimeError("intentional action failure")
    except RuntimeError as e:
        check("intentional" in str(e), "wrong error surfaced")
    check(not dist.is_initialized(), "withDistributed did not tear down")
    print(f"RANK{rank} OK")


if __name__ == "__main__":
    main()
