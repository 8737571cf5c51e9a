"""Child process of tests/test_gpu_multi.py: one rank checking the peer-memory collectives.

Every collective of ``tyr_b200.distributed`` runs twice on the same inputs, first over NCCL and then over the symmetric-heap
kernels (``enable_peer_collectives``), and the results are compared; then the public optimizer steps
(``distadam.step_distributed``, ``normuon.step_distributed_group``) run both ways."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from tyr_b200 import distributed as D  # noqa: E402
from tyr_b200.ops._common import raise_on_device_error  # noqa: E402
from tyr_b200.optim import distadam, normuon  # noqa: E402


def close(a, b, tol):
    a, b = a.float(), b.float()
    return (a - b).abs().max().item() <= tol * max(1.0, b.abs().max().item())


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    D.init_process_group("nccl", os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]), rank, world)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn(world * 37, 515, device=dev, generator=g)          # odd sizes: padded pieces, scalar tails
    xb = torch.randn(world * 8, 64, device=dev, generator=g).bfloat16()
    lst = [torch.randn(33, 129, device=dev, generator=g) for _ in range(world)]
    small = torch.randn(5, device=dev, generator=g)

    def run_all():
        return {
            "all_reduce_avg": D.all_reduce(x, D.ReduceOp.avg),
            "all_reduce_sum_bf16": D.all_reduce(xb, D.ReduceOp.sum),
            "reduce_scatter_avg": D.reduce_scatter(x, D.ReduceOp.avg),
            "reduce_scatter_list": D.reduce_scatter_list(lst, D.ReduceOp.sum),
            "all_gather": D.all_gather(x[:37]),
            "all_gather_small": D.all_gather(small),
            "all_gather_list": torch.stack(D.all_gather_list(lst[0])),
        }

    def optim_steps():
        gp = torch.Generator(device=dev).manual_seed(7)                 # same parameters on every rank
        p = torch.randn(world * 16, 96, device=dev, generator=gp)
        grad = torch.randn(world * 16, 96, device=dev, generator=g)    # rank-specific gradients (g advances: reseed below)
        acfg = distadam.Config(distributed=True)
        st = distadam.init_param_state(p)
        p1, s1 = distadam.step_distributed(p, grad, st, acfg)
        mats = [torch.randn(64, 96, device=dev, generator=gp) for _ in range(world + 1)]
        grads = [torch.randn(64, 96, device=dev, generator=g) for _ in range(world + 1)]
        mcfg = normuon.Config(distributed=True)
        states = [normuon.init_param_state(m) for m in mats]
        mp, ms = normuon.step_distributed_group(mats, grads, states, mcfg)
        return [p1.detach(), s1.exp_avg, s1.exp_avg_sq] + [q.detach() for q in mp] + [s.momentum_buffer for s in ms]

    ref = run_all()
    g.manual_seed(500 + rank)
    ref_opt = optim_steps()
    D.enable_peer_collectives(capacity_bytes=8 << 20)
    got = run_all()
    g.manual_seed(500 + rank)
    got_opt = optim_steps()
    torch.cuda.synchronize()
    raise_on_device_error(dev)
    ok, msg = True, ""
    for k in ref:
        tol = 2e-2 if "bf16" in k else 1e-5
        if ref[k].shape != got[k].shape or ref[k].dtype != got[k].dtype or not close(got[k], ref[k], tol):
            ok = False
            msg += f"rank {rank}: {k} differs (max {(got[k].float() - ref[k].float()).abs().max().item():.3e})\n"
    for i, (a, b) in enumerate(zip(got_opt, ref_opt)):
        if not close(a, b, 2e-3):
            ok = False
            msg += f"rank {rank}: optimizer output {i} differs (max {(a.float() - b.float()).abs().max().item():.3e})\n"
    # a tensor larger than the staging buffer must fall back to the transport and still be right
    big = torch.ones(world * (3 << 20), device=dev)
    if not torch.equal(D.reduce_scatter(big, D.ReduceOp.sum), torch.full((3 << 20,), float(world), device=dev)):
        ok, msg = False, msg + f"rank {rank}: fallback reduce_scatter wrong\n"
    flag = torch.tensor([1 if ok else 0], device=dev)
    import torch.distributed as tdist
    tdist.all_reduce(flag, op=tdist.ReduceOp.MIN)
    D.destroy_process_group()
    if msg:
        print(msg, file=sys.stderr)
    if rank == 0:
        print("PEER_COLLECTIVES_OK" if int(flag.item()) == 1 else "PEER_COLLECTIVES_FAILED")
    return 0 if int(flag.item()) == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
