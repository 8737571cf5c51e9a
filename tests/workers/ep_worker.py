"""Child process of the expert-parallel tests: one rank (nccl on GPUs, gloo on CPU)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from tyr_b200.ops import moe  # noqa: E402
from tyr_b200.parallel.ep import ExpertParallel, local_expert_fn  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    backend = os.environ.get("TYR_TEST_BACKEND", "nccl")
    if backend == "nccl":
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=dev)
        dtype, E, h, mi, k, T = torch.bfloat16, 8 * world, 256, 128, 4, 96
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
        dtype, E, h, mi, k, T = torch.float32, 4 * world, 32, 16, 2, 7
    g = torch.Generator().manual_seed(11)
    gate_up = (torch.randn(E, 2 * mi, h, generator=g) * h ** -0.5).to(dtype)
    down = (torch.randn(E, h, mi, generator=g) * mi ** -0.5).to(dtype)
    El = E // world
    mine = (gate_up[rank * El:(rank + 1) * El].to(dev).contiguous(), down[rank * El:(rank + 1) * El].to(dev).contiguous())
    ep = ExpertParallel(rank, world, dev, E, h, T, k)
    ok = True
    for it in range(3):
        gi = torch.Generator().manual_seed(100 * it + rank)
        x = torch.randn(T, h, generator=gi).to(dtype)
        logits = torch.randn(T, E, generator=gi)
        if it == 2:
            logits[:, :k] += 20.0                       # maximally skewed: every token to the first experts (rank 0)
        ids, w, cnt = moe.route(logits.to(dev), k)
        add = torch.randn(T, h, generator=gi).to(dtype)
        y = ep.forward(x.to(dev), ids, w, local_expert_fn(mine), add=add.to(dev), counts=cnt)
        ref = moe.moe_eager(x.float(), ids.cpu(), w.cpu(), gate_up[:, :mi].float(), gate_up[:, mi:].float(), down.float()) + add.float()
        err = (y.float().cpu() - ref).abs().max().item()
        tol = (0.05 if dtype == torch.bfloat16 else 1e-4) * max(1.0, ref.abs().max().item())
        if err > tol:
            ok = False
            print(f"rank {rank} it {it}: err {err} tol {tol}", flush=True)
    if dev.type == "cuda" and ep.fused:
        # the exchange replayed from a CUDA graph (two layers per step, fresh inputs per replay) against the eager result
        from tyr_b200.utils.graph import GraphedStep
        fn_e = local_expert_fn(mine)

        def two_layers(x, logits):
            for _ in range(2):
                ids, w, cnt = moe.route(logits, k)
                x = ep.forward(x, ids, w, fn_e, counts=cnt)
            return x
        gi = torch.Generator().manual_seed(500 + rank)
        xs = [torch.randn(T, h, generator=gi).to(dtype).to(dev) * 0.5 for _ in range(3)]
        ls = [torch.randn(T, E, generator=gi).to(dev) for _ in range(3)]
        step = GraphedStep(two_layers, (xs[0], ls[0]))
        for x, l in zip(xs, ls):
            got = step(x, l).clone()
            want = two_layers(x, l)
            err = (got.float() - want.float()).abs().max().item()
            if err > 0.05 * max(1.0, want.float().abs().max().item()):
                ok = False
                print(f"rank {rank} graph replay: err {err}", flush=True)
    if dev.type == "cuda":
        torch.cuda.synchronize()
        from tyr_b200.ops._common import raise_on_device_error
        raise_on_device_error(dev)
    flag = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("EP_WORKER_RESULT", "PASS" if flag.item() == 1.0 else "FAIL", flush=True)
    ep.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
