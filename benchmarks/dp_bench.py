"""Device time of every fused data-parallel kernel of a NanoChat step, next to its NVLink roofline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m benchmarks.dp_bench [--depth 20]

Every rank runs the d20 trainer through `FusedDataParallel` with `TYR_DP_TIMING=1` (CUDA events around each kernel on the
launching stream).  For every kernel the table gives the median over the timed steps of the MAX over ranks, the bytes that
cross NVLink into and out of one GPU, the achieved bandwidth in the busier direction and its fraction of the measured
peer-copy bandwidth (770 GB/s per direction).  A kernel's time includes its in-kernel wait for the peers' gradients, so
the first kernel after backward also absorbs the skew between ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

LINK_GBS = 770.0


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--depth", type=int, default=20)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    os.environ["TYR_DP_TIMING"] = "1"
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from tyr_b200.models import nanochat as nc
    from tyr_b200.parallel.dp import FusedDataParallel
    from tyr_b200.train import nanochat_engine as eng
    cfg = nc.depth_config(a.depth, max_seq_len=a.seq)
    hp = eng.Hyperparameters(device_batch_size=a.batch, max_seq_len=a.seq, total_batch_size_tokens=a.batch * a.seq * world)
    dp = FusedDataParallel(rank, world, dev)
    tr = eng.NanoChatTrainer(cfg, hp, device=dev, seed=1, world_size=world, rank=rank, dp=dp)
    tok = torch.randint(0, cfg.vocab_size, (a.batch, a.seq + 1), device=dev, generator=torch.Generator(device=dev).manual_seed(rank))
    mb = [(tok[:, :-1].contiguous(), tok[:, 1:].contiguous())]
    for _ in range(a.warmup):
        tr.step(mb)
    dp.timings()
    per_step = []
    for _ in range(a.steps):
        dist.barrier()
        tr.step(mb)
        per_step.append(dp.timings())
    labels = [t[0] for t in per_step[0]]
    rows = []
    for i, lab in enumerate(labels):
        ms = torch.tensor([s[i][1] for s in per_step], dtype=torch.float64, device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        med = statistics.median(ms.tolist())
        bi, bo = per_step[0][i][2], per_step[0][i][3]
        busy = max(bi, bo)
        gbs = busy / med / 1e6 if med > 0 else 0.0
        rows.append({"kernel": lab, "ms": med, "nvlink_in_bytes": bi, "nvlink_out_bytes": bo, "gbs_busier_direction": gbs,
                     "fraction_of_link": gbs / LINK_GBS if busy else None})
    if rank == 0:
        print(f"fused data-parallel kernels, {world} ranks, nanochat d{a.depth}, {a.batch} x {a.seq} tokens per rank")
        for r in rows:
            frac = f"{r['fraction_of_link']:.2f} of {LINK_GBS:.0f} GB/s" if r["fraction_of_link"] is not None else "compute only"
            print(f"  {r['kernel']:28s} {r['ms']:8.3f} ms   in {r['nvlink_in_bytes'] / 1e6:9.1f} MB  out {r['nvlink_out_bytes'] / 1e6:9.1f} MB"
                  f"   {r['gbs_busier_direction']:7.1f} GB/s   {frac}")
        print(f"  total {sum(r['ms'] for r in rows):.3f} ms")
        if a.out:
            with open(a.out, "w") as f:
                json.dump({"world": world, "rows": rows}, f, indent=1)
    dp.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
