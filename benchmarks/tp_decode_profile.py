"""Kernel list of one tensor-parallel Qwen3.5 decode step.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m benchmarks.tp_decode_profile \
        [--preset 27b] [--layers 8] [--batch 32] [--prompt 256] [--out FILE]

Random-init weights created in sharded form.  After a prefill and two warm-up steps, rank 0 records three eager decode steps
(the body that the CUDA-graph step replays) under torch.profiler and prints every kernel with its launches per step and device
time per step, then times the graph step itself with CUDA events (max over ranks).  Shares only under the profiler.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="27b")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prompt", type=int, default=256)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--rows", type=int, default=40)
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from torch.profiler import ProfilerActivity, profile

    from tyr_b200.cli.run_qwen35 import PRESETS
    from tyr_b200.models import qwen35_tp as QT
    from tyr_b200.parallel.tp import TensorParallel
    import dataclasses
    cfg = dataclasses.replace(PRESETS[a.preset](), num_hidden_layers=a.layers, layer_types=None)
    B, S = a.batch, a.prompt
    tp = TensorParallel(rank, world, dev, max_rows=max(B * S, 1024), max_cols=cfg.hidden_size, max_k=cfg.hidden_size,
                        gather_elems=B * -(-cfg.vocab_size // world))
    m = QT.init_sharded(cfg, rank, world, tp, device=dev)
    cache = QT.TPCache(m, B, S + a.steps + 16)
    ids = torch.randint(0, cfg.vocab_size, (B, S), device=dev, generator=torch.Generator(device=dev).manual_seed(1))
    with torch.no_grad():
        tok = cache.prefill(ids).argmax(-1)
        cache.pos_t = torch.full((1,), cache.pos, dtype=torch.int32, device=dev)
        for _ in range(2):
            cache._device_step(tok)
        torch.cuda.synchronize()
        dist.barrier()
        n_prof = 3
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(n_prof):
                cache._device_step(tok)
            torch.cuda.synchronize()
        dist.barrier()
        # the graph step, timed on the device
        cache.pos = int(cache.pos_t.item())
        for c in cache.kv:
            if c is not None:
                c.length = cache.pos
        for _ in range(3):
            cache.step(tok)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            cache.step(tok)
        e1.record()
        torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        rows = sorted(((e.device_time_total / n_prof, e.count / n_prof, e.key) for e in prof.key_averages() if e.device_time_total > 0),
                      reverse=True)
        lines = [f"qwen3.5 {a.preset} widths, {a.layers} layers, TP = {world}, batch {B}: graph decode step {t.item():.3f} ms "
                 f"({B / t.item() * 1e3:.0f} tok/s); eager step under the profiler: {sum(r[0] for r in rows) / 1e3:.3f} ms of kernels "
                 f"in {sum(r[1] for r in rows):.0f} launches"]
        for us, n, k in rows[:a.rows]:
            lines.append(f"  {us:9.1f} us  x{n:<6.1f} {k[:120]}")
        text = "\n".join(lines)
        print(text)
        if a.out:
            with open(a.out, "w") as f:
                f.write(text + "\n")
    tp.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
