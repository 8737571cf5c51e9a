"""Kernel-time shares of one NanoChat training step: `python -m benchmarks.step_profile [--depth 20] [--out FILE]`.

Runs the trainer for two warm-up steps, records one step under torch.profiler (CUDA activity
only) and prints every kernel with its launch count and summed device time, largest first,
followed by the split between this repository's kernels and everything else (ATen, cuDNN,
cuBLAS).  The figures are shares: absolute step time comes from `bench.py`, which runs without
a profiler attached.
"""
from __future__ import annotations

import argparse
import sys

import torch

# Kernel-name fragments of the kernels compiled from csrc/*.cu.
OWN = ("tcgen05", "flash_", "rmsnorm", "qkv_post", "softcap_ce", "adamw", "muon", "dp_", "embed", "nanochat_",
       "ns_", "lincomb", "moe_", "ep_", "gdr_", "skinny", "decode_attn", "modulate", "gate_residual", "tyr_",
       "scalars_", "smear", "cast_", "ce_", "rope")


def is_own(name: str) -> bool:
    n = name.lower()
    if n.startswith("void at::") or "at::native" in n or "cudnn" in n or "cublas" in n or "cutlass" in n or "nccl" in n:
        return False
    return any(f in n for f in OWN)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--depth", type=int, default=20)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--rows", type=int, default=70)
    ap.add_argument("--out", default=None)
    ap.add_argument("--gaps", type=int, default=0, help="also list the N largest idle gaps of the device inside the step")
    args = ap.parse_args(argv)
    from torch.profiler import ProfilerActivity, profile

    from tyr_b200.models import nanochat as nc
    from tyr_b200.train import nanochat_engine as eng

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    cfg = nc.depth_config(args.depth, max_seq_len=args.seq)
    hp = eng.Hyperparameters(device_batch_size=args.batch, max_seq_len=args.seq,
                             total_batch_size_tokens=args.batch * args.seq)
    tr = eng.NanoChatTrainer(cfg, hp, device=dev, seed=0)
    tok = torch.randint(0, cfg.vocab_size, (args.batch, args.seq + 1), device=dev)
    mb = [(tok[:, :-1].contiguous(), tok[:, 1:].contiguous())]
    for _ in range(3):
        tr.step(mb)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        tr.step(mb)
        torch.cuda.synchronize()
    rows = sorted(((e.device_time_total, e.count, e.key) for e in prof.key_averages() if e.device_time_total > 0),
                  reverse=True)
    own_t = sum(t for t, _, k in rows if is_own(k))
    own_n = sum(c for _, c, k in rows if is_own(k))
    all_t = sum(t for t, _, _ in rows)
    all_n = sum(c for _, c, _ in rows)
    lines = [f"{t / 1000:10.3f} ms  x{c:<5d} {'own' if is_own(k) else 'lib'}  {k[:130]}" for t, c, k in rows[:args.rows]]
    lines.append(f"total kernel time {all_t / 1000:.2f} ms in {all_n} launches; repository kernels "
                 f"{own_t / 1000:.2f} ms ({100 * own_t / max(all_t, 1):.1f} %) in {own_n} launches "
                 f"({100 * own_n / max(all_n, 1):.1f} %)")
    if args.gaps:
        # Idle time of the device inside the step: kernels sorted by start time, a gap is the time between the latest end
        # seen so far and the next start.
        evs = sorted(((e.time_range.start, e.time_range.end, e.name) for e in prof.events()
                      if str(e.device_type).endswith("CUDA") and e.time_range.end > e.time_range.start), key=lambda t: t[0])
        gaps, busy_end, prev = [], None, ""
        for st, en, name in evs:
            if busy_end is not None and st > busy_end:
                gaps.append((st - busy_end, prev, name, st - evs[0][0]))
            if busy_end is None or en > busy_end:
                busy_end, prev = en, name
        span = evs[-1][1] - evs[0][0] if evs else 0.0
        idle = sum(g[0] for g in gaps)
        lines.append(f"device span {span / 1000:.2f} ms, idle {idle / 1000:.2f} ms in {len(gaps)} gaps; "
                     f"gaps > 20 us: {sum(g[0] for g in gaps if g[0] > 20) / 1000:.2f} ms")
        for d, a_, b_, at in sorted(gaps, reverse=True)[:args.gaps]:
            lines.append(f"  gap {d:8.1f} us at +{at / 1000:7.2f} ms  after {a_[:60]}  before {b_[:60]}")
    text = "\n".join(lines)
    print(text)
    if args.out:
        with open(args.out, "w") as f:
            f.write(text + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
