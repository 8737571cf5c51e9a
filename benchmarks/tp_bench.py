"""Fused tensor-parallel GEMMs against the NCCL formulation of the same ops.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m benchmarks.tp_bench

Shapes: Qwen3.5-27B-like row-parallel projections (hidden 5120; attention output 24*256 and FFN 17408
input channels split over the ranks) and the matching column-parallel projections, for a prefill batch
of 16384 tokens.  Times are CUDA-event medians over 10 iterations after 3 warm-ups, max over ranks;
the roofline is max(FLOPs / measured GEMM peak, bytes over NVLink / 770 GB/s per direction).
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist

from tyr_b200.parallel.tp import TensorParallel


def _time(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    t = torch.tensor(sorted(ts)[len(ts) // 2], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    M, H = 16384, 5120
    tp = TensorParallel(rank, world, dev, max_rows=M, max_cols=H, max_k=H)
    peak = 1.4e15
    results = []
    for name, k_total in (("attn_out", 24 * 256), ("ffn_down", 17408)):
        kl = (k_total // world + 7) // 8 * 8
        x = (torch.randn(M, kl, device=dev) * 0.1).bfloat16()
        w = (torch.randn(H, kl, device=dev) * 0.02).bfloat16()
        out_nccl = torch.empty(M // world, H, device=dev, dtype=torch.bfloat16)

        def nccl():
            y = torch.matmul(x, w.T)
            dist.reduce_scatter_tensor(out_nccl, y)
        t_f = _time(lambda: tp.gemm_reduce_scatter(x, w))
        t_n = _time(nccl)
        flops = 2.0 * M * H * kl
        link = M * H * 2 * (world - 1) / world
        roof = max(flops / peak, link / 770e9) * 1e3
        results.append({"op": f"gemm_rs_{name}", "world": world, "fused_ms": t_f, "nccl_ms": t_n, "roofline_ms": roof,
                        "fused_frac_of_roofline": roof / t_f})
    for name, n_total in (("qkv", 24 * 256 * 2 + 2 * 4 * 256), ("ffn_gate_up", 2 * 17408)):
        nl = (n_total // world + 7) // 8 * 8
        xs = (torch.randn(M // world, H, device=dev) * 0.1).bfloat16()
        w = (torch.randn(nl, H, device=dev) * 0.02).bfloat16()
        full = torch.empty(M, H, device=dev, dtype=torch.bfloat16)

        def nccl():
            dist.all_gather_into_tensor(full, xs)
            return torch.matmul(full, w.T)
        t_f = _time(lambda: tp.allgather_gemm(xs, w))
        t_n = _time(nccl)
        flops = 2.0 * M * H * nl
        link = M * H * 2 * (world - 1) / world
        roof = max(flops / peak, link / 770e9) * 1e3
        results.append({"op": f"ag_gemm_{name}", "world": world, "fused_ms": t_f, "nccl_ms": t_n, "roofline_ms": roof,
                        "fused_frac_of_roofline": roof / t_f})
    if rank == 0:
        for r in results:
            print(f"{r['op']:24s} tp{world}: fused {r['fused_ms']:7.3f} ms | matmul+NCCL {r['nccl_ms']:7.3f} ms | roofline {r['roofline_ms']:6.3f} ms", flush=True)
        print(json.dumps(results))
    tp.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
