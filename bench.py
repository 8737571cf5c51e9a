#!/usr/bin/env python
"""Headline benchmark: NanoChat d20 pre-training throughput (tokens/s) on N B200s of one node.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Model/config (the reference's d20: Examples/NanoChat/Pipeline.lean:167-244, ModdedGPT.lean):
20 layers, d_model 1280, 10 heads x 128, vocab 65536, seq 2048, 32 x 2048 tokens per GPU per
step, bf16 compute, Muon on matrices + AdamW on embeddings/head/scalars, synthetic Zipf(1.1)
token ids, random-init weights.  One step = forward + backward + optimizer update.

After the training half the same process measures the second half of the metric, Laguna MoE decode tokens/s
(``laguna_decode`` object of the same line; see :func:`laguna_decode_bench`), and with N > 1 a ``dp_selfcheck``
value (largest difference between any rank's parameters and rank 0's after the warm-up steps).

Prints ONE JSON line on rank 0.  ``value`` is the whole-job tokens/s over all N GPUs, timed on
the device with CUDA events around exactly K steps (max over ranks).  ``e2e`` repeats the
measurement through the public trainer entry (`NanoChatTrainer.train_step_from_host`): every step
copies that step's tokens from pinned host memory and reads the loss back to the host.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "nanochat_d20_train_tokens_per_s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "restated"])
    ap.add_argument("--depth", type=int, default=20)
    ap.add_argument("--device-batch", type=int, default=32)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--vocab", type=int, default=65536)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-laguna", action="store_true", help="skip the Laguna MoE decode half of the metric")
    ap.add_argument("--laguna-steps", type=int, default=48)
    ap.add_argument("--laguna-layers", type=int, default=24)
    ap.add_argument("--restated-micro-batch", type=int, default=4, help="--impl restated in fp32: rows per micro-batch")
    ap.add_argument("--restated-precision", default="fp32", choices=["fp32", "bf16"],
                    help="--impl restated: fp32 as the reference trains, or bf16 autocast (the generous reading)")
    return ap.parse_args()


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for nm, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def reference_arm(args):
    """The reference is a Lean 4 project (lakefile.lean + a C++ FFI library built by Lake); it has
    no Python packaging, so a `pip install` of its source tree cannot produce anything runnable and the
    Lean toolchain is not in this image."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    why = ("reference is a Lean 4 + LibTorch FFI project (no setup.py/pyproject; needs elan/Lean 4.29 "
           "and torch 2.10+cu130 wheels that are not in this offline image); pip install produced nothing runnable")
    if os.path.isdir(ref_dir) and any(n.endswith(".py") for n in os.listdir(ref_dir)):
        why = "baseline/_ref holds no runnable NanoChat trainer (Lean executable TrainNanoChat cannot be built offline)"
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def laguna_decode_bench(args, world, rank, device):
    """Second half of the headline metric: decode tokens/s of the Laguna-style NVFP4 MoE decoder
    (24 layers, d 2048, 16 q / 4 kv heads x 128, 64 routed experts top-8 + one shared expert, expert FFN 768;
    reference entry Examples/Laguna/RunHF.lean:90-122).  Every rank prefills 64 sequences x 64 tokens (4096 tokens) and
    then decodes with batch 64; with N > 1 ranks the experts are split over the ranks (expert parallel) and the rows
    travel through the fused dispatch / combine kernels over peer memory.  Device-timed exactly like the training half
    (CUDA events, max over ranks); the end-to-end figure copies each step's tokens from pinned host memory and reads the
    sampled tokens back every step."""
    import torch
    import torch.distributed as dist
    from tyr_b200.models import laguna as L
    from tyr_b200.ops import _common as opc

    B, S, K, W = 64, 64, args.laguna_steps, max(3, args.warmup)
    cfg = L.LagunaConfig(hidden_size=2048, intermediate_size=8192, num_hidden_layers=args.laguna_layers,
                         num_attention_heads=16, num_attention_heads_sliding=16, num_key_value_heads=4, num_experts=64,
                         num_experts_per_tok=8, moe_intermediate_size=768, shared_expert_intermediate_size=768)
    ep = None
    if world > 1:
        from tyr_b200.parallel.ep import ExpertParallel
        ep = ExpertParallel(rank, world, device, cfg.num_experts, cfg.hidden_size, B * S, cfg.num_experts_per_tok,
                            capacity_factor=min(world, 2))
    model = L.init(cfg, device=device, dtype=torch.bfloat16, ep=ep)
    ids = torch.randint(32, cfg.vocab_size, (B, S), device=device, generator=torch.Generator(device=device).manual_seed(rank))
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.no_grad():
        sess = L.CacheSession(model, B, S + 2 * (K + W) + 8)
        barrier()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        tok = sess.prefill(ids).argmax(-1)
        p1.record()
        for _ in range(W):                      # the first step captures the CUDA graph of the decode step
            tok = sess.step(tok).argmax(-1)
        barrier()
        opc.raise_on_device_error(device)
        launches0 = opc.LAUNCH_COUNT[0]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            flush.zero_()                       # L2 flush between steps: weights and caches come from HBM every step
            tok = sess.step(tok).argmax(-1)
        e1.record()
        barrier()
        launches = opc.LAUNCH_COUNT[0] - launches0
        opc.raise_on_device_error(device)
        # end to end: tokens come from pinned host memory, the sampled tokens go back to the host, every step
        host_in = tok.cpu().pin_memory()
        host_out = torch.empty_like(host_in).pin_memory()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(K):
            flush.zero_()
            t_dev = host_in.to(device, non_blocking=True)
            nxt = sess.step(t_dev).argmax(-1)
            host_out.copy_(nxt, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            host_in.copy_(host_out)
        f1.record()
        barrier()
    t = torch.tensor([e0.elapsed_time(e1), f0.elapsed_time(f1), p0.elapsed_time(p1)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dec_ms, e2e_ms, pre_ms = (float(x) for x in t.tolist())
    out = {"metric": "laguna_moe_decode_tokens_per_s", "value": B * world * K / (dec_ms / 1e3), "unit": "tokens/s",
           "ms_per_step": dec_ms / K, "steps": K, "warmup": W, "batch_per_gpu": B,
           "prefill_tokens": B * S * world, "prefill_ms": pre_ms, "prefill_tokens_per_s": B * S * world / (pre_ms / 1e3),
           "e2e": {"value": B * world * K / (e2e_ms / 1e3), "unit": "tokens/s",
                   "h2d_bytes_per_step": int(host_in.numel() * host_in.element_size()),
                   "d2h_bytes_per_step": int(host_out.numel() * host_out.element_size())},
           "gpu_launches": launches,
           "config": {"model": f"laguna-moe {cfg.num_hidden_layers} layers, d 2048, 16q/4kv x 128, 64 experts top-8 + shared, FFN 768, NVFP4",
                      "parallelism": f"ep{world}" if world > 1 else "1 GPU", "decode_step": "CUDA graph" if sess._graph is not None else "eager",
                      "l2": "256 MB buffer written between steps"}}
    if ep is not None:
        ep.close()
    return out


def dp_selfcheck(trainer, world, device):
    """max over ranks and parameters of |working copy on this rank - working copy on rank 0| (0.0 = the replicas agree
    bit for bit after the fused reduce-scatter / update / all-gather); run outside the timed region."""
    import torch
    import torch.distributed as dist
    worst = torch.zeros((), dtype=torch.float32, device=device)
    for name, w in trainer.params.work.items():
        ref = w.detach().clone()
        dist.broadcast(ref, src=0)
        worst = torch.maximum(worst, (w.detach().float() - ref.float()).abs().max())
        del ref
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    return float(worst.item())


def zipf_tokens(n_batches, batch, seq_plus_one, vocab, seed):
    import numpy as np
    import torch
    rng = np.random.default_rng(seed)
    z = rng.zipf(1.1, size=(n_batches, batch, seq_plus_one))
    tok = torch.from_numpy(((z - 1) % vocab).astype("int64"))
    return tok


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world and world == 1 and args.gpus > 1:
        print(json.dumps({"error": f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks"}))
        return 2
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    from tyr_b200.models import nanochat as nc
    from tyr_b200.ops import _common as opc
    from tyr_b200.train import nanochat_engine as eng

    cfg = nc.depth_config(args.depth, vocab_size=args.vocab, max_seq_len=args.seq_len)
    hp = eng.Hyperparameters(device_batch_size=args.device_batch, max_seq_len=args.seq_len,
                             total_batch_size_tokens=args.device_batch * args.seq_len * world)
    dp = None
    if world > 1:
        from tyr_b200.parallel.dp import FusedDataParallel
        dp = FusedDataParallel(rank=rank, world_size=world, device=device)
    if args.impl == "restated":
        from baseline.restated_reference import RestatedTrainer
        trainer = RestatedTrainer(cfg, hp, device=device, world_size=world, rank=rank, precision=args.restated_precision)
    else:
        trainer = eng.NanoChatTrainer(cfg, hp, device=device, compute_dtype=torch.bfloat16, seed=1234,
                                      world_size=world, rank=rank, dp=dp)

    B, T = args.device_batch, args.seq_len
    n_pool = 4
    host_tok = zipf_tokens(n_pool, B, T + 1, args.vocab, seed=1000 + rank).pin_memory()
    dev_tok = host_tok.to(device)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # the restated arm in fp32 accumulates the same 32 x 2048 tokens over micro-batches (its fp32 logits and activations
    # for all rows at once do not fit in 180 GB)
    micro = B
    if args.impl == "restated" and args.restated_precision == "fp32":
        micro = min(B, args.restated_micro_batch)

    def run_device_step(i):
        tok = dev_tok[i % n_pool]
        flush.zero_()  # L2 flush (256 MB > 126 MB L2) between iterations
        return trainer.step([(tok[r:r + micro, :-1], tok[r:r + micro, 1:]) for r in range(0, B, micro)])

    for i in range(args.warmup):
        run_device_step(i)
    barrier()
    opc.raise_on_device_error(device)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = opc.LAUNCH_COUNT[0]
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    last = None
    for i in range(args.steps):
        last = run_device_step(args.warmup + i)
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    launches = opc.LAUNCH_COUNT[0] - launches0
    clocks = sampler.stop() if rank == 0 else None
    opc.raise_on_device_error(device)
    final_loss = float(last.loss.item())

    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    tokens_per_step = B * T * world
    value = tokens_per_step * args.steps / (ms_max / 1e3)

    e2e = None
    if not args.no_e2e:
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            flush.zero_()
            loss_f = trainer.train_step_from_host(host_tok[(args.warmup + i) % n_pool])
        e1.record()
        barrier()
        t2 = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        e2e = {"value": tokens_per_step * args.steps / (float(t2.item()) / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": int(host_tok[0].numel() * host_tok.element_size()),
               "d2h_bytes_per_step": 4, "final_loss": loss_f}

    selfcheck = dp_selfcheck(trainer, world, device) if (world > 1 and args.impl == "ours") else None
    laguna = None
    if not args.no_laguna and args.impl == "ours":
        del trainer, dp, dev_tok, flush
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        try:
            laguna = laguna_decode_bench(args, world, rank, device)
        except Exception as e:                                   # the training half still reports
            laguna = {"metric": "laguna_moe_decode_tokens_per_s", "error": f"{type(e).__name__}: {e}"[:300]}

    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_max / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": args.restated_precision if args.impl == "restated" else "bf16",
            "data": "synthetic Zipf(1.1) token ids, random-init weights",
            "impl": "restated reference (PyTorch + NCCL restatement, not the reference itself)" if args.impl == "restated" else args.impl,
            "config": {"model": f"nanochat-d{args.depth} (dim {cfg.model_dim}, {cfg.n_head}x{cfg.head_dim} heads, vocab {cfg.vocab_size})",
                       "global_batch": B * world, "seq_len": T, "tokens_per_gpu_per_step": B * T,
                       "parallelism": f"dp{world}",
                       "optimizer": "Muon(matrices)+AdamW(embeddings,head,scalars)",
                       "l2": "256 MB buffer written between iterations (L2 flush); per-step working set >> 126 MB"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "final_loss": final_loss,
            "dp_selfcheck": selfcheck, "laguna_decode": laguna,
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
