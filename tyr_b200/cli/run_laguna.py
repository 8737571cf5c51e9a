"""Laguna text generation / throughput CLI (counterpart of Examples/Laguna/RunHF.lean).

    python -m tyr_b200.cli.run_laguna --source <dir|repo> --prompt "..." --max-new-tokens 64 --stream
    python -m tyr_b200.cli.run_laguna --random-init --layers 8 --bench --prompt-tokens 4096 --batch-size 64

``--random-init`` builds the Laguna-S-2.1 architecture with synthetic NVFP4 banks (no checkpoint or
tokenizer needed) and feeds random token ids; ``--bench`` prints prefill and decode tokens/s
measured with CUDA events around the two phases.
"""
from __future__ import annotations

import argparse
import sys
import time

import torch

from ..io import hub
from ..models import laguna as L
from ..models.generation import SamplingStrategy
from ..tokenizer import hf as tok_hf


def parse(argv):
    p = argparse.ArgumentParser(prog="run_laguna")
    p.add_argument("--source", default="poolside/Laguna-S-2.1-NVFP4", help="model directory or hub repo id")
    p.add_argument("--revision", default=None)
    p.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    p.add_argument("--prompt", default="Write a haiku about GPUs.")
    p.add_argument("--prompt-file", default=None, help="one prompt per non-empty line")
    p.add_argument("--batch-size", type=int, default=1)
    p.add_argument("--max-new-tokens", type=int, default=64)
    p.add_argument("--stream", action="store_true")
    p.add_argument("--no-thinking", action="store_true")
    p.add_argument("--debug-ids", action="store_true")
    p.add_argument("--bench", action="store_true")
    p.add_argument("--random-init", action="store_true")
    p.add_argument("--layers", type=int, default=None, help="with --random-init: number of decoder layers")
    p.add_argument("--shape", default="laguna-s", choices=["laguna-s", "moe-24x2048"],
                   help="with --random-init: Laguna-S-2.1 (hidden 3072, 256 experts top-10, FFN 1024) or the 24-layer benchmark shape "
                        "(hidden 2048, 16 q / 4 kv heads x 128, 64 experts top-8 + shared, FFN 768)")
    p.add_argument("--prompt-tokens", type=int, default=4096, help="with --random-init: synthetic prompt length")
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-k", type=int, default=None)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--ep", action="store_true",
                   help="under torchrun: split the experts over the ranks (expert parallel), every rank decodes its own batch")
    return p.parse_args(argv)


def _sync(dev):
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)


def bench(model, input_ids, max_new_tokens, eos=()):
    """Returns dict(prefill_ms, prefill_tok_s, decode_ms, decode_tok_s); greedy, no early stop unless eos given."""
    dev = input_ids.device
    B, S = input_ids.shape
    with torch.no_grad():
        warm = L.CacheSession(model, B, S + 4)
        warm.step(warm.prefill(input_ids).argmax(-1))
        del warm
        sess = L.CacheSession(model, B, S + max_new_tokens)
        _sync(dev)
        t0 = time.perf_counter()
        logits = sess.prefill(input_ids)
        tok = logits.argmax(-1)
        _sync(dev)
        t1 = time.perf_counter()
        tok = sess.step(tok).argmax(-1)            # untimed: the first step of a session captures its CUDA graph
        _sync(dev)
        t2 = time.perf_counter()
        n = 0
        for _ in range(max_new_tokens - 2):
            tok = sess.step(tok).argmax(-1)
            n += 1
        _sync(dev)
        t3 = time.perf_counter()
    pre_ms, dec_ms = (t1 - t0) * 1e3, (t3 - t2) * 1e3
    return {"prompt_tokens": B * S, "prefill_ms": pre_ms, "prefill_tok_s": B * S / pre_ms * 1e3,
            "decode_tokens": B * n, "decode_ms": dec_ms, "decode_tok_s": (B * n / dec_ms * 1e3) if n else 0.0,
            "first_step_ms": (t2 - t1) * 1e3, "batch": B}


def main(argv=None) -> int:
    a = parse(sys.argv[1:] if argv is None else argv)
    import os
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    ep = None
    if a.ep and world > 1:
        import torch.distributed as dist
        local = int(os.environ.get("LOCAL_RANK", "0"))
        if a.device.startswith("cuda"):
            torch.cuda.set_device(local)
            a.device = f"cuda:{local}"
            dist.init_process_group("nccl", device_id=torch.device(a.device))
        else:
            dist.init_process_group("gloo")
    dev = torch.device(a.device)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    strategy = (SamplingStrategy.greedy() if a.temperature <= 0 else
                SamplingStrategy.multinomial(a.temperature, a.top_k, a.top_p))
    if a.random_init:
        if a.shape == "moe-24x2048":
            cfg = L.LagunaConfig(hidden_size=2048, intermediate_size=8192, num_hidden_layers=a.layers or 24, num_attention_heads=16,
                                 num_attention_heads_sliding=16, num_key_value_heads=4, num_experts=64, num_experts_per_tok=8,
                                 moe_intermediate_size=768, shared_expert_intermediate_size=768)
        else:
            cfg = L.LagunaConfig(num_hidden_layers=a.layers) if a.layers else L.LagunaConfig()
        if a.ep and world > 1:
            from ..parallel.ep import ExpertParallel
            ep = ExpertParallel(rank, world, dev, cfg.num_experts, cfg.hidden_size, a.batch_size * a.prompt_tokens,
                                cfg.num_experts_per_tok, capacity_factor=min(world, 2))
        if rank == 0:
            print(f"Random-init Laguna: {cfg.num_hidden_layers} layers, hidden {cfg.hidden_size}, {cfg.num_experts} experts "
                  f"top-{cfg.num_experts_per_tok}" + (f", expert parallel over {world} ranks" if ep else ""), flush=True)
        model = L.init(cfg, device=dev, dtype=dtype, ep=ep)
        ids = torch.randint(32, cfg.vocab_size, (a.batch_size, a.prompt_tokens), device=dev,
                            generator=torch.Generator(device=dev).manual_seed(rank))
        if a.bench:
            r = bench(model, ids, a.max_new_tokens)
            if ep is not None:
                import torch.distributed as dist
                t = torch.tensor([r["prefill_ms"], r["decode_ms"]], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                r["prefill_ms"], r["decode_ms"] = t.tolist()
                r["prompt_tokens"] *= world
                r["decode_tokens"] *= world
                r["prefill_tok_s"] = r["prompt_tokens"] / r["prefill_ms"] * 1e3
                r["decode_tok_s"] = r["decode_tokens"] / r["decode_ms"] * 1e3 if r["decode_ms"] else 0.0
            if rank == 0:
                print(f"BENCH prompt_tokens={r['prompt_tokens']} prefill_ms={r['prefill_ms']:.1f} prefill_tok_s={r['prefill_tok_s']:.1f}")
                print(f"BENCH decode_tokens={r['decode_tokens']} decode_ms={r['decode_ms']:.1f} decode_tok_s={r['decode_tok_s']:.1f} "
                      f"batch={r['batch']} ranks={world}")
            if ep is not None:
                ep.close()
                dist.destroy_process_group()
            return 0
        out = L.generate(model, ids, a.max_new_tokens, strategy, eos_token_ids=())
        print(out[:, a.prompt_tokens:].tolist())
        return 0
    model_dir = hub.resolve_pretrained_dir(a.source, a.revision)
    cfg = L.LagunaConfig.load_from_pretrained_dir(model_dir)
    tok = tok_hf.load_laguna(model_dir)
    model = L.load(cfg, model_dir, device=dev, dtype=dtype, log=lambda s: print(s, flush=True))
    prompts = [a.prompt]
    if a.prompt_file:
        prompts = [l.strip() for l in open(a.prompt_file, encoding="utf-8") if l.strip()]
    if a.bench:
        prompts = prompts[:1]
    for b0 in range(0, len(prompts), a.batch_size):
        chunk = prompts[b0:b0 + a.batch_size]
        enc = [tok_hf.laguna_encode(tok, tok_hf.laguna_prompt(p, not a.no_thinking)) for p in chunk]
        width = max(len(e) for e in enc)
        # left-pad so every row's last prompt token sits at the same position
        ids = torch.tensor([[tok_hf.LAGUNA_PAD_ID] * (width - len(e)) + e for e in enc], device=dev)
        if a.bench:
            print("Warming up...\nMeasuring...", flush=True)
            r = bench(model, ids, a.max_new_tokens, cfg.eos_token_ids)
            print(f"BENCH prompt_tokens={r['prompt_tokens']} prefill_ms={r['prefill_ms']:.1f} prefill_tok_s={r['prefill_tok_s']:.1f}")
            print(f"BENCH decode_tokens={r['decode_tokens']} decode_ms={r['decode_ms']:.1f} decode_tok_s={r['decode_tok_s']:.1f}")
            return 0
        cb = None
        if a.stream and len(chunk) == 1:
            cb = lambda i, t: print(tok.decode([int(t[0])]), end="", flush=True)
        out = L.generate(model, ids, a.max_new_tokens, strategy, on_step=cb)
        if cb is not None:
            print()
        for row, p in zip(out.tolist(), chunk):
            gen = row[width:]
            if not (a.stream and len(chunk) == 1):
                print(f"### {p}\n{tok.decode(gen)}")
            if a.debug_ids:
                print(f"ids: {gen}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
