"""Qwen3.5 / Qwen3.6 text generation and throughput CLI (counterpart of Examples/Qwen35/RunHF.lean).

    python -m tyr_b200.cli.run_qwen35 --source Qwen/Qwen3.5-9B --prompt "..." --max-new-tokens 64 --stream
    python -m tyr_b200.cli.run_qwen35 --random-init --preset 27b --bench --batch-size 32 --prompt-tokens 2048 --max-new-tokens 256
    torchrun --nproc-per-node 8 -m tyr_b200.cli.run_qwen35 --random-init --preset 27b --tp --bench ...

``--tp`` (under torchrun) shards heads, MLP columns and the vocabulary over the ranks and runs the fused
GEMM+collective kernels; without it every process holds the whole model.  ``--bench`` prints prefill and decode
tokens/s from CUDA events (max over ranks).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from ..io import hub
from ..models import qwen35 as Q
from ..models.generation import SamplingStrategy

PRESETS = {"0.8b": Q.Qwen35Config.qwen35_0_8b, "9b": Q.Qwen35Config.qwen35_9b, "27b": Q.Qwen35Config.qwen35_27b,
           "35b-a3b": Q.Qwen35Config.qwen35_35b_a3b, "3.6-35b-a3b": Q.Qwen35Config.qwen36_35b_a3b}


def parse(argv):
    p = argparse.ArgumentParser(prog="run_qwen35")
    p.add_argument("--source", default="Qwen/Qwen3.5-9B")
    p.add_argument("--revision", default=None)
    p.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    p.add_argument("--prompt", default="Explain NVLink in one sentence.")
    p.add_argument("--batch-size", type=int, default=1)
    p.add_argument("--max-new-tokens", type=int, default=64)
    p.add_argument("--stream", action="store_true")
    p.add_argument("--no-thinking", action="store_true")
    p.add_argument("--bench", action="store_true")
    p.add_argument("--random-init", action="store_true")
    p.add_argument("--preset", default="9b", choices=sorted(PRESETS))
    p.add_argument("--layers", type=int, default=None)
    p.add_argument("--prompt-tokens", type=int, default=2048)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-k", type=int, default=None)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--tp", action="store_true", help="under torchrun: tensor parallel over all ranks")
    p.add_argument("--json", action="store_true", help="with --bench: print one JSON line")
    return p.parse_args(argv)


def _time_phase(fn, dev):
    if dev.type != "cuda":
        import time
        t0 = time.perf_counter()
        out = fn()
        return out, (time.perf_counter() - t0) * 1e3
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    a.record()
    out = fn()
    b.record()
    torch.cuda.synchronize(dev)
    return out, a.elapsed_time(b)


def bench(make_cache, ids, new_tokens, dev, group=None):
    """Greedy prefill + ``new_tokens`` decode steps, after one warm-up pass on a throwaway cache."""
    B, S = ids.shape
    warm = make_cache(S + 4)
    warm.step(warm.prefill(ids).argmax(-1))
    del warm
    cache = make_cache(S + new_tokens + 1)
    logits, pre_ms = _time_phase(lambda: cache.prefill(ids), dev)

    first = cache.step(logits.argmax(-1)).argmax(-1)          # untimed: the first step of a cache captures its CUDA graph
    new_tokens = max(1, new_tokens - 1)

    def decode():
        tok = first
        for _ in range(new_tokens):
            tok = cache.step(tok).argmax(-1)
        return tok
    _, dec_ms = _time_phase(decode, dev)
    if group is not None or (dist.is_available() and dist.is_initialized()):
        t = torch.tensor([pre_ms, dec_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        pre_ms, dec_ms = t.tolist()
    return {"prefill_ms": pre_ms, "prefill_tok_s": B * S / pre_ms * 1e3, "decode_ms": dec_ms, "decode_tok_s": B * new_tokens / dec_ms * 1e3,
            "batch": B, "prompt_tokens": S, "new_tokens": new_tokens}


def main(argv=None):
    a = parse(sys.argv[1:] if argv is None else argv)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    dev = torch.device(a.device)
    if world > 1:
        if dev.type == "cuda":
            dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
            torch.cuda.set_device(dev)
            dist.init_process_group("nccl", device_id=dev)
        else:
            dist.init_process_group("gloo")
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    say = (lambda *x: print(*x, flush=True)) if rank == 0 else (lambda *x: None)
    tok = None
    if a.random_init:
        cfg = PRESETS[a.preset]()
        if a.layers:
            import dataclasses
            cfg = dataclasses.replace(cfg, num_hidden_layers=a.layers, layer_types=None)
        ids = torch.randint(0, cfg.vocab_size, (a.batch_size, a.prompt_tokens), generator=torch.Generator().manual_seed(1)).to(dev)
    else:
        from ..tokenizer import hf as tok_hf
        model_dir = hub.resolve_pretrained_dir(a.source, revision=a.revision)
        cfg = Q.Qwen35Config.load_from_pretrained_dir(model_dir)
        tok = tok_hf.load_qwen3(model_dir)
        text = tok_hf.chatml_prompt([{"role": "user", "content": a.prompt}]) + ("<think>\n\n</think>\n\n" if a.no_thinking else "")
        ids = torch.tensor([tok.encode(text)] * a.batch_size, device=dev)
    tp_on = a.tp and world > 1
    if tp_on:
        from ..models import qwen35_tp as QT
        from ..parallel.tp import TensorParallel
        rows = a.batch_size * ids.shape[1]
        tp = TensorParallel(rank, world, dev, max_rows=max(rows, 128 * world), max_cols=cfg.hidden_size, max_k=cfg.hidden_size,
                            gather_elems=a.batch_size * -(-cfg.vocab_size // world))
        if a.random_init:
            model = QT.init_sharded(cfg, rank, world, tp, dev, dtype)
        else:
            model = QT.shard(Q.load(cfg, model_dir, "cpu", dtype), rank, world, tp)
            model = _to_device(model, dev)
        make_cache = lambda n: QT.TPCache(model, ids.shape[0], n)
        gen = lambda on_step: QT.generate(model, ids, a.max_new_tokens, _strategy(a), on_step=on_step)
    else:
        model = Q.init(cfg, dev, dtype) if a.random_init else Q.load(cfg, model_dir, dev, dtype, log=say)
        make_cache = lambda n: Q.HybridCache(model, ids.shape[0], n)
        gen = lambda on_step: Q.generate(model, ids, a.max_new_tokens, _strategy(a), on_step=on_step)
    if a.bench:
        with torch.no_grad():
            r = bench(make_cache, ids, a.max_new_tokens, dev)
        r.update(model=a.preset if a.random_init else a.source, layers=cfg.num_hidden_layers, tp=world if tp_on else 1, dtype=str(dtype).split(".")[-1])
        if a.json:
            say(json.dumps(r))
        else:
            say(f"prefill: {r['prompt_tokens']} x {r['batch']} tokens in {r['prefill_ms']:.1f} ms = {r['prefill_tok_s']:.0f} tok/s")
            say(f"decode:  {r['new_tokens']} x {r['batch']} tokens in {r['decode_ms']:.1f} ms = {r['decode_tok_s']:.0f} tok/s")
    else:
        on_step = None
        if a.stream and tok is not None and rank == 0:
            on_step = lambda step, t: print(tok.decode([int(t[0])]), end="", flush=True)
        out = gen(on_step)
        if tok is not None and not a.stream:
            for row in out.tolist():
                say(tok.decode(row[ids.shape[1]:]))
        elif tok is None:
            say(out[:, ids.shape[1]:].tolist())
    if tp_on:
        tp.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


def _strategy(a):
    return SamplingStrategy.greedy() if a.temperature <= 0 else SamplingStrategy.multinomial(a.temperature, a.top_k, a.top_p)


def _to_device(m, dev):
    import dataclasses

    def mv(o):
        if isinstance(o, torch.Tensor):
            return o.to(dev)
        if dataclasses.is_dataclass(o) and not isinstance(o, (type, Q.Qwen35Config)):
            return dataclasses.replace(o, **{f.name: mv(getattr(o, f.name)) for f in dataclasses.fields(o)})
        if isinstance(o, list):
            return [mv(x) for x in o]
        return o
    return mv(m)


if __name__ == "__main__":
    sys.exit(main())
