"""Shared runner for the pretrained text families (counterpart of Examples/ModelRunner.lean and the per-family RunHF
executables: Qwen3, Qwen2.5-Omni thinker, Qwen3.5 / 3.6, Gemma 4) plus the speech demos (Whisper, Qwen3-ASR).

    python -m tyr_b200.cli.model_runner --family gemma4 --source google/gemma-4-e2b --prompt "Hi" --max-new-tokens 64 --stream
    python -m tyr_b200.cli.model_runner --family qwen3 --source Qwen/Qwen3-4B --prompt-file prompts.txt --batch-size 4
    python -m tyr_b200.cli.model_runner --family whisper --source openai/whisper-small --audio speech.wav

Common flags: ``--source`` (directory or hub repo id), ``--prompt`` / ``--prompt-file``, ``--batch-size``, ``--max-new-tokens``,
``--stream``, ``--device`` (auto | cpu | cuda | cuda:N, falling back to CPU with a warning), ``--bench``.
"""
from __future__ import annotations

import argparse
import sys
import time
from typing import Callable, List, Optional, Tuple

import torch

from ..io import hub
from ..models.generation import SamplingStrategy
from ..tokenizer import hf as tok_hf

TEXT_FAMILIES = ("qwen3", "qwen25omni", "qwen35", "gemma4")
SPEECH_FAMILIES = ("whisper", "qwen3asr")


def resolve_device(arg: str) -> Tuple[torch.device, Optional[str]]:
    """(device, warning).  Unknown selectors and CUDA requests on a machine without CUDA fall back to CPU."""
    req = arg.strip().lower()
    cuda = torch.cuda.is_available()
    if req == "auto":
        return torch.device("cuda" if cuda else "cpu"), None
    if req == "cpu":
        return torch.device("cpu"), None
    if req == "cuda" or req.startswith("cuda:"):
        idx = req[5:] if req.startswith("cuda:") else "0"
        if not idx.isdigit():
            return torch.device("cpu"), f"Warning: invalid device selector '{arg}'; falling back to CPU."
        if not cuda:
            return torch.device("cpu"), f"Warning: --device {req} requested but CUDA is unavailable; falling back to CPU."
        return torch.device("cuda", int(idx)), None
    return torch.device("cpu"), f"Warning: invalid device selector '{arg}'; falling back to CPU."


def load_prompts(prompt_file: Optional[str], default: str) -> List[str]:
    if not prompt_file:
        return [default]
    prompts = [l.strip() for l in open(prompt_file, encoding="utf-8") if l.strip()]
    if not prompts:
        raise ValueError(f"prompt file {prompt_file} has no non-empty lines")
    return prompts


def batches(xs: List, n: int):
    for i in range(0, len(xs), max(1, n)):
        yield xs[i:i + max(1, n)]


def left_pad(rows: List[List[int]], pad: int) -> torch.Tensor:
    w = max(len(r) for r in rows)
    return torch.tensor([[pad] * (w - len(r)) + r for r in rows])


def load_text_family(family: str, model_dir: str, device, dtype):
    """Returns (generate(ids, max_new, strategy, on_step) -> ids, tokenizer, render(prompt) -> str, eos ids, pad id)."""
    if family in ("qwen3", "qwen25omni"):
        from ..models import qwen as Q
        lm = Q.load_qwen25_omni_thinker(model_dir, device, dtype) if family == "qwen25omni" else Q.load_from_pretrained(model_dir, device, dtype)
        tok = tok_hf.load_qwen3(model_dir)
        eos = [i for i in (tok.token_id("<|im_end|>"), tok.token_id("<|endoftext|>")) if i is not None]
        gen = lambda ids, n, st, cb: Q.generate(lm, ids, n, st, eos, cb)
        return gen, tok, lambda p: tok_hf.chatml_prompt([{"role": "user", "content": p}]), eos, eos[-1] if eos else 0
    if family == "qwen35":
        from ..models import qwen35 as Q5
        m = Q5.load_pretrained(model_dir, device, dtype)
        tok = tok_hf.load_qwen3(model_dir)
        eos = [i for i in (tok.token_id("<|im_end|>"), tok.token_id("<|endoftext|>")) if i is not None]
        gen = lambda ids, n, st, cb: Q5.generate(m, ids, n, st, eos, cb)
        return gen, tok, lambda p: tok_hf.chatml_prompt([{"role": "user", "content": p}]), eos, eos[-1] if eos else 0
    if family == "gemma4":
        from ..models import gemma4 as G
        cfg = G.Gemma4Config.load_from_pretrained_dir(model_dir)
        files = hub.shard_files(model_dir)
        from ..io import safetensors as st
        m = G.load(cfg, st.Source.open(model_dir if len(files) != 1 else files[0]), device, dtype)
        tok = tok_hf.load_gemma4(model_dir)
        gen = lambda ids, n, st_, cb: G.generate(m, ids, n, st_, cfg.eos_token_id, cb)
        return gen, tok, lambda p: tok_hf.gemma_prompt([{"role": "user", "content": p}]), list(cfg.eos_token_id), cfg.pad_token_id or 0
    raise ValueError(f"unknown text family {family}")


def run_text(a, device, dtype, out=print) -> int:
    model_dir = hub.resolve_pretrained_dir(a.source, a.revision)
    gen, tok, render, eos, pad = load_text_family(a.family, model_dir, device, dtype)
    strategy = SamplingStrategy.greedy() if a.temperature <= 0 else SamplingStrategy.multinomial(a.temperature, a.top_k, a.top_p)
    prompts = load_prompts(a.prompt_file, a.prompt)
    for chunk in batches(prompts, a.batch_size):
        ids = left_pad([tok.encode(render(p)) for p in chunk], pad).to(device)
        on_step = None
        if a.stream and len(chunk) == 1:
            on_step = lambda step, t: print(tok.decode([int(t[0])], skip_special=True), end="", flush=True)
        t0 = time.perf_counter()
        res = gen(ids, a.max_new_tokens, strategy, on_step)
        if device.type == "cuda":
            torch.cuda.synchronize(device)
        dt = time.perf_counter() - t0
        new = res[:, ids.shape[1]:]
        if on_step is not None:
            print()
        else:
            for p, row in zip(chunk, new.tolist()):
                cut = next((i for i, t in enumerate(row) if t in eos), len(row))
                out(f"> {p}\n{tok.decode(row[:cut], skip_special=True)}")
        if a.bench:
            out(f"BENCH batch={len(chunk)} prompt_tokens={ids.shape[1]} new_tokens={new.shape[1]} seconds={dt:.3f} tok_s={new.numel() / dt:.1f}")
    return 0


def run_speech(a, device, dtype, out=print) -> int:
    if not a.audio:
        print("--audio is required for speech families", file=sys.stderr)
        return 2
    model_dir = hub.resolve_pretrained_dir(a.source, a.revision)
    if a.family == "whisper":
        from ..models import whisper as W
        r = W.transcribe_wav(W.load_from_pretrained_dir(model_dir, device, dtype), a.audio)
        out(r.text)
        return 0
    import json
    import os
    from ..audio import frontend as fe
    from ..models import qwen3_asr as A
    cfg = A.Qwen3ASRConfig.from_json(json.load(open(os.path.join(model_dir, "config.json"))))
    files = hub.shard_files(model_dir)
    from ..io import safetensors as st
    m = A.load(cfg, st.Source.open(model_dir if len(files) != 1 else files[0]), device, dtype)
    tok = tok_hf.load_qwen3(model_dir)
    wave, rate = fe.load_mono_pcm16_wav(a.audio)
    r = A.transcribe_waveform(m, tok.encode, lambda ids: tok.decode(ids, skip_special=False), wave, rate, language=a.language, max_new_tokens=a.max_new_tokens)
    out(f"[{r.language}] {r.text}")
    return 0


def parse(argv):
    p = argparse.ArgumentParser(prog="model_runner")
    p.add_argument("--family", required=True, choices=TEXT_FAMILIES + SPEECH_FAMILIES)
    p.add_argument("--source", required=True)
    p.add_argument("--revision", default=None)
    p.add_argument("--prompt", default="Hello!")
    p.add_argument("--prompt-file", default=None)
    p.add_argument("--audio", default=None)
    p.add_argument("--language", default=None)
    p.add_argument("--batch-size", type=int, default=1)
    p.add_argument("--max-new-tokens", type=int, default=64)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-k", type=int, default=None)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--stream", action="store_true")
    p.add_argument("--bench", action="store_true")
    p.add_argument("--device", default="auto")
    return p.parse_args(argv)


def main(argv=None) -> int:
    a = parse(sys.argv[1:] if argv is None else argv)
    device, warn = resolve_device(a.device)
    if warn:
        print(warn, file=sys.stderr)
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    return run_speech(a, device, dtype) if a.family in SPEECH_FAMILIES else run_text(a, device, dtype)


if __name__ == "__main__":
    sys.exit(main())
