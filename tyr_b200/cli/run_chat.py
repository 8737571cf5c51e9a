"""Chat with a NanoChat checkpoint (counterpart of Examples/NanoChat/RunChat.lean).

    python -m tyr_b200.cli.run_chat --base-dir ~/.cache/nanochat --stage sft --prompt "What is 2+2?" --chat-markers
    python -m tyr_b200.cli.run_chat --checkpoint <dir> --tokenizer <dir> --interactive

The checkpoint is a published snapshot directory of the trainer (``checkpoints/<stage>`` under the base directory unless
``--checkpoint`` is given); the model shape comes from its ``meta.json``.  ``--chat-markers`` wraps the prompt as
``<|bos|><|user_start|>...<|user_end|><|assistant_start|>`` and stops at ``<|assistant_end|>``; generation runs on the
row-state engine, so calculator tool blocks are executed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional

import torch

from ..io import checkpoint as snap
from ..io import safetensors as st
from ..models import nanochat as nc
from ..nanochat.generator import EngineConfig, SpecialTokens, session_runner
from ..nanochat.inference import NanoChatSession
from ..tokenizer.bpe import BPETokenizer


def parse(argv):
    p = argparse.ArgumentParser(prog="run_chat")
    p.add_argument("--base-dir", default=os.environ.get("NANOCHAT_DIR", "~/.cache/nanochat"))
    p.add_argument("--checkpoint", default=None)
    p.add_argument("--stage", default="sft", choices=["base", "mid", "sft", "rl"])
    p.add_argument("--tokenizer", default=None)
    p.add_argument("--prompt", default=None)
    p.add_argument("--max-new-tokens", type=int, default=128)
    p.add_argument("--temperature", type=float, default=0.8)
    p.add_argument("--top-k", type=int, default=50)
    p.add_argument("--eos-token", type=int, default=None)
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--interactive", action="store_true")
    p.add_argument("--chat-markers", action="store_true")
    p.add_argument("--show-tokens", action="store_true")
    p.add_argument("--device", default=os.environ.get("TYR_DEVICE", "cuda" if torch.cuda.is_available() else "cpu"))
    p.add_argument("prompt_words", nargs="*")
    return p.parse_args(argv)


def load_model(checkpoint_dir: str, device):
    """Returns (params dict on ``device``, model config) from a published trainer snapshot."""
    s = snap.resolve_snapshot(checkpoint_dir)
    meta = json.load(open(os.path.join(s, "meta.json")))
    cfg = nc.Config.from_json(meta["config"])
    src = st.Source.open(os.path.join(s, "model.safetensors"))
    dtype = torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32
    master = {n: src.load(n) for n in src.names()}
    holder = nc.ModdedGPTParams(cfg, device=device, compute_dtype=dtype, seed=0)
    holder.load_named(master)
    holder.sync_work_from_master()
    return {k: v.detach() for k, v in holder.named_parameters("work").items()}, cfg


class Chat:
    def __init__(self, params, cfg: nc.Config, tok: BPETokenizer, max_new_tokens=128, temperature=0.8, top_k: Optional[int] = 50,
                 eos_token: Optional[int] = None, chat_markers=False, seed=42):
        self.params, self.cfg, self.tok, self.chat_markers = params, cfg, tok, chat_markers
        s = tok.encode_special
        self.bos = s("<|bos|>")
        end = eos_token if eos_token is not None else (s("<|assistant_end|>") if chat_markers else self.bos)
        self.specials = SpecialTokens(eot=end, bot=self.bos, tool_start=s("<|python_start|>"), tool_end=s("<|python_end|>"),
                                      output_start=s("<|output_start|>"), output_end=s("<|output_end|>"),
                                      calc_start=s("<|python_start|>"), calc_end=s("<|python_end|>"))
        self.engine_cfg = EngineConfig(temperature=temperature, top_k=top_k, max_tokens=max_new_tokens)
        self.gen = torch.Generator().manual_seed(seed)
        self.history: List[int] = [self.bos]

    def prompt_tokens(self, text: str) -> List[int]:
        ids = self.tok.encode_ordinary(text)
        if not self.chat_markers:
            return self.history + ids
        s = self.tok.encode_special
        return self.history + [s("<|user_start|>")] + ids + [s("<|user_end|>"), s("<|assistant_start|>")]

    def reply(self, text: str, keep_history: bool = False):
        """Returns (reply text, reply token ids)."""
        prompt = self.prompt_tokens(text)
        room = self.cfg.max_seq_len - len(prompt) - 1
        if room <= 0:
            raise ValueError("prompt does not fit the model's context")
        engine = EngineConfig(self.engine_cfg.temperature, self.engine_cfg.top_p, self.engine_cfg.top_k, min(self.engine_cfg.max_tokens, room)).create(self.specials)
        dev = self.params["embed"].device
        sess = NanoChatSession(self.params, self.cfg, 1, self.cfg.max_seq_len)
        if len(prompt) > 1:
            sess.prefill(torch.tensor([prompt[:-1]], device=dev))
        out = engine.generate_one(prompt, session_runner(sess), self.tok.decode, self.tok.encode_ordinary, generator=self.gen)
        new = out[len(prompt):]
        if keep_history:
            self.history = out if out and out[-1] == self.specials.eot else out + [self.specials.eot]
        shown = [t for t in new if t != self.specials.eot]
        return self.tok.decode(shown), new


def main(argv=None) -> int:
    a = parse(sys.argv[1:] if argv is None else argv)
    base = os.path.expanduser(a.base_dir)
    ckpt_dir = os.path.expanduser(a.checkpoint) if a.checkpoint else os.path.join(base, "checkpoints", a.stage)
    tok_dir = os.path.expanduser(a.tokenizer) if a.tokenizer else os.path.join(base, "tokenizer")
    tok_file = tok_dir if os.path.isfile(tok_dir) else os.path.join(tok_dir, "tokenizer.bin")
    if not os.path.exists(tok_file):
        print(f"tokenizer not found: {tok_file}", file=sys.stderr)
        return 1
    try:
        params, cfg = load_model(ckpt_dir, a.device)
    except (FileNotFoundError, snap.CheckpointError) as e:
        print(f"checkpoint not usable: {e}", file=sys.stderr)
        return 1
    tok = BPETokenizer.load(tok_file)
    chat = Chat(params, cfg, tok, a.max_new_tokens, a.temperature, a.top_k if a.top_k > 0 else None, a.eos_token, a.chat_markers, a.seed)
    prompt = a.prompt if a.prompt is not None else (" ".join(a.prompt_words) if a.prompt_words else None)

    def turn(text, keep):
        reply, ids = chat.reply(text, keep_history=keep)
        print(reply, flush=True)
        if a.show_tokens:
            print(f"[tokens] {ids}", flush=True)
    if prompt is not None:
        turn(prompt, a.interactive)
    if a.interactive:
        while True:
            try:
                line = input("> ")
            except EOFError:
                break
            if line.strip() in ("/quit", "/exit"):
                break
            if line.strip() == "/reset":
                chat.history = [chat.bos]
                continue
            if line.strip():
                turn(line, True)
    elif prompt is None:
        print("nothing to do: give --prompt or --interactive", file=sys.stderr)
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main())
