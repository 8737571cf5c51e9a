"""Generator of a tiny Laguna parity fixture in the checkpoint layout the loaders read.

    python tests/fixtures/make_tiny_laguna.py OUT_DIR [--seed 1234] [--nvfp4]

Writes ``config.json`` (HF form), ``model.safetensors`` (bf16 weights under the checkpoint's tensor names; with ``--nvfp4`` the
routed experts as packed e2m1 + e4m3 block scales + fp32 global scales), ``reference.safetensors`` (fp32 logits and hidden
states of two prompts and of the last greedy step, computed on the CPU in fp32 from the bf16-rounded weights through the
un-fused path) and ``reference.json`` (prompts, 16 greedy token ids, seeds).  Every value is a function of the seed, so two
runs write identical bytes.  The reference project generates its checked-in fixture the same way from the vendor's PyTorch
implementation (scripts/laguna/make_tiny_fixture.py); this one uses this repository's fp32 forward as the oracle, which the
vendored fixture under tests/fixtures/reference/laguna/tiny pins in turn.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from tyr_b200.io import safetensors as st  # noqa: E402
from tyr_b200.models import laguna as lg  # noqa: E402

INPUT_A = [2, 37, 101, 456, 1000, 5, 9]
GEN_STEPS = 16


def tiny_config() -> lg.LagunaConfig:
    return lg.LagunaConfig(vocab_size=1024, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
                           num_attention_heads_sliding=6, num_key_value_heads=2, head_dim=16, half_rotary_dim_full=4,
                           half_rotary_dim_sliding=8, sliding_window=8, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32,
                           shared_expert_intermediate_size=32, yarn_original_max_position_embeddings=64)


def generate(out_dir: str, seed: int = 1234, nvfp4: bool = False) -> dict:
    os.makedirs(out_dir, exist_ok=True)
    cfg = tiny_config()
    torch.manual_seed(seed)
    model = lg.init(cfg, device="cpu", dtype=torch.float32, seed=seed, dense_experts=not nvfp4)
    # canonical weights = the bf16 rounding of the seeded draw; the checkpoint stores them, the references are computed from them
    sd = {k: (v.to(torch.bfloat16) if v.is_floating_point() and v.dtype in (torch.float32, torch.bfloat16) and "scale" not in k else v).contiguous()
          for k, v in lg.state_dict(model).items()}
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg.to_json(), f, indent=1, sort_keys=True)
    st.save_file(sd, os.path.join(out_dir, "model.safetensors"))
    m = lg.load_pretrained(out_dir, device="cpu", dtype=torch.float32)
    g = torch.Generator().manual_seed(seed + 1)
    input_b = [2] + torch.randint(3, cfg.vocab_size, (11,), generator=g).tolist()
    ids_a, ids_b = torch.tensor([INPUT_A]), torch.tensor([input_b])
    with torch.no_grad():
        ref = {"logits_a": lg.forward(m, ids_a, use_fused=False)[0], "logits_b": lg.forward(m, ids_b, use_fused=False)[0],
               "hidden_a_final": lg.forward_hidden(m, ids_a, use_fused=False)[0]}
        out = lg.generate_greedy(m, ids_a, max_new_tokens=GEN_STEPS, eos_token_ids=[])
        gen = out[0, len(INPUT_A):].tolist()
        full = torch.tensor([INPUT_A + gen[:GEN_STEPS - 1]])
        ref["gen_logits_last"] = lg.forward(m, full, use_fused=False)[0, -1]
    st.save_file({k: v.float().contiguous() for k, v in ref.items()}, os.path.join(out_dir, "reference.safetensors"))
    meta = {"input_ids_a": INPUT_A, "input_ids_b": input_b, "gen_ids": gen, "weight_seed": seed, "nvfp4": bool(nvfp4)}
    with open(os.path.join(out_dir, "reference.json"), "w") as f:
        json.dump(meta, f, indent=1, sort_keys=True)
    return meta


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("out_dir")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--nvfp4", action="store_true")
    a = ap.parse_args(argv)
    meta = generate(a.out_dir, a.seed, a.nvfp4)
    print(f"wrote {a.out_dir}: {len(meta['gen_ids'])} greedy ids, prompt b of {len(meta['input_ids_b'])} tokens")
    return 0


if __name__ == "__main__":
    sys.exit(main())
