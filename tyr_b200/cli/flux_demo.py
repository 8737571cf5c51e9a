"""Text-to-image demo and denoiser benchmark for Flux Klein (counterpart of Examples/Flux/FluxDemo.lean).

    python -m tyr_b200.cli.flux_demo --qwen-dir Q --flux-path F.safetensors --vae-path V.safetensors --prompt "a fox"
    python -m tyr_b200.cli.flux_demo --random-init --bench --latent-h 64 --latent-w 64 --steps 4

Pipeline: Qwen3 text encoder (hidden states of layers 8/17/26 concatenated) -> rectified-flow
denoising of packed latents -> BN de-normalisation, unpack, VAE decode -> binary PPM.
``--random-init --bench`` times denoising steps on random weights of the Klein-4B architecture.
"""
from __future__ import annotations

import argparse
import sys
import time

import torch

from ..io import media
from ..models import flux as FX
from ..models import qwen as Q
from ..models import vae as V
from ..tokenizer import hf as tok_hf

MAX_SEQ = 512


def parse(argv):
    p = argparse.ArgumentParser(prog="flux_demo")
    p.add_argument("--qwen-dir")
    p.add_argument("--flux-path")
    p.add_argument("--vae-path")
    p.add_argument("--prompt", default="a photo of a red fox in the snow")
    p.add_argument("--steps", type=int, default=4)
    p.add_argument("--latent-h", type=int, default=16)
    p.add_argument("--latent-w", type=int, default=16)
    p.add_argument("--output", default="flux_out.ppm")
    p.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--random-init", action="store_true")
    p.add_argument("--bench", action="store_true")
    p.add_argument("--batch", type=int, default=1)
    p.add_argument("--kernel-shares", action="store_true", help="with --bench: kernel time shares of one denoising step")
    p.add_argument("--txt-len", type=int, default=MAX_SEQ)
    return p.parse_args(argv)


def encode_prompt(tok, prompt: str, max_len: int = MAX_SEQ):
    ids = tok.encode(tok_hf.chatml_prompt([{"role": "user", "content": prompt}], enable_thinking=False))[:max_len]
    pad = tok.token_id("<|endoftext|>") or 0
    mask = [1] * len(ids) + [0] * (max_len - len(ids))
    return torch.tensor([ids + [pad] * (max_len - len(ids))]), torch.tensor([mask])


def main(argv=None) -> int:
    a = parse(sys.argv[1:] if argv is None else argv)
    dev = torch.device(a.device)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    cfg = FX.FluxConfig.klein4b()
    img_ids = FX.compute_image_position_ids(a.latent_h, a.latent_w, dev).expand(a.batch, -1, -1)
    txt_ids = FX.compute_text_position_ids(a.txt_len, dev).expand(a.batch, -1, -1)
    gen = torch.Generator().manual_seed(a.seed)
    if a.random_init:
        print("=== Flux Klein 4B (random weights) ===", flush=True)
        model = FX.init(cfg, device=dev, dtype=dtype, seed=a.seed)
        txt = torch.randn((a.batch, a.txt_len, cfg.context_in_dim), generator=gen).to(device=dev, dtype=dtype)
    else:
        if not (a.qwen_dir and a.flux_path and a.vae_path):
            print("need --qwen-dir, --flux-path and --vae-path (or --random-init)", file=sys.stderr)
            return 2
        if (a.latent_h, a.latent_w) != (16, 16):
            print(f"the VAE decode path expects 16x16 latents, got {a.latent_h}x{a.latent_w}", file=sys.stderr)
            return 2
        print("=== Flux Klein 4B Demo ===\nLoading models...", flush=True)
        emb = Q.load_qwen_flux_embedder(a.qwen_dir, max_seq=MAX_SEQ, device=dev, dtype=dtype)
        if emb.output_dim() != cfg.context_in_dim:
            raise SystemExit(f"text encoder emits {emb.output_dim()} features, Flux expects {cfg.context_in_dim}")
        model = FX.load(cfg, a.flux_path, device=dev, dtype=dtype, log=print)
        ae = V.load_auto_encoder(a.vae_path, device=dev, dtype=torch.float32, log=print)
        tok = tok_hf.load_qwen3(a.qwen_dir)
        tokens, mask = encode_prompt(tok, a.prompt)
        print(f"  [1/4] Encoding text... tokens: {int(mask.sum())}", flush=True)
        txt = emb.encode_masked(tokens.to(dev), mask.to(dev)).to(dtype)
    noise = torch.randn((a.batch, 128, a.latent_h, a.latent_w), generator=gen).permute(0, 2, 3, 1).reshape(a.batch, -1, 128)
    noise = noise.to(device=dev, dtype=dtype)
    if a.bench:
        for _ in range(3):                                   # warm-up: module loading, workspaces, clocks
            FX.denoise(model, noise, txt, img_ids, txt_ids, 1)
        toks = a.batch * (noise.shape[1] + a.txt_len)
        if dev.type == "cuda":
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            FX.denoise(model, noise, txt, img_ids, txt_ids, a.steps)
            e1.record()
            torch.cuda.synchronize()
            dt = e0.elapsed_time(e1) / 1e3                   # device time of the whole sampling run
        else:
            t0 = time.perf_counter()
            FX.denoise(model, noise, txt, img_ids, txt_ids, a.steps)
            dt = time.perf_counter() - t0
        print(f"BENCH steps={a.steps} batch={a.batch} ms_per_step={dt / a.steps * 1e3:.2f} it_s={a.steps / dt:.3f} "
              f"tokens_per_step={toks} images_per_s={a.batch / dt:.3f}")
        if a.kernel_shares and dev.type == "cuda":
            from torch.profiler import ProfilerActivity, profile
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                FX.denoise(model, noise, txt, img_ids, txt_ids, 1)
                torch.cuda.synchronize()
            rows = sorted(((e.device_time_total, e.count, e.key) for e in prof.key_averages() if e.device_time_total > 0), reverse=True)
            total = sum(r[0] for r in rows)
            print(f"kernel time of one denoising step: {total / 1e3:.2f} ms in {sum(r[1] for r in rows)} launches")
            for t_us, n, k in rows[:14]:
                print(f"  {t_us / 1e3:8.3f} ms  {100 * t_us / total:5.1f} %  x{n:<4d} {k[:100]}")
        return 0
    print("  [3/4] Running Flux denoising...", flush=True)
    latents = FX.denoise(model, noise, txt, img_ids, txt_ids, a.steps)
    if a.random_init:
        print(f"latents: {tuple(latents.shape)} mean {latents.float().mean().item():.4f}")
        return 0
    packed = latents.float().reshape(1, a.latent_h, a.latent_w, 128).permute(0, 3, 1, 2)
    print("  [4/4] Decoding with VAE...", flush=True)
    image = ae.decode(packed)
    media.save_ppm(a.output, image[0].clamp(-1, 1).add(1).mul(0.5).cpu())
    print(f"  Image saved to {a.output}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
