"""`python -m tyr_b200.cli.train_gpt [--data FILE] [--config NAME] [--iters N]` - the reference's
TrainGPT executable (Examples/TrainGPT.lean:83-196).  Device from ``TYR_DEVICE`` (default CPU);
falls back to random tokens when no data file is given (:171-174)."""
from __future__ import annotations

import argparse
import sys

import torch

from ..models import gpt
from ..train import gpt_train
from ..typed import get_best_device, Device


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", default=None, help="text file; characters become tokens")
    ap.add_argument("--config", default="nanogpt_cpu_shakespeare")
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    import os
    device = get_best_device() if os.environ.get("TYR_DEVICE") else Device.CPU
    cfg = getattr(gpt.Config, a.config)()
    if a.data:
        text = open(a.data, encoding="utf-8").read()
        chars = sorted(set(text))
        stoi = {c: i for i, c in enumerate(chars)}
        data = torch.tensor([stoi[c] % cfg.vocab_size for c in text], dtype=torch.int64)
    else:
        print("no data file: training on random tokens")
        data = torch.randint(0, cfg.vocab_size, (100000,))
    n = int(0.9 * data.numel())
    params = gpt.GPTParams.init(cfg, device, seed=a.seed)
    tc = gpt_train.TrainConfig(max_iters=a.iters, batch_size=a.batch_size, block_size=cfg.block_size, device=device)
    gpt_train.train_loop(tc, params, data[:n], log=print, val_data=data[n:])
    return 0


if __name__ == "__main__":
    sys.exit(main())
