"""NanoChat / modded-nanogpt pretraining entry point (counterpart of Examples/NanoChat/TrainNanoChat.lean).

    python -m tyr_b200.cli.train_nanochat --data data/fineweb10B --val data/fineweb_val --checkpoint-dir ckpt --depth 20
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m tyr_b200.cli.train_nanochat ...

Flags: --data --val --checkpoint-dir --resume --iterations --local-rank/--local_rank --debug, plus --depth,
--device-batch-size, --seq-len, --total-batch-tokens, --save-every, --eval-every, --log-every, --synthetic.
Distributed runs read RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* (torchrun) and use the fused data-parallel
optimizer step over the symmetric heap.  ``--synthetic`` trains on Zipf-distributed random tokens (no data files).
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import torch

from ..data import loader as dl
from ..models import nanochat as nc
from ..pipeline import resolve_training_device
from ..train import nanochat_checkpoint as nck
from ..train import nanochat_engine as eng
from ..train import run_ledger as rl
from ..utils.log import Handlers


def parse(argv):
    p = argparse.ArgumentParser(prog="train_nanochat")
    p.add_argument("--data", default="data/fineweb10B")
    p.add_argument("--val", default="data/fineweb_val")
    p.add_argument("--checkpoint-dir", default="checkpoints/modded")
    p.add_argument("--resume", default=None, help="checkpoint directory to resume from")
    p.add_argument("--iterations", type=int, default=None)
    p.add_argument("--local-rank", "--local_rank", type=int, default=None)
    p.add_argument("--debug", action="store_true", help="small model and batch")
    p.add_argument("--depth", type=int, default=20)
    p.add_argument("--device-batch-size", type=int, default=None)
    p.add_argument("--seq-len", type=int, default=None)
    p.add_argument("--total-batch-tokens", type=int, default=None)
    p.add_argument("--save-every", type=int, default=0)
    p.add_argument("--eval-every", type=int, default=0)
    p.add_argument("--eval-batches", type=int, default=8)
    p.add_argument("--log-every", type=int, default=10)
    p.add_argument("--synthetic", action="store_true")
    p.add_argument("--seed", type=int, default=0)
    return p.parse_args(argv)


def build_config(a):
    if a.debug:
        cfg = nc.Config(vocab_size=4096, n_layer=7, n_head=2, half_head_dim=32, max_seq_len=a.seq_len or 256)
        hp = eng.Hyperparameters(device_batch_size=a.device_batch_size or 4, max_seq_len=cfg.max_seq_len,
                                 total_batch_size_tokens=a.total_batch_tokens or 4 * cfg.max_seq_len,
                                 num_iterations=a.iterations or 20)
        return cfg, hp
    cfg = nc.depth_config(a.depth, max_seq_len=a.seq_len or 2048)
    hp = eng.Hyperparameters(device_batch_size=a.device_batch_size or 32, max_seq_len=cfg.max_seq_len)
    if a.total_batch_tokens:
        hp.total_batch_size_tokens = a.total_batch_tokens
    if a.iterations:
        hp.num_iterations = a.iterations
    return cfg, hp


class SyntheticStream:
    def __init__(self, cfg, hp, rank):
        self.cfg, self.hp, self.i, self.rank = cfg, hp, 0, rank

    def next_batch(self, B, T):
        t = dl.synthetic_zipf_tokens(B * T + 1, self.cfg.vocab_size, seed=self.rank * 1000003 + self.i)
        self.i += 1
        return t[:-1].reshape(B, T), t[1:].reshape(B, T)


@torch.no_grad()
def evaluate(trainer, stream, batches, B, T, device):
    tot = 0.0
    for _ in range(batches):
        x, y = stream.next_batch(B, T)
        tot += float(nc.loss_fused(trainer.params, x.to(device), y.to(device), trainer.ce_chunk_rows).item())
    return tot / max(1, batches)


def main(argv=None) -> int:
    a = parse(sys.argv[1:] if argv is None else argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = a.local_rank if a.local_rank is not None else int(os.environ.get("LOCAL_RANK", "0"))
    device = resolve_training_device(rank, local, world > 1)
    log = Handlers.stdout().master_only(rank)
    dp = None
    if world > 1:
        import torch.distributed as dist
        if device.type == "cuda":
            torch.cuda.set_device(device)
            dist.init_process_group("nccl", device_id=device)
            from ..parallel.dp import FusedDataParallel
            dp = FusedDataParallel(rank, world, device)
        else:
            dist.init_process_group("gloo")
    cfg, hp = build_config(a)
    eng.validate_grad_accum_config(hp, world)
    accum = eng.effective_grad_accum_steps(hp, world)
    log.on_info(f"NanoChat: {cfg.n_layer} layers, dim {cfg.model_dim}, vocab {cfg.vocab_size}, seq {cfg.max_seq_len}; "
                f"{world} rank(s) on {device}; {accum} micro-batch(es) of {hp.device_batch_size} x {hp.max_seq_len} per step")
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    trainer = eng.NanoChatTrainer(cfg, hp, device=device, compute_dtype=dtype, seed=a.seed, world_size=world, rank=rank, dp=dp)
    if a.synthetic:
        train, val, gen = SyntheticStream(cfg, hp, rank), SyntheticStream(cfg, hp, 7777 + rank), None
    else:
        gen = dl.DistributedDataGenerator(dl.LoaderConfig(a.data, seed=a.seed, batch_size=hp.device_batch_size, seq_len=hp.max_seq_len), rank, world)
        vgen = dl.DistributedDataGenerator(dl.LoaderConfig(a.val, seed=a.seed, shuffle=False, batch_size=hp.device_batch_size,
                                                           seq_len=hp.max_seq_len), rank, world) if a.eval_every else None
        train = type("S", (), {"next_batch": lambda self, B, T: gen.next_batch(B, T)})()
        val = type("S", (), {"next_batch": lambda self, B, T: vgen.next_batch(B, T)})() if vgen else None
    art = rl.RunArtifacts.of_base_dir(a.checkpoint_dir)
    if rank == 0:
        rl.prepare(art, {"config": cfg.to_json(), "hyperparameters": hp.to_json(), "world_size": world})
    ckpt_root = os.path.join(a.checkpoint_dir, "checkpoints")
    if a.resume:
        meta = nck.load(a.resume if os.path.isdir(os.path.join(a.resume, "snapshots")) else os.path.join(a.resume, "checkpoints"), trainer, gen)
        if a.synthetic:
            train.i = trainer.step_index * accum           # the synthetic stream is a function of the batch index
        log.on_info(f"Resumed from step {meta['step']} (loss {meta['loss']:.4f})")
    barrier = (lambda: torch.distributed.barrier()) if world > 1 else None
    B, T = hp.device_batch_size, hp.max_seq_len
    t_last, tok_last = time.perf_counter(), 0
    loss = float("nan")
    while trainer.step_index < hp.num_iterations:
        step = trainer.step_index
        micro = []
        for _ in range(accum):
            x, y = train.next_batch(B, T)
            micro.append((x.to(device, non_blocking=True), y.to(device, non_blocking=True)))
        res = trainer.step(micro)
        tok_last += res.tokens_processed * world
        if a.log_every and step % a.log_every == 0:
            loss = float(res.loss.item())
            if device.type == "cuda":
                torch.cuda.synchronize()
            dt = time.perf_counter() - t_last
            tps = tok_last / dt if dt > 0 else 0.0
            log.on_info(f"Step {step} | loss {loss:.4f} | {tps:,.0f} tok/s | {dt * 1e3 / max(1, a.log_every):.1f} ms/step")
            if rank == 0:
                rl.append_metric_event(art, rl.MetricEvent("train", step, [("loss", loss), ("tokens_per_s", tps)]))
            t_last, tok_last = time.perf_counter(), 0
        if a.eval_every and val is not None and step > 0 and step % a.eval_every == 0:
            vl = evaluate(trainer, val, a.eval_batches, B, T, device)
            log.on_info(f"Step {step} | val loss {vl:.4f}")
            if rank == 0:
                rl.append_metric_event(art, rl.MetricEvent("val", step, [("loss", vl)]))
        if a.save_every and trainer.step_index % a.save_every == 0:
            snap = nck.save(ckpt_root, trainer, gen, loss, barrier)
            if rank == 0:
                rl.append_checkpoint_event(art, rl.CheckpointEvent(f"step{trainer.step_index}", snap, "train", trainer.step_index, [("loss", loss)]))
    snap = nck.save(ckpt_root, trainer, gen, loss, barrier)
    if rank == 0:
        rl.append_checkpoint_event(art, rl.CheckpointEvent("final", snap, "train", trainer.step_index, [("loss", loss)]))
    log.on_info(f"Finished at step {trainer.step_index}; checkpoint {snap}")
    if dp is not None:
        dp.close()
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
