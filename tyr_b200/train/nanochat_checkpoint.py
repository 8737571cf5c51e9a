"""Checkpoint / resume for NanoChat training: model weights by reference names, an optimizer-state sidecar per
rank, the data-stream cursor and a meta file, published atomically as a snapshot
(Examples/NanoChat/ModdedTrain.lean:420-836; snapshot layout of Tyr/Checkpoint.lean)."""
from __future__ import annotations

import json
import os
from dataclasses import asdict
from typing import Optional, Tuple

import torch

from ..data.loader import DistributedDataGenerator, StreamCursor
from ..io import checkpoint as ckpt
from ..io import safetensors as st
from ..models import nanochat as nc
from .nanochat_engine import Hyperparameters, NanoChatTrainer

MODEL_FILE, META_FILE = "model.safetensors", "meta.json"


def _opt_file(rank: int) -> str:
    return f"optimizer.rank{rank}.safetensors"


def _cursor_file(rank: int) -> str:
    return f"cursor.rank{rank}.json"


def save(root: str, trainer: NanoChatTrainer, data: Optional[DistributedDataGenerator], loss: float,
         barrier=None, extra: Optional[dict] = None) -> str:
    """All ranks call this.  Rank 0 creates the snapshot and writes the weights; every rank writes its optimizer
    sidecar and cursor; rank 0 publishes after a barrier."""
    rank, world = trainer.rank, trainer.world_size
    if trainer.dp is not None and world > 1:
        trainer.dp.gather_master(trainer)
    snap_holder = [None]
    if rank == 0:
        snap_holder[0] = ckpt.begin_snapshot(root)
    if world > 1:
        import torch.distributed as dist
        dist.broadcast_object_list(snap_holder, src=0)
    snap = snap_holder[0]
    if rank == 0:
        named = {k: v.detach().float().cpu().contiguous() for k, v in trainer.params.named_parameters("master").items()}
        st.save_file(named, os.path.join(snap, MODEL_FILE))
        meta = {"step": trainer.step_index, "loss": float(loss), "world_size": world, "config": trainer.cfg.to_json(),
                "hyperparameters": trainer.hp.to_json()}
        if extra:
            meta["extra"] = extra
        with open(os.path.join(snap, META_FILE), "w") as f:
            json.dump(meta, f, indent=2)
        # the reference's metadata file (iteration / loss bits / optimizer step count) beside the run description above
        ckpt.save_meta(snap, ckpt.CheckpointMeta.with_loss(trainer.step_index, float(loss), optim_count=trainer.step_index))
    sd = {k: v.detach().cpu().contiguous() for k, v in trainer.optimizer_state_dict().items()}
    st.save_file(sd, os.path.join(snap, _opt_file(rank)))
    if data is not None:
        with open(os.path.join(snap, _cursor_file(rank)), "w") as f:
            f.write(data.cursor().to_json())
    if barrier is not None:
        barrier()
    if rank == 0:
        ckpt.publish_snapshot(root, snap)
    return snap


def load(root: str, trainer: NanoChatTrainer, data: Optional[DistributedDataGenerator] = None, weights_only: bool = False) -> dict:
    """Restore weights, this rank's optimizer state and data cursor from the published snapshot; returns the meta.
    ``weights_only`` takes just the parameters (the next stage of a recipe starts its own optimizer and step count)."""
    snap = ckpt.resolve_snapshot(root)
    meta = json.load(open(os.path.join(snap, META_FILE)))
    if meta["config"] != trainer.cfg.to_json():
        raise ckpt.CheckpointError("checkpoint was written for a different model configuration")
    if weights_only:
        src = st.Source.open(os.path.join(snap, MODEL_FILE))
        trainer.params.load_named({n: src.load(n) for n in src.names()})
        if trainer.dp is not None and trainer.world_size > 1 and hasattr(trainer.dp, "scatter_master"):
            trainer.dp.scatter_master(trainer)
        return meta
    if meta["world_size"] != trainer.world_size:
        raise ckpt.CheckpointError(f"checkpoint was written by {meta['world_size']} ranks, this run has {trainer.world_size}")
    src = st.Source.open(os.path.join(snap, MODEL_FILE))
    trainer.params.load_named({n: src.load(n) for n in src.names()})
    if trainer.dp is not None and trainer.world_size > 1 and hasattr(trainer.dp, "scatter_master"):
        trainer.dp.scatter_master(trainer)
    osrc = st.Source.open(os.path.join(snap, _opt_file(trainer.rank)))
    trainer.load_optimizer_state_dict({n: osrc.load(n).to(trainer.device) if "step" not in n else osrc.load(n) for n in osrc.names()})
    trainer.step_index = int(meta["step"])
    cpath = os.path.join(snap, _cursor_file(trainer.rank))
    if data is not None and os.path.exists(cpath):
        data.restore_cursor(StreamCursor.from_json(open(cpath).read()))
    return meta
