"""Snapshot-directory checkpoint protocol (Tyr/Checkpoint.lean:42-302).

A save writes everything into a fresh ``.snapshots/snapshot-<ms>-<nonce>/`` directory and then
atomically renames a ``CURRENT`` pointer file, so a crash mid-save leaves the previous snapshot
intact and readers pin exactly one snapshot.  Leaves are stored as safetensors (one file per tree
prefix, tensors named by their traversal paths) with a ``<prefix>_count.txt`` beside it; loading
validates count, shape and dtype against a typed template.  Metadata (v2) stores the loss as
IEEE-754 bits.  A reader for the reference's own ``{prefix}_{i}.pt`` layout is provided for
compatibility.
"""
from __future__ import annotations

import json
import os
import secrets
import struct
import time
from dataclasses import dataclass, asdict
from typing import Dict, Optional

import torch

from ..struct import schema as sch
from ..struct.tree import leaves_with_paths
from ..typed.tensor import Tensor
from . import safetensors as st

CURRENT = "CURRENT"
SNAPSHOTS = ".snapshots"


class CheckpointError(IOError):
    pass


def _fsync_dir(path: str):
    try:
        fd = os.open(path, os.O_RDONLY)
        try:
            os.fsync(fd)
        finally:
            os.close(fd)
    except OSError:
        pass


def begin_snapshot(root: str) -> str:
    """Create and return a fresh snapshot directory (not yet visible to readers)."""
    snaps = os.path.join(root, SNAPSHOTS)
    os.makedirs(snaps, exist_ok=True)
    name = f"snapshot-{int(time.time() * 1000)}-{secrets.token_hex(4)}"
    path = os.path.join(snaps, name)
    os.makedirs(path)
    return path


def publish_snapshot(root: str, snapshot_dir: str) -> None:
    """Atomically point ``CURRENT`` at ``snapshot_dir``."""
    rel = os.path.relpath(snapshot_dir, root)
    tmp = os.path.join(root, f".{CURRENT}.{secrets.token_hex(4)}.tmp")
    with open(tmp, "w") as f:
        f.write(rel + "\n")
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, os.path.join(root, CURRENT))
    _fsync_dir(root)


def resolve_snapshot(root: str) -> str:
    """The snapshot directory readers should use; raises when there is no published snapshot or
    the pointer names a missing / escaping directory."""
    cur = os.path.join(root, CURRENT)
    if not os.path.exists(cur):
        raise CheckpointError(f"no checkpoint published in {root} (missing {CURRENT})")
    rel = open(cur).read().strip()
    if not rel or os.path.isabs(rel) or ".." in rel.split(os.sep):
        raise CheckpointError(f"checkpoint pointer in {root} is invalid: {rel!r}")
    path = os.path.join(root, rel)
    if not os.path.isdir(path):
        raise CheckpointError(f"checkpoint pointer names a missing snapshot: {rel}")
    return path


def has_checkpoint(root: str) -> bool:
    try:
        resolve_snapshot(root)
        return True
    except CheckpointError:
        return False


def save_tree(snapshot_dir: str, prefix: str, tree) -> int:
    flat = sch.flatten(tree)
    st.save_file({k: v for k, v in flat.items()}, os.path.join(snapshot_dir, f"{prefix}.safetensors"))
    with open(os.path.join(snapshot_dir, f"{prefix}_count.txt"), "w") as f:
        f.write(f"{len(flat)}\n")
    return len(flat)


def load_tree(snapshot_dir: str, prefix: str, template, device=None):
    """Load into the structure of ``template`` validating count, shape and dtype."""
    cpath = os.path.join(snapshot_dir, f"{prefix}_count.txt")
    fpath = os.path.join(snapshot_dir, f"{prefix}.safetensors")
    if not os.path.exists(cpath) or not os.path.exists(fpath):
        raise CheckpointError(f"checkpoint {snapshot_dir} has no '{prefix}' tree")
    want = sch.schema_of(template)
    try:
        count = int(open(cpath).read().strip())
    except ValueError:
        raise CheckpointError(f"{cpath} is not a number") from None
    if count != len(want):
        raise CheckpointError(f"checkpoint '{prefix}' holds {count} tensors, the template has {len(want)}")
    src = st.Source.open(fpath)
    tensors = {}
    for s in want:
        if src.find(s.path) is None:
            raise CheckpointError(f"checkpoint '{prefix}' is missing tensor {s.path}")
        shape, dtype = src.spec(s.path)
        if shape != s.shape:
            raise CheckpointError(f"checkpoint '{prefix}': {s.path} has shape {list(shape)}, expected {list(s.shape)}")
        if dtype is not s.dtype:
            raise CheckpointError(f"checkpoint '{prefix}': {s.path} has dtype {dtype}, expected {s.dtype}")
        t = src.load(s.path)
        tensors[s.path] = t.to(device) if device is not None else t
    # rebuild on the devices of the loaded tensors
    from ..struct.tree import with_leaves
    new = []
    for path, leaf, _ in leaves_with_paths(template):
        t = tensors[path]
        if device is None:
            t = t.to((leaf.raw if isinstance(leaf, Tensor) else leaf).device)
        new.append(Tensor.of_tensor(t) if isinstance(leaf, Tensor) else t)
    return with_leaves(template, new)


@dataclass
class CheckpointMeta:
    version: int = 2
    step: int = 0
    loss_bits: int = 0
    extra: Optional[dict] = None

    @staticmethod
    def with_loss(step: int, loss: float, extra: Optional[dict] = None) -> "CheckpointMeta":
        bits = struct.unpack("<Q", struct.pack("<d", float(loss)))[0]
        return CheckpointMeta(2, step, bits, extra)

    @property
    def loss(self) -> float:
        return struct.unpack("<d", struct.pack("<Q", self.loss_bits))[0]


def save_meta(snapshot_dir: str, meta: CheckpointMeta, name: str = "meta.json") -> None:
    with open(os.path.join(snapshot_dir, name), "w") as f:
        json.dump(asdict(meta), f)


def load_meta(snapshot_dir: str, name: str = "meta.json") -> CheckpointMeta:
    p = os.path.join(snapshot_dir, name)
    if not os.path.exists(p):
        raise CheckpointError(f"checkpoint {snapshot_dir} has no {name}")
    j = json.load(open(p))
    if j.get("version") not in (1, 2):
        raise CheckpointError(f"unsupported checkpoint metadata version {j.get('version')}")
    if j.get("version") == 1:  # v1 stored a decimal loss
        return CheckpointMeta.with_loss(j.get("step", 0), j.get("loss", 0.0), j.get("extra"))
    return CheckpointMeta(2, j["step"], j["loss_bits"], j.get("extra"))


def save_training_checkpoint(root: str, params, mu, nu, meta: CheckpointMeta) -> str:
    """params + first/second moments + metadata in ONE snapshot (Checkpoint.lean:284)."""
    snap = begin_snapshot(root)
    save_tree(snap, "param", params)
    if mu is not None:
        save_tree(snap, "mu", mu)
    if nu is not None:
        save_tree(snap, "nu", nu)
    save_meta(snap, meta)
    publish_snapshot(root, snap)
    return snap


def load_training_checkpoint(root: str, params_template, mu_template=None, nu_template=None, device=None):
    snap = resolve_snapshot(root)
    params = load_tree(snap, "param", params_template, device)
    mu = load_tree(snap, "mu", mu_template, device) if mu_template is not None else None
    nu = load_tree(snap, "nu", nu_template, device) if nu_template is not None else None
    return params, mu, nu, load_meta(snap)


def load_reference_pt_layout(directory: str, prefix: str, template):
    """Read the reference's ``{prefix}_{i}.pt`` + ``{prefix}_count.txt`` layout
    (Checkpoint.lean:167-213): leaves in traversal order, validated against the template."""
    want = sch.schema_of(template)
    count = int(open(os.path.join(directory, f"{prefix}_count.txt")).read().strip())
    if count != len(want):
        raise CheckpointError(f"checkpoint '{prefix}' holds {count} tensors, the template has {len(want)}")
    tensors = {}
    for i, s in enumerate(want):
        t = torch.load(os.path.join(directory, f"{prefix}_{i}.pt"), map_location="cpu", weights_only=True)
        tensors[s.path] = t
    return sch.rebuild(template, tensors)
