"""Snapshot-directory checkpoint protocol (Tyr/Checkpoint.lean:42-302).

A save writes everything into a fresh ``.snapshots/snapshot-<ms>-<nonce>/`` directory and then
atomically renames a pointer file (``CURRENT``; optimizer state may use its own pointer such as
``OPTIMIZER_CURRENT``), so a crash mid-save leaves the previous snapshot intact and readers pin
exactly one snapshot.  A save that fails removes its partial snapshot.

What is interchangeable with the reference and what is not:

* pointer files hold the bare snapshot name (no separator, no dot), as the reference writes and
  requires (Checkpoint.lean:126-137); pointers written by earlier versions of this module
  (``.snapshots/<name>``) are still read;
* a directory without a pointer file is a flat legacy checkpoint and is returned unchanged
  (Checkpoint.lean:129);
* metadata is ``meta.txt`` holding the reference's version-2 JSON (``version``, ``iteration``,
  ``bestValLossBits``, ``trainLossBits``, ``optimCount``; losses as IEEE-754 bits); the reader also
  takes the reference's legacy ``key=value`` text and the ``meta.json`` of earlier versions of this
  module.  Fields the reference does not have (``extra``) go to ``meta_extra.json``;
* tensors: this module WRITES one safetensors file per tree prefix (tensors named by traversal path)
  plus ``<prefix>_count.txt``; the reference writes ``{prefix}_{i}.pt`` files with libtorch's
  ``torch::save(std::vector<Tensor>)`` (TorchScript archives).  :func:`load_reference_pt_layout`
  READS that layout; a reference build cannot read the safetensors trees written here.
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
from ..typed.dtype import DType
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


def publish_snapshot(root: str, snapshot_dir: str, pointer: str = CURRENT) -> None:
    """Atomically point ``pointer`` at ``snapshot_dir`` (the bare snapshot name is written)."""
    name = os.path.basename(os.path.normpath(snapshot_dir))
    if os.path.normpath(os.path.join(root, SNAPSHOTS, name)) != os.path.normpath(snapshot_dir):
        raise CheckpointError(f"{snapshot_dir} is not a snapshot of {root}")
    tmp = os.path.join(root, f".{pointer}.{secrets.token_hex(4)}.tmp")
    with open(tmp, "w") as f:
        f.write(name)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, os.path.join(root, pointer))
    _fsync_dir(root)


def discard_snapshot(snapshot_dir: str) -> None:
    """Remove a snapshot that was never published (a failed save)."""
    import shutil
    shutil.rmtree(snapshot_dir, ignore_errors=True)


def write_snapshot(root: str, write, pointer: str = CURRENT) -> str:
    """``write(snapshot_dir)`` into a fresh snapshot, then publish it; a failure removes the partial snapshot and is
    re-raised (Checkpoint.lean:142-152)."""
    snap = begin_snapshot(root)
    try:
        write(snap)
        publish_snapshot(root, snap, pointer)
    except BaseException:
        discard_snapshot(snap)
        raise
    return snap


def resolve_snapshot(root: str, pointer: str = CURRENT) -> str:
    """The directory readers should use for every file of one read.  No pointer file: ``root`` itself (a flat legacy
    checkpoint).  Raises when the pointer is malformed or names a missing snapshot."""
    cur = os.path.join(root, pointer)
    if not os.path.exists(cur):
        return root
    name = open(cur).read().strip()
    legacy_prefix = SNAPSHOTS + "/"
    if name.startswith(legacy_prefix):                      # pointer written by earlier versions of this module
        name = name[len(legacy_prefix):]
    if not name.startswith("snapshot-") or "/" in name or "\\" in name or "." in name:
        raise CheckpointError(f"Invalid checkpoint snapshot pointer: {cur}")
    path = os.path.join(root, SNAPSHOTS, name)
    if not os.path.isdir(path):
        raise CheckpointError(f"Missing checkpoint snapshot: {path}")
    return path


def has_checkpoint(root: str, pointer: str = CURRENT) -> bool:
    """A committed checkpoint with metadata exists (Checkpoint.lean:155-157)."""
    try:
        snap = resolve_snapshot(root, pointer)
    except CheckpointError:
        return False
    return any(os.path.exists(os.path.join(snap, n)) for n in (META_TXT, "meta.json"))


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


META_TXT = "meta.txt"
META_EXTRA = "meta_extra.json"


def _f2b(x: float) -> int:
    return struct.unpack("<Q", struct.pack("<d", float(x)))[0]


def _b2f(b: int) -> float:
    return struct.unpack("<d", struct.pack("<Q", int(b)))[0]


@dataclass
class CheckpointMeta:
    """``step`` = the reference's ``iteration``, ``loss_bits`` = ``trainLossBits``."""
    version: int = 2
    step: int = 0
    loss_bits: int = 0
    extra: Optional[dict] = None
    best_val_loss_bits: int = 0
    optim_count: int = 0

    @staticmethod
    def with_loss(step: int, loss: float, extra: Optional[dict] = None, best_val_loss: Optional[float] = None,
                  optim_count: int = 0) -> "CheckpointMeta":
        return CheckpointMeta(2, step, _f2b(loss), extra, _f2b(loss if best_val_loss is None else best_val_loss), optim_count)

    @property
    def loss(self) -> float:
        return _b2f(self.loss_bits)

    @property
    def best_val_loss(self) -> float:
        return _b2f(self.best_val_loss_bits)


def save_meta(snapshot_dir: str, meta: CheckpointMeta, name: str = META_TXT) -> None:
    """The reference's version-2 JSON (Checkpoint.lean:42-75), written through a temporary file and a rename."""
    body = {"version": 2, "iteration": int(meta.step), "bestValLossBits": int(meta.best_val_loss_bits),
            "trainLossBits": int(meta.loss_bits), "optimCount": int(meta.optim_count)}
    tmp = os.path.join(snapshot_dir, f".{name}.{secrets.token_hex(4)}.tmp")
    with open(tmp, "w") as f:
        json.dump(body, f, indent=2)
    os.replace(tmp, os.path.join(snapshot_dir, name))
    if meta.extra is not None:
        with open(os.path.join(snapshot_dir, META_EXTRA), "w") as f:
            json.dump(meta.extra, f)


def _parse_legacy_meta(text: str) -> CheckpointMeta:
    """``key=value`` lines: iteration, bestValLoss, trainLoss, optional optimCount (Checkpoint.lean:77-104)."""
    fields: Dict[str, str] = {}
    for raw in text.split("\n"):
        line = raw.strip()
        if not line:
            continue
        parts = line.split("=")
        if len(parts) != 2:
            raise CheckpointError(f"Malformed checkpoint metadata line: {line}")
        if parts[0] in fields:
            raise CheckpointError(f"Duplicate checkpoint metadata field: {parts[0]}")
        fields[parts[0]] = parts[1].strip()

    def need(k):
        if k not in fields:
            raise CheckpointError(f"Missing checkpoint metadata field: {k}")
        return fields[k]

    def nat(k, v):
        if not v.isdigit():
            raise CheckpointError(f"Invalid Nat value for {k}: {v}")
        return int(v)

    def flt(k, v):
        try:
            return float(json.loads(v))
        except Exception:
            raise CheckpointError(f"Invalid Float value for {k}: {v}") from None

    it = nat("iteration", need("iteration"))
    best = flt("bestValLoss", need("bestValLoss"))
    train = flt("trainLoss", need("trainLoss"))
    oc = nat("optimCount", fields.get("optimCount", "0"))
    return CheckpointMeta(2, it, _f2b(train), None, _f2b(best), oc)


def load_meta(snapshot_dir: str, name: Optional[str] = None) -> CheckpointMeta:
    """Reads ``meta.txt`` (version-2 JSON or legacy ``key=value`` text); falls back to the ``meta.json`` earlier versions
    of this module wrote."""
    cands = [name] if name else [META_TXT, "meta.json"]
    p = next((os.path.join(snapshot_dir, n) for n in cands if os.path.exists(os.path.join(snapshot_dir, n))), None)
    if p is None:
        raise CheckpointError(f"checkpoint {snapshot_dir} has no {cands[0]}")
    text = open(p).read()
    if not text.strip().startswith("{"):
        return _parse_legacy_meta(text)
    try:
        j = json.loads(text)
    except ValueError as e:
        raise CheckpointError(f"{p}: {e}") from None
    extra = None
    ep = os.path.join(snapshot_dir, META_EXTRA)
    if os.path.exists(ep):
        extra = json.load(open(ep))
    if "iteration" in j:                                     # the reference's schema
        if j.get("version") != 2:
            raise CheckpointError(f"Unsupported checkpoint metadata version: {j.get('version')}")
        return CheckpointMeta(2, int(j["iteration"]), int(j["trainLossBits"]), extra, int(j["bestValLossBits"]),
                              int(j.get("optimCount", 0)))
    if j.get("version") not in (1, 2):                       # earlier versions of this module
        raise CheckpointError(f"unsupported checkpoint metadata version {j.get('version')}")
    if j.get("version") == 1:
        return CheckpointMeta.with_loss(j.get("step", 0), j.get("loss", 0.0), j.get("extra"))
    return CheckpointMeta(2, j["step"], j["loss_bits"], j.get("extra"), j.get("best_val_loss_bits", j["loss_bits"]),
                          j.get("optim_count", 0))


def save_training_checkpoint(root: str, params, mu, nu, meta: CheckpointMeta) -> str:
    """params + first/second moments + metadata in ONE snapshot (Checkpoint.lean:284)."""
    def write(snap):
        save_tree(snap, "param", params)
        if mu is not None:
            save_tree(snap, "mu", mu)
        if nu is not None:
            save_tree(snap, "nu", nu)
        save_meta(snap, meta)
    return write_snapshot(root, write)


def load_training_checkpoint(root: str, params_template, mu_template=None, nu_template=None, device=None):
    snap = resolve_snapshot(root)
    params = load_tree(snap, "param", params_template, device)
    mu = load_tree(snap, "mu", mu_template, device) if mu_template is not None else None
    nu = load_tree(snap, "nu", nu_template, device) if nu_template is not None else None
    return params, mu, nu, load_meta(snap)


def load_reference_pt_tensor(path: str) -> torch.Tensor:
    """One ``.pt`` file as the reference writes it: libtorch ``torch::save(std::vector<Tensor>{t}, path)``
    (cc/src/tyr.cpp:2149-2151), i.e. a TorchScript archive whose single parameter is named "0".  ``torch.load`` with
    ``weights_only=True`` refuses such archives, so the file is opened with ``torch.jit.load``."""
    m = torch.jit.load(path, map_location="cpu")
    items = list(m.named_parameters()) + list(m.named_buffers())
    if len(items) != 1:
        raise CheckpointError(f"{path}: expected one tensor, found {len(items)}")
    return items[0][1].detach()


def load_reference_pt_layout(directory: str, prefix: str, template):
    """Read the reference's ``{prefix}_{i}.pt`` + ``{prefix}_count.txt`` layout (Checkpoint.lean:167-213): leaves in
    traversal order, count, shape and dtype validated against the template."""
    want = sch.schema_of(template)
    cpath = os.path.join(directory, f"{prefix}_count.txt")
    if os.path.exists(cpath):
        text = open(cpath).read().strip()
        if not text.isdigit():
            raise CheckpointError(f"Invalid checkpoint tensor count: {cpath}")
        if int(text) != len(want):
            raise CheckpointError(f"Checkpoint tensor count mismatch: expected {len(want)}, stored {int(text)}")
    tensors = {}
    for i, s in enumerate(want):
        t = load_reference_pt_tensor(os.path.join(directory, f"{prefix}_{i}.pt"))
        if tuple(t.shape) != tuple(s.shape):
            raise CheckpointError(f"checkpoint '{prefix}': leaf {i} ({s.path}) has shape {list(t.shape)}, expected {list(s.shape)}")
        if DType.of_torch(t.dtype) is not s.dtype:
            raise CheckpointError(f"checkpoint '{prefix}': leaf {i} ({s.path}) has dtype {t.dtype}, expected {s.dtype}")
        tensors[s.path] = t
    return sch.rebuild(template, tensors)
