"""Hugging Face repo id -> local directory (Tyr/Hub.lean:54-244): cache lookup in the standard HF
cache layout, optional download with ``curl`` (no network here, so downloads fail with a clear
message), shard list from ``model.safetensors.index.json``."""
from __future__ import annotations

import json
import os
import shutil
import subprocess
from typing import List, Optional


class HubError(IOError):
    pass


def hf_cache_root() -> str:
    if os.environ.get("HF_HUB_CACHE"):
        return os.environ["HF_HUB_CACHE"]
    home = os.environ.get("HF_HOME", os.path.join(os.path.expanduser("~"), ".cache", "huggingface"))
    return os.path.join(home, "hub")


def repo_cache_dir(repo_id: str) -> str:
    return os.path.join(hf_cache_root(), "models--" + repo_id.replace("/", "--"))


def find_cached_snapshot(repo_id: str, revision: Optional[str] = None) -> Optional[str]:
    base = repo_cache_dir(repo_id)
    snaps = os.path.join(base, "snapshots")
    if not os.path.isdir(snaps):
        return None
    if revision is None:
        ref = os.path.join(base, "refs", "main")
        if os.path.exists(ref):
            revision = open(ref).read().strip()
    if revision and os.path.isdir(os.path.join(snaps, revision)):
        return os.path.join(snaps, revision)
    cands = sorted(os.listdir(snaps))
    return os.path.join(snaps, cands[-1]) if cands else None


def shard_files(directory: str) -> List[str]:
    idx = os.path.join(directory, "model.safetensors.index.json")
    if os.path.exists(idx):
        wm = json.load(open(idx)).get("weight_map", {})
        return sorted(set(wm.values()))
    return ["model.safetensors"]


def ensure_remote_file(repo_id: str, filename: str, dest_dir: str, revision: str = "main", retries: int = 3) -> str:
    dest = os.path.join(dest_dir, filename)
    if os.path.exists(dest):
        return dest
    if shutil.which("curl") is None:
        raise HubError("curl is not available to download " + filename)
    os.makedirs(os.path.dirname(dest) or ".", exist_ok=True)
    url = f"https://huggingface.co/{repo_id}/resolve/{revision}/{filename}"
    for _ in range(retries):
        r = subprocess.run(["curl", "-fL", "--retry", "2", "-o", dest + ".part", url], capture_output=True)
        if r.returncode == 0:
            os.replace(dest + ".part", dest)
            return dest
    raise HubError(f"failed to download {url}")


def resolve_pretrained_dir(source: str, revision: Optional[str] = None, allow_download: bool = True) -> str:
    """A local directory for ``source``: an existing path, else the HF cache, else a download."""
    if os.path.isdir(source):
        return source
    cached = find_cached_snapshot(source, revision)
    if cached is not None:
        return cached
    if not allow_download:
        raise HubError(f"{source} is neither a directory nor a cached Hugging Face repo")
    dest = os.path.join(repo_cache_dir(source), "snapshots", revision or "main")
    ensure_remote_file(source, "config.json", dest, revision or "main")
    try:
        ensure_remote_file(source, "model.safetensors.index.json", dest, revision or "main")
    except HubError:
        pass
    for f in shard_files(dest):
        ensure_remote_file(source, f, dest, revision or "main")
    for opt in ("tokenizer.json", "tokenizer_config.json", "generation_config.json"):
        try:
            ensure_remote_file(source, opt, dest, revision or "main", retries=1)
        except HubError:
            pass
    return dest


def load_model_from_pretrained(source: str, loader, **kw):
    """``loader(directory, **kw)`` on the resolved directory (Hub.lean:225)."""
    return loader(resolve_pretrained_dir(source), **kw)
