"""Downloads with retry and the dataset cache layout (Tyr/Data/Download.lean).  Network access is optional: every
``ensure_*`` first looks for the file on disk and only then tries to fetch it."""
from __future__ import annotations

import os
import shutil
import time
import urllib.request
import zipfile
from dataclasses import dataclass
from typing import Callable, Optional

from ..utils.log import Handlers


@dataclass
class DownloadConfig:
    max_retries: int = 5
    initial_delay_ms: int = 1000
    timeout_s: float = 60.0


def expand_home(path: str) -> str:
    return os.path.expanduser(path)


def ensure_dir(path: str) -> None:
    os.makedirs(path, exist_ok=True)


def file_exists(path: str) -> bool:
    return os.path.isfile(path)


def download_with_retry(url: str, dest: str, max_retries: int = 5, initial_delay_ms: int = 1000, log: Optional[Handlers] = None,
                        fetch: Optional[Callable[[str, str], None]] = None, sleep=time.sleep) -> bool:
    """Fetch ``url`` to ``dest`` (atomic rename of a ``.tmp`` file), exponential back-off between attempts."""
    log = log or Handlers()
    if file_exists(dest):
        return True
    ensure_dir(os.path.dirname(dest) or ".")

    def default_fetch(u, d):
        with urllib.request.urlopen(u, timeout=60) as r, open(d, "wb") as f:
            shutil.copyfileobj(r, f)
    fetch = fetch or default_fetch
    delay = initial_delay_ms
    for attempt in range(max_retries):
        tmp = dest + ".tmp"
        try:
            fetch(url, tmp)
            os.replace(tmp, dest)
            return True
        except Exception as e:                       # network errors are expected here; report and retry
            if os.path.exists(tmp):
                os.remove(tmp)
            log.on_warn(f"download attempt {attempt + 1}/{max_retries} failed for {url}: {e}")
            if attempt + 1 < max_retries:
                sleep(delay / 1000.0)
                delay *= 2
    return False


def download_and_extract_zip(url: str, dest_dir: str, max_retries: int = 5, log: Optional[Handlers] = None, fetch=None) -> bool:
    ensure_dir(dest_dir)
    z = os.path.join(dest_dir, "download.zip")
    if not download_with_retry(url, z, max_retries, log=log, fetch=fetch):
        return False
    with zipfile.ZipFile(z) as zf:
        zf.extractall(dest_dir)
    os.remove(z)
    return True


CORE_BUNDLE_URL = "https://karpathy-public.s3.us-west-2.amazonaws.com/eval_bundle.zip"
WORD_LIST_URL = "https://raw.githubusercontent.com/dwyl/english-words/master/words_alpha.txt"


def ensure_core_data(cache_dir: str = "~/.cache/nanochat", log: Optional[Handlers] = None, fetch=None) -> str:
    d = os.path.join(expand_home(cache_dir), "eval_bundle")
    if not os.path.isdir(d):
        if not download_and_extract_zip(CORE_BUNDLE_URL, expand_home(cache_dir), log=log, fetch=fetch):
            raise IOError("failed to fetch the CORE evaluation bundle")
    return d


def ensure_word_list(cache_dir: str = "~/.cache/nanochat", log: Optional[Handlers] = None, fetch=None) -> str:
    p = os.path.join(expand_home(cache_dir), "words_alpha.txt")
    if not download_with_retry(WORD_LIST_URL, p, log=log, fetch=fetch):
        raise IOError("failed to fetch the word list")
    return p


def ensure_hf_parquet(repo_id: str, subset: str, split: str, cache_dir: str = "~/.cache/huggingface", shard: int = 0,
                      log: Optional[Handlers] = None, fetch=None) -> str:
    out_dir = os.path.join(expand_home(cache_dir), "datasets", repo_id.replace("/", "_"), subset)
    dest = os.path.join(out_dir, f"{split}-{shard:05d}.parquet")
    url = f"https://huggingface.co/datasets/{repo_id}/resolve/refs%2Fconvert%2Fparquet/{subset}/{split}/{shard:04d}.parquet"
    if not download_with_retry(url, dest, log=log, fetch=fetch):
        raise IOError(f"failed to fetch {repo_id}/{subset}/{split}")
    return dest
