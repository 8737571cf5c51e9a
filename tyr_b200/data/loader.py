"""Token-stream data loading (Tyr/DataLoader.lean).

uint16 ``.bin`` shards (optional 256-int32 header with magic 20240520), ``BOSFinder`` document
windows (documents are packed across batch boundaries, never padded; optional seeded document
shuffle), ``DataShard.load(path, rank, world)`` slicing one file across ranks, ``BatchIterator`` and
``DistributedDataGenerator`` with a resumable ``StreamCursor`` (seed, epoch, file index, position)
that refuses to restore into a different stream (world size, files, BOS policy...).
File reads go through the native loader (csrc/host/io.cpp).
"""
from __future__ import annotations

import bisect
import ctypes
import json
import os
from dataclasses import dataclass, asdict, field, replace
from typing import List, Optional, Tuple

import torch

from .._native import host, register_host_signatures

_MASK = (1 << 64) - 1


@register_host_signatures
def _sigs(lib):
    L, P = ctypes.c_longlong, ctypes.c_void_p
    lib.tyr_bin_token_count.argtypes = [ctypes.c_char_p, ctypes.POINTER(L), ctypes.POINTER(L)]
    lib.tyr_load_u16_bin.argtypes = [ctypes.c_char_p, L, L, P]
    lib.tyr_find_bos.argtypes = [P, L, L, P, L]
    lib.tyr_find_bos.restype = L


def lcg_next(state: int) -> int:
    return (state * 6364136223846793005 + 1442695040888963407) & _MASK


def fisher_yates(arr: List[int], seed: int) -> List[int]:
    if len(arr) <= 1:
        return list(arr)
    res, state, n = list(arr), seed & _MASK, len(arr)
    for i in range(n - 1):
        state = lcg_next(state)
        j = i + state % (n - i)
        res[i], res[j] = res[j], res[i]
    return res


def bin_file_token_count(path: str) -> int:
    lib = host()
    c, h = ctypes.c_longlong(), ctypes.c_longlong()
    if lib.tyr_bin_token_count(path.encode(), ctypes.byref(c), ctypes.byref(h)) != 0:
        raise IOError(lib.tyr_host_last_error().decode())
    return int(c.value)


def load_u16_bin(path: str, start: int = 0, count: Optional[int] = None) -> torch.Tensor:
    """Int64 tensor of tokens [start, start+count) of a shard (payload only, header skipped)."""
    total = bin_file_token_count(path)
    if count is None:
        count = total - start
    out = torch.empty(count, dtype=torch.int64)
    lib = host()
    if lib.tyr_load_u16_bin(path.encode(), start, count, ctypes.c_void_p(out.data_ptr())) != 0:
        raise IOError(lib.tyr_host_last_error().decode())
    return out


def write_u16_bin(path: str, tokens: torch.Tensor, with_header: bool = True) -> None:
    import numpy as np
    t = tokens.to(torch.int64).numpy().astype("uint16")
    with open(path, "wb") as f:
        if with_header:
            head = np.zeros(256, dtype="int32")
            head[0], head[1], head[2] = 20240520, 1, t.size
            f.write(head.tobytes())
        f.write(t.tobytes())


def find_bos_positions(tokens: torch.Tensor, bos: int) -> List[int]:
    t = tokens.contiguous()
    n = t.numel()
    lib = host()
    k = lib.tyr_find_bos(ctypes.c_void_p(t.data_ptr()), n, bos, None, 0)
    out = torch.empty(k, dtype=torch.int64)
    lib.tyr_find_bos(ctypes.c_void_p(t.data_ptr()), n, bos, ctypes.c_void_p(out.data_ptr()), k)
    return out.tolist()


def resolve_shard_paths(spec: str) -> List[str]:
    """A directory (all .bin inside), a file, or a file-name prefix."""
    if os.path.isdir(spec):
        files = sorted(os.path.join(spec, f) for f in os.listdir(spec) if f.endswith(".bin"))
        if not files:
            raise IOError(f"No .bin files found under directory: {spec}")
        return files
    if os.path.isfile(spec):
        return [spec]
    parent, stem = os.path.dirname(spec) or ".", os.path.basename(spec)
    if os.path.isdir(parent):
        files = sorted(os.path.join(parent, f) for f in os.listdir(parent) if f.startswith(stem) and f.endswith(".bin"))
        if files:
            return files
    raise IOError(f"Could not resolve shard path: {spec}")


class BOSFinder:
    def __init__(self, tokens: torch.Tensor, bos_token: int):
        self.tokens = tokens
        self.n = tokens.numel()
        self.bos_token = bos_token
        pos = find_bos_positions(tokens, bos_token)
        if self.n > 0 and (not pos or pos[0] != 0):
            pos = [0] + pos
        self.bos_positions = pos
        self.current_pos = 0
        self.ordered_docs: List[Tuple[int, int]] = []
        self.ordered_ends: List[int] = []

    def find_next_valid_start(self, after: int) -> Optional[int]:
        i = bisect.bisect_left(self.bos_positions, after)
        return self.bos_positions[i] if i < len(self.bos_positions) else None

    def reset(self) -> "BOSFinder":
        self.current_pos = 0
        self.ordered_docs, self.ordered_ends = [], []
        return self

    def shuffle(self, seed: int) -> "BOSFinder":
        order = fisher_yates(list(range(len(self.bos_positions))), seed)
        docs, ends, total = [], [], 0
        for idx in order:
            start = self.bos_positions[idx]
            stop = self.bos_positions[idx + 1] if idx + 1 < len(self.bos_positions) else self.n
            docs.append((start, stop - start))
            total += stop - start
            ends.append(total)
        self.ordered_docs, self.ordered_ends, self.current_pos = docs, ends, 0
        return self

    def take(self, count: int) -> torch.Tensor:
        count = min(count, self.n - self.current_pos)
        if count == 0:
            return self.tokens[:0]
        end = self.current_pos + count
        if not self.ordered_docs:
            out = self.tokens[self.current_pos:end]
            self.current_pos = end
            return out
        doc = bisect.bisect_right(self.ordered_ends, self.current_pos)
        pos, chunks = self.current_pos, []
        while pos < end and doc < len(self.ordered_docs):
            start, dlen = self.ordered_docs[doc]
            doc_start = 0 if doc == 0 else self.ordered_ends[doc - 1]
            off = min(pos - doc_start, dlen)
            ln = min(end - pos, dlen - off)
            chunks.append(self.tokens[start + off:start + off + ln])
            pos += ln
            doc += 1
        self.current_pos = end
        return torch.cat(chunks) if chunks else self.tokens[:0]

    def get_batch(self, batch_size: int, seq_len: int) -> Optional[torch.Tensor]:
        need = batch_size * seq_len
        if need <= self.n - self.current_pos:
            return self.take(need).reshape(batch_size, seq_len)
        return None


@dataclass
class DataShard:
    tokens: torch.Tensor
    bos_finder: BOSFinder
    shard_idx: int
    num_shards: int

    @staticmethod
    def load(path: str, shard_idx: int, num_shards: int, bos_token: int) -> "DataShard":
        if not 0 <= shard_idx < num_shards:
            raise ValueError("Invalid data-loader rank/world size")
        if not os.path.exists(path):
            raise IOError(f"Data shard not found: {path}")
        total = bin_file_token_count(path)
        per = total // num_shards
        start = per * shard_idx
        end = total if shard_idx == num_shards - 1 else start + per
        toks = load_u16_bin(path, start, end - start)
        return DataShard(toks, BOSFinder(toks, bos_token), shard_idx, num_shards)

    @property
    def num_tokens(self) -> int:
        return self.tokens.numel()


class BatchIterator:
    def __init__(self, shard: DataShard, shuffle_seed: Optional[int] = None, epoch: int = 0):
        self.shard, self.shuffle_seed, self.epoch, self.batch_count = shard, shuffle_seed, epoch, 0
        if shuffle_seed is None:
            shard.bos_finder.reset()
        else:
            shard.bos_finder.shuffle(lcg_next((shuffle_seed + epoch) & _MASK))

    @property
    def num_tokens(self) -> int:
        return self.shard.num_tokens

    def next(self, batch_size: int, seq_len: int) -> Optional[torch.Tensor]:
        """``None`` marks the end of an epoch (the iterator has been re-armed for the next one)."""
        b = self.shard.bos_finder.get_batch(batch_size, seq_len)
        if b is None:
            self.__init__(self.shard, self.shuffle_seed, self.epoch + 1)
            return None
        self.batch_count += 1
        return b


@dataclass
class LoaderConfig:
    data_path: str
    bos_token: int = 50256
    seed: int = 42
    shuffle: bool = True
    batch_size: int = 32
    seq_len: int = 2048


@dataclass
class StreamCursor:
    seed: int
    shuffle: bool
    bos_token: int
    rank: int
    world_size: int
    train_paths: List[str]
    train_path_idx: int
    shard_length: int
    position: int
    epoch: int
    global_step: int
    batch_count: int
    version: int = 1

    def to_json(self) -> str:
        return json.dumps(asdict(self))

    @staticmethod
    def from_json(s: str) -> "StreamCursor":
        return StreamCursor(**json.loads(s))


def _stream_seed(cfg: LoaderConfig, rank: int, path_idx: int) -> Optional[int]:
    return ((lcg_next((cfg.seed + rank) & _MASK) + path_idx) & _MASK) if cfg.shuffle else None


class DistributedDataGenerator:
    def __init__(self, config: LoaderConfig, rank: int, world_size: int):
        self.config, self.rank, self.world_size = config, rank, world_size
        self.train_paths = resolve_shard_paths(config.data_path)
        self.train_path_idx = 0
        self.global_step = 0
        self.iterator = self._open(0, 0)

    @staticmethod
    def init(config: LoaderConfig) -> "DistributedDataGenerator":
        from .. import distributed as dist
        if dist.is_initialized():
            return DistributedDataGenerator(config, dist.get_rank(), dist.get_world_size())
        return DistributedDataGenerator(config, 0, 1)

    def _open(self, path_idx: int, epoch: int) -> BatchIterator:
        shard = DataShard.load(self.train_paths[path_idx], self.rank, self.world_size, self.config.bos_token)
        return BatchIterator(shard, _stream_seed(self.config, self.rank, path_idx), epoch)

    def cursor(self) -> StreamCursor:
        it = self.iterator
        return StreamCursor(self.config.seed, self.config.shuffle, self.config.bos_token, self.rank, self.world_size,
                            list(self.train_paths), self.train_path_idx, it.num_tokens,
                            it.shard.bos_finder.current_pos, it.epoch, self.global_step, it.batch_count)

    def restore_cursor(self, c: StreamCursor) -> "DistributedDataGenerator":
        if (c.version != 1 or c.seed != self.config.seed or c.shuffle != self.config.shuffle
                or c.bos_token != self.config.bos_token or c.rank != self.rank or c.world_size != self.world_size
                or list(c.train_paths) != list(self.train_paths)):
            raise ValueError("Data cursor stream mismatch (version, seed, rank, world size, BOS policy or files)")
        if c.train_path_idx >= len(self.train_paths):
            raise ValueError("Data cursor shard index out of bounds")
        it = self._open(c.train_path_idx, c.epoch)
        if it.num_tokens != c.shard_length or c.position > it.num_tokens:
            raise ValueError("Data cursor shard length or position mismatch")
        it.shard.bos_finder.current_pos = c.position
        it.batch_count = c.batch_count
        self.iterator, self.train_path_idx, self.global_step = it, c.train_path_idx, c.global_step
        return self

    def next_tokens(self, count: int) -> torch.Tensor:
        """Exactly ``count`` tokens of the continuous stream; file tails carry over, crossing the
        last file starts a new seeded epoch."""
        if count == 0:
            raise ValueError("Batch token count must be positive")
        remaining, chunks, empty = count, [], 0
        while remaining > 0:
            it = self.iterator
            avail = it.num_tokens - it.shard.bos_finder.current_pos
            ln = min(remaining, avail)
            if ln > 0:
                chunks.append(it.shard.bos_finder.take(ln))
                remaining -= ln
                empty = 0
            if remaining == 0:
                break
            if avail == 0:
                empty += 1
            if empty > len(self.train_paths):
                raise IOError("Training corpus has no tokens for this rank")
            nxt = (self.train_path_idx + 1) % len(self.train_paths)
            epoch = self.iterator.epoch + (1 if nxt == 0 else 0)
            self.iterator = self._open(nxt, epoch)
            self.train_path_idx = nxt
        self.global_step += 1
        self.iterator.batch_count += 1
        return torch.cat(chunks)

    def next_batch(self, batch_size: Optional[int] = None, seq_len: Optional[int] = None):
        """(inputs, targets) of shape [B, T] taken from B*T+1 stream tokens."""
        B = batch_size or self.config.batch_size
        T = seq_len or self.config.seq_len
        toks = self.next_tokens(B * T + 1)
        return toks[:-1].reshape(B, T), toks[1:].reshape(B, T)


def synthetic_zipf_tokens(count: int, vocab: int, exponent: float = 1.1, seed: int = 0) -> torch.Tensor:
    """Zipf-distributed token ids (benchmark data when no corpus is available)."""
    import numpy as np
    rng = np.random.default_rng(seed)
    return torch.from_numpy(((rng.zipf(exponent, size=count) - 1) % vocab).astype("int64"))
