"""Byte-level BPE tokenizer (Tyr/Tokenizer/{Types,Encode,Decode,Training,IO,Pretokenize,
SpecialTokens,TokenBytes}.lean): training (`train_bpe`, Training.lean:211), encode/decode with
special tokens, the GPT-4 split pattern (IO.lean:23), the `TYR_BPE1` binary format (IO.lean:19-197:
magic, u32 version / vocab / merges / specials, u16-length-prefixed token bytes, u32 merge triples,
specials as u16 length + utf-8 + u32 id) and the bytes-per-token table used for bits-per-byte
evaluation (TokenBytes.lean:25-135).

The two hot loops - encoding pre-tokenised chunks against the merge table and the merge training itself - run in native code
(csrc/host/bpe.cpp) with exactly the semantics of the Python loops below, which remain as the fallback and the oracle of the
tests (``TYR_BPE_NATIVE=0`` selects them).
"""
from __future__ import annotations

import ctypes
import os
import struct
from collections import Counter
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

try:
    import regex as _re
except ImportError:  # pragma: no cover
    import re as _re

MAGIC = b"TYR_BPE1"
FORMAT_VERSION = 1

GPT4_SPLIT_PATTERN = (r"'(?i:[sdmt]|ll|ve|re)|[^\r\n\p{L}\p{N}]?+\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]++[\r\n]*|"
                      r"\s*[\r\n]|\s+(?!\S)|\s+")
DEFAULT_SPECIAL_TOKENS = ["<|bos|>", "<|user_start|>", "<|user_end|>", "<|assistant_start|>", "<|assistant_end|>",
                          "<|python_start|>", "<|python_end|>", "<|output_start|>", "<|output_end|>"]


_NATIVE = os.environ.get("TYR_BPE_NATIVE", "1") != "0"
_native_lib = None


def _host():
    """libtyr_host.so with the BPE entry points declared, or None when it cannot be loaded or predates them."""
    global _native_lib
    if _native_lib is None:
        try:
            from .._native import host
            lib = host()
            P, L, I = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
            lib.tyr_bpe_new.argtypes, lib.tyr_bpe_new.restype = [P, P, P, L, P], P
            lib.tyr_bpe_free.argtypes, lib.tyr_bpe_free.restype = [P], None
            lib.tyr_bpe_encode_chunks.argtypes, lib.tyr_bpe_encode_chunks.restype = [P, P, P, L, P, P, I], L
            lib.tyr_bpe_encode_concat.argtypes, lib.tyr_bpe_encode_concat.restype = [P, P, P, L, P, I], L
            lib.tyr_bpe_train.argtypes, lib.tyr_bpe_train.restype = [P, P, P, L, L, ctypes.c_int32, P, P], L
            _native_lib = lib
        except Exception:
            _native_lib = False
    return _native_lib or None


def _pack_chunks(chunks: Sequence[bytes]):
    """Concatenated bytes and the int64 offsets array (n + 1 entries) of a list of byte strings."""
    offsets = (ctypes.c_longlong * (len(chunks) + 1))()
    total = 0
    for i, c in enumerate(chunks):
        offsets[i] = total
        total += len(c)
    offsets[len(chunks)] = total
    return b"".join(chunks), offsets, total


def pretokenize(text: str, pattern: str = GPT4_SPLIT_PATTERN) -> List[str]:
    return _re.findall(pattern, text)


@dataclass
class MergeRule:
    left: int
    right: int
    result: int


class BPETokenizer:
    def __init__(self, id_to_bytes: List[bytes], merges: List[MergeRule], special_tokens: Optional[Dict[str, int]] = None,
                 pattern: str = GPT4_SPLIT_PATTERN):
        self.id_to_bytes = list(id_to_bytes)
        self.merges = list(merges)
        self.special_tokens = dict(special_tokens or {})
        self.id_to_special = {v: k for k, v in self.special_tokens.items()}
        self.pattern = pattern
        self.bytes_to_id = {b: i for i, b in enumerate(self.id_to_bytes) if b}
        self.merge_lookup = {(m.left, m.right): m.result for m in self.merges}
        self.merge_priority = {(m.left, m.right): i for i, m in enumerate(self.merges)}
        self._cache: Dict[str, List[int]] = {}
        self._handle = None                 # native merge table, built on first use

    def __del__(self):
        h, lib = getattr(self, "_handle", None), _native_lib
        if h and lib:
            lib.tyr_bpe_free(h)
            self._handle = None

    def _native_handle(self):
        if self._handle is None and _NATIVE:
            lib = _host()
            if lib is None:
                return None
            n = len(self.merges)
            arr = lambda vals: (ctypes.c_int32 * max(1, n))(*vals)
            b2i = (ctypes.c_int32 * 256)(*[self.bytes_to_id.get(bytes([b]), -1) for b in range(256)])
            self._handle = lib.tyr_bpe_new(arr(m.left for m in self.merges), arr(m.right for m in self.merges),
                                           arr(m.result for m in self.merges), n, b2i) or None
        return self._handle

    @property
    def vocab_size(self) -> int:
        return max(len(self.id_to_bytes), max(self.special_tokens.values(), default=-1) + 1)

    @staticmethod
    def byte_level() -> "BPETokenizer":
        return BPETokenizer([bytes([i]) for i in range(256)], [])

    # -- encoding ------------------------------------------------------------------------------------------
    def _encode_chunk(self, chunk: str) -> List[int]:
        hit = self._cache.get(chunk)
        if hit is not None:
            return hit
        ids = [self.bytes_to_id[bytes([b])] for b in chunk.encode("utf-8")]
        while len(ids) >= 2:
            best, best_rank = None, None
            for i in range(len(ids) - 1):
                r = self.merge_priority.get((ids[i], ids[i + 1]))
                if r is not None and (best_rank is None or r < best_rank):
                    best, best_rank = i, r
            if best is None:
                break
            pair = (ids[best], ids[best + 1])
            new, out, i = self.merge_lookup[pair], [], 0
            while i < len(ids):
                if i < len(ids) - 1 and (ids[i], ids[i + 1]) == pair:
                    out.append(new)
                    i += 2
                else:
                    out.append(ids[i])
                    i += 1
            ids = out
        if len(self._cache) < 200000:
            self._cache[chunk] = ids
        return ids

    def encode_ordinary(self, text: str) -> List[int]:
        chunks = pretokenize(text, self.pattern)
        if _NATIVE and self.merges and chunks:
            h = self._native_handle()
            if h is not None:            # every chunk through the native loop, ids back to back: no per-chunk Python work
                raw = [c.encode("utf-8") for c in chunks]
                data, offsets, total = _pack_chunks(raw)
                buf = (ctypes.c_int32 * max(1, total))()
                n = _native_lib.tyr_bpe_encode_concat(h, data, offsets, len(raw), buf, min(8, os.cpu_count() or 1))
                if n <= -2:
                    raise KeyError(f"chunk {chunks[-n - 2]!r} holds a byte without a token")
                if n >= 0:
                    return buf[:n]
        out = []
        for chunk in chunks:
            out.extend(self._encode_chunk(chunk))
        return out

    def encode(self, text: str, allowed_special: bool = True, prepend: Optional[str] = None,
               append: Optional[str] = None) -> List[int]:
        out: List[int] = []
        if prepend is not None:
            out.append(self.encode_special(prepend))
        if allowed_special and self.special_tokens:
            pat = "(" + "|".join(_re.escape(s) for s in sorted(self.special_tokens, key=len, reverse=True)) + ")"
            for part in _re.split(pat, text):
                if part in self.special_tokens:
                    out.append(self.special_tokens[part])
                elif part:
                    out.extend(self.encode_ordinary(part))
        else:
            out.extend(self.encode_ordinary(text))
        if append is not None:
            out.append(self.encode_special(append))
        return out

    def encode_special(self, token: str) -> int:
        if token not in self.special_tokens:
            raise KeyError(f"unknown special token {token!r}")
        return self.special_tokens[token]

    def get_bos_token_id(self) -> int:
        for name in ("<|bos|>", "<|endoftext|>"):
            if name in self.special_tokens:
                return self.special_tokens[name]
        raise KeyError("tokenizer has no BOS token")

    def encode_batch(self, texts: Sequence[str], **kw) -> List[List[int]]:
        return [self.encode(t, **kw) for t in texts]

    # -- decoding ------------------------------------------------------------------------------------------
    def decode_bytes(self, ids: Iterable[int]) -> bytes:
        out = bytearray()
        for i in ids:
            if i in self.id_to_special:
                out += self.id_to_special[i].encode("utf-8")
            elif 0 <= i < len(self.id_to_bytes):
                out += self.id_to_bytes[i]
            else:
                raise ValueError(f"token id {i} outside the vocabulary")
        return bytes(out)

    def decode(self, ids: Iterable[int]) -> str:
        return self.decode_bytes(ids).decode("utf-8", errors="replace")

    def token_bytes(self) -> List[int]:
        """Byte length of every token id (0 for special tokens): the bits-per-byte denominator."""
        n = self.vocab_size
        out = [0] * n
        for i, b in enumerate(self.id_to_bytes):
            out[i] = len(b)
        for i in self.id_to_special:
            if i < n:
                out[i] = 0
        return out

    # -- binary format -------------------------------------------------------------------------------------
    def serialize(self) -> bytes:
        entries = max(self.vocab_size if not self.special_tokens else len(self.id_to_bytes), len(self.id_to_bytes))
        out = bytearray(MAGIC)
        out += struct.pack("<IIII", FORMAT_VERSION, entries, len(self.merges), len(self.special_tokens))
        for i in range(entries):
            b = self.id_to_bytes[i] if i < len(self.id_to_bytes) else b""
            if len(b) > 65535:
                raise ValueError(f"token byte length {len(b)} exceeds UInt16 range for token id {i}")
            out += struct.pack("<H", len(b)) + b
        for m in self.merges:
            out += struct.pack("<III", m.left, m.right, m.result)
        for s, i in self.special_tokens.items():
            sb = s.encode("utf-8")
            out += struct.pack("<H", len(sb)) + sb + struct.pack("<I", i)
        return bytes(out)

    @staticmethod
    def deserialize(data: bytes) -> "BPETokenizer":
        if len(data) < 24 or data[:8] != MAGIC:
            raise ValueError("not a TYR_BPE1 tokenizer file")
        ver, vocab, nm, ns = struct.unpack_from("<IIII", data, 8)
        if ver != FORMAT_VERSION:
            raise ValueError(f"unsupported tokenizer format version {ver}")
        off = 24
        id_to_bytes = []
        for _ in range(vocab):
            if off + 2 > len(data):
                raise ValueError("truncated tokenizer file (vocabulary)")
            (ln,) = struct.unpack_from("<H", data, off)
            off += 2
            if off + ln > len(data):
                raise ValueError("truncated tokenizer file (token bytes)")
            id_to_bytes.append(data[off:off + ln])
            off += ln
        merges = []
        for _ in range(nm):
            if off + 12 > len(data):
                raise ValueError("truncated tokenizer file (merges)")
            l, r, res = struct.unpack_from("<III", data, off)
            merges.append(MergeRule(l, r, res))
            off += 12
        specials = {}
        for _ in range(ns):
            (ln,) = struct.unpack_from("<H", data, off)
            off += 2
            s = data[off:off + ln].decode("utf-8")
            off += ln
            (i,) = struct.unpack_from("<I", data, off)
            off += 4
            specials[s] = i
        return BPETokenizer(id_to_bytes, merges, specials)

    def save(self, path: str) -> None:
        with open(path, "wb") as f:
            f.write(self.serialize())

    @staticmethod
    def load(path: str) -> "BPETokenizer":
        with open(path, "rb") as f:
            return BPETokenizer.deserialize(f.read())


def train_bpe(texts: Iterable[str], vocab_size: int, special_tokens: Optional[Sequence[str]] = None,
              pattern: str = GPT4_SPLIT_PATTERN, doc_cap: Optional[int] = None, max_chars: Optional[int] = None) -> BPETokenizer:
    """Classic BPE over pre-tokenised chunks with incremental pair counts.  ``vocab_size`` includes
    the 256 byte tokens and the special tokens."""
    specials = list(special_tokens if special_tokens is not None else [])
    n_merges = vocab_size - 256 - len(specials)
    if n_merges < 0:
        raise ValueError("vocab_size must be at least 256 + number of special tokens")
    words: Counter = Counter()
    seen = 0
    for t in texts:
        if doc_cap is not None:
            t = t[:doc_cap]
        if max_chars is not None:
            if seen >= max_chars:
                break
            t = t[:max_chars - seen]
        seen += len(t)
        words.update(pretokenize(t, pattern))
    lib = _host() if _NATIVE else None
    if lib is not None and n_merges > 0 and words:
        raw = [w.encode("utf-8") for w in words]
        data, offsets, _ = _pack_chunks(raw)
        fr = (ctypes.c_longlong * len(raw))(*[words[w] for w in words])
        left, right = (ctypes.c_int32 * n_merges)(), (ctypes.c_int32 * n_merges)()
        made = lib.tyr_bpe_train(data, offsets, fr, len(raw), n_merges, 256, left, right)
        if made >= 0:
            id_to_bytes = [bytes([i]) for i in range(256)]
            merges = []
            for j in range(made):
                id_to_bytes.append(id_to_bytes[left[j]] + id_to_bytes[right[j]])
                merges.append(MergeRule(left[j], right[j], 256 + j))
            special_map = {s: len(id_to_bytes) + i for i, s in enumerate(specials)}
            return BPETokenizer(id_to_bytes, merges, special_map, pattern)
    seqs = [list(w.encode("utf-8")) for w in words]
    freqs = [words[w] for w in words]
    pair_counts: Counter = Counter()
    where: Dict[Tuple[int, int], set] = {}
    for wi, s in enumerate(seqs):
        for a, b in zip(s, s[1:]):
            pair_counts[(a, b)] += freqs[wi]
            where.setdefault((a, b), set()).add(wi)
    id_to_bytes = [bytes([i]) for i in range(256)]
    merges: List[MergeRule] = []
    for _ in range(n_merges):
        if not pair_counts:
            break
        best = max(pair_counts.items(), key=lambda kv: (kv[1], -kv[0][0], -kv[0][1]))
        (a, b), c = best
        if c <= 0:
            break
        new_id = len(id_to_bytes)
        id_to_bytes.append(id_to_bytes[a] + id_to_bytes[b])
        merges.append(MergeRule(a, b, new_id))
        for wi in list(where.get((a, b), ())):
            s, f = seqs[wi], freqs[wi]
            for x, y in zip(s, s[1:]):
                pair_counts[(x, y)] -= f
                if pair_counts[(x, y)] <= 0:
                    del pair_counts[(x, y)]
            out, i = [], 0
            while i < len(s):
                if i < len(s) - 1 and s[i] == a and s[i + 1] == b:
                    out.append(new_id)
                    i += 2
                else:
                    out.append(s[i])
                    i += 1
            seqs[wi] = out
            for x, y in zip(out, out[1:]):
                pair_counts[(x, y)] += f
                where.setdefault((x, y), set()).add(wi)
        where.pop((a, b), None)
    special_map = {s: len(id_to_bytes) + i for i, s in enumerate(specials)}
    return BPETokenizer(id_to_bytes, merges, special_map, pattern)
