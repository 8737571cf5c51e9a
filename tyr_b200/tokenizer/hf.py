"""Hugging Face ``tokenizer.json`` loaders and chat templates (Tyr/Tokenizer/{Qwen3,Qwen35,Qwen36,
Gemma4,Laguna}.lean): byte-level BPE with the GPT-2 byte<->unicode table, ranked merges, added
(special) tokens, and the ChatML-style templates of the Qwen / Laguna families plus Gemma's turn
format."""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

try:
    import regex as _re
except ImportError:  # pragma: no cover
    import re as _re


def bytes_to_unicode() -> Dict[int, str]:
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("\xa1"), ord("\xac") + 1)) + list(range(ord("\xae"), ord("\xff") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return dict(zip(bs, map(chr, cs)))


QWEN_PATTERN = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|"
                r"\s*[\r\n]+|\s+(?!\S)|\s+")


class HFTokenizer:
    def __init__(self, vocab: Dict[str, int], merges: Sequence[Tuple[str, str]], added: Dict[str, int],
                 pattern: str = QWEN_PATTERN, byte_level: bool = True):
        self.vocab = dict(vocab)
        self.ranks = {tuple(m): i for i, m in enumerate(merges)}
        self.added = dict(added)
        self.id_to_token = {i: t for t, i in self.vocab.items()}
        self.id_to_token.update({i: t for t, i in self.added.items()})
        self.pattern = pattern
        self.byte_level = byte_level
        self.b2u = bytes_to_unicode()
        self.u2b = {v: k for k, v in self.b2u.items()}
        self._cache: Dict[str, List[int]] = {}

    @staticmethod
    def from_file(path: str) -> "HFTokenizer":
        if os.path.isdir(path):
            path = os.path.join(path, "tokenizer.json")
        j = json.load(open(path, encoding="utf-8"))
        model = j.get("model", {})
        if model.get("type", "BPE") != "BPE":
            raise ValueError(f"unsupported tokenizer model {model.get('type')}")
        merges = [tuple(m.split(" ", 1)) if isinstance(m, str) else tuple(m) for m in model.get("merges", [])]
        added = {a["content"]: a["id"] for a in j.get("added_tokens", [])}
        pattern = QWEN_PATTERN
        pre = j.get("pre_tokenizer") or {}
        for p in ([pre] + list(pre.get("pretokenizers", []))):
            pat = (p.get("pattern") or {}).get("Regex") if isinstance(p, dict) else None
            if pat:
                pattern = pat
        return HFTokenizer(model.get("vocab", {}), merges, added, pattern)

    @property
    def vocab_size(self) -> int:
        return max(list(self.vocab.values()) + list(self.added.values()) + [-1]) + 1

    def _bpe(self, word: str) -> List[int]:
        hit = self._cache.get(word)
        if hit is not None:
            return hit
        parts = list(word)
        while len(parts) > 1:
            best, rank = None, None
            for i in range(len(parts) - 1):
                r = self.ranks.get((parts[i], parts[i + 1]))
                if r is not None and (rank is None or r < rank):
                    best, rank = i, r
            if best is None:
                break
            parts = parts[:best] + [parts[best] + parts[best + 1]] + parts[best + 2:]
        ids = []
        for p in parts:
            if p in self.vocab:
                ids.append(self.vocab[p])
            else:  # unknown piece: fall back to its characters
                ids.extend(self.vocab[c] for c in p if c in self.vocab)
        self._cache[word] = ids
        return ids

    def encode_ordinary(self, text: str) -> List[int]:
        out: List[int] = []
        for chunk in _re.findall(self.pattern, text):
            mapped = "".join(self.b2u[b] for b in chunk.encode("utf-8")) if self.byte_level else chunk
            out.extend(self._bpe(mapped))
        return out

    def encode(self, text: str, allowed_special: bool = True) -> List[int]:
        if not (allowed_special and self.added):
            return self.encode_ordinary(text)
        pat = "(" + "|".join(_re.escape(s) for s in sorted(self.added, key=len, reverse=True)) + ")"
        out: List[int] = []
        for part in _re.split(pat, text):
            if part in self.added:
                out.append(self.added[part])
            elif part:
                out.extend(self.encode_ordinary(part))
        return out

    def decode(self, ids: Iterable[int], skip_special: bool = False) -> str:
        buf = bytearray()
        for i in ids:
            tok = self.id_to_token.get(int(i))
            if tok is None:
                continue
            if tok in self.added:
                if not skip_special:
                    buf += tok.encode("utf-8")
                continue
            if self.byte_level:
                buf += bytes(self.u2b.get(c, ord("?")) for c in tok)
            else:
                buf += tok.encode("utf-8")
        return buf.decode("utf-8", errors="replace")

    def token_id(self, token: str) -> Optional[int]:
        return self.added.get(token, self.vocab.get(token))


def chatml_prompt(messages: Sequence[Dict[str, str]], add_generation_prompt: bool = True,
                  system: Optional[str] = None, enable_thinking: Optional[bool] = None) -> str:
    """Qwen3 / Qwen3.5 / Laguna chat template: <|im_start|>role\\ncontent<|im_end|>\\n ..."""
    out = []
    if system is not None and not (messages and messages[0]["role"] == "system"):
        out.append(f"<|im_start|>system\n{system}<|im_end|>\n")
    for m in messages:
        out.append(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n")
    if add_generation_prompt:
        out.append("<|im_start|>assistant\n")
        if enable_thinking is False:
            out.append("<think>\n\n</think>\n\n")
    return "".join(out)


def gemma_prompt(messages: Sequence[Dict[str, str]], add_generation_prompt: bool = True) -> str:
    """Gemma turn format: <start_of_turn>role\\ncontent<end_of_turn>\\n (assistant is 'model')."""
    out = ["<bos>"]
    for m in messages:
        role = "model" if m["role"] == "assistant" else m["role"]
        out.append(f"<start_of_turn>{role}\n{m['content']}<end_of_turn>\n")
    if add_generation_prompt:
        out.append("<start_of_turn>model\n")
    return "".join(out)


def load_qwen3(path: str) -> HFTokenizer:
    return HFTokenizer.from_file(path)


load_qwen35 = load_qwen36 = load_laguna = load_qwen3


def load_gemma4(path: str) -> HFTokenizer:
    t = HFTokenizer.from_file(path)
    t.byte_level = False
    return t


# ---- Laguna (Tyr/Tokenizer/Laguna.lean:29-50, 751-757) ---------------------------------------------------
LAGUNA_EOS_ID, LAGUNA_PAD_ID, LAGUNA_CLS_ID, LAGUNA_ASSISTANT_END_ID = 2, 9, 10, 24
LAGUNA_EOS_TOKEN, LAGUNA_PAD_TOKEN = "〈|EOS|〉", "〈|PAD|〉"
LAGUNA_SYSTEM = ("You are a helpful, conversationally-fluent assistant made by Poolside. "
                 "You are here to be helpful to users through natural language conversations.")


def laguna_prompt(prompt: str, enable_thinking: bool = True, system: str = LAGUNA_SYSTEM) -> str:
    """Single user turn; ends with ``<assistant><think>`` (thinking on) or ``<assistant></think>``."""
    return (f"{LAGUNA_EOS_TOKEN}<system>{system}</system>\n<user>{prompt}</user>\n<assistant>"
            + ("<think>" if enable_thinking else "</think>"))


def laguna_encode(tok: HFTokenizer, text: str) -> List[int]:
    """HF post-processor behaviour: the EOS token (id 2, doubling as BOS) is always prepended."""
    bos = tok.token_id(LAGUNA_EOS_TOKEN)
    return [LAGUNA_EOS_ID if bos is None else bos] + tok.encode(text)
