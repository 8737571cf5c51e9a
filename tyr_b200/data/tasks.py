"""Built-in synthetic tasks and the LLM evaluation tasks (Tyr/Data/Tasks.lean, Examples/NanoChat/Tasks/LLM.lean,
Tyr/Data/HuggingFace.lean): identity, arithmetic with a calculator call, spelling, multiple choice; ARC, MMLU, GSM8K,
SmolTalk and custom JSONL loaders over parquet / jsonl rows."""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

from . import download as dl
from . import parquet as pq
from .task import ASSISTANT, TOOL, USER, ContentPart, Conversation, LoadedTask, Message, MixtureEntry, TaskMixture, lcg_next
from .task_class import CATEGORICAL, GENERATIVE, EvalResult, EvalTask

# ---- synthetic tasks -------------------------------------------------------------------------------------------


def create_identity_task(model_name: str, num_examples: int = 100) -> LoadedTask:
    t = [("What is your name?", f"My name is {model_name}."), ("Who are you?", f"I am {model_name}, an AI assistant."),
         ("Tell me about yourself.", f"I'm {model_name}, a helpful AI assistant trained to be informative and safe."),
         ("What can you do?", "I can help with questions, writing, analysis, coding, math, and general conversation."),
         ("Are you an AI?", f"Yes, I am {model_name}, an artificial intelligence assistant."),
         ("Who created you?", "I was created by a team of researchers and engineers."),
         ("What's your purpose?", "My purpose is to be helpful, harmless, and honest in my interactions.")]
    return LoadedTask("identity", [Conversation([Message.user(t[i % len(t)][0]), Message.assistant(t[i % len(t)][1])])
                                   for i in range(num_examples)])


def create_math_conversation(question: str, answer: str, use_calculator: bool = False) -> Conversation:
    msgs = [Message.user(question)]
    if use_calculator:
        msgs.append(Message(ASSISTANT, "Let me work through this step by step.", [ContentPart("tool_call:calculator", "2+2")]))
        msgs.append(Message(TOOL, "4"))
    msgs.append(Message.assistant(answer))
    return Conversation(msgs)


SAMPLE_MATH = [("What is 2 + 2?", "2 + 2 = 4", False), ("What is 15 * 7?", "15 * 7 = 105", True),
               ("If I have 3 apples and buy 5 more, how many do I have?", "3 + 5 = 8 apples", False),
               ("What is 144 / 12?", "144 / 12 = 12", True), ("What is 2^10?", "2^10 = 1024", True)]


def create_math_task() -> LoadedTask:
    return LoadedTask("math", [create_math_conversation(*p) for p in SAMPLE_MATH])


def create_spelling_conversation(word: str) -> Conversation:
    return Conversation([Message.user(f"Spell the word '{word}'."), Message.assistant(f"{word}: " + "-".join(word.upper()))])


def create_letter_count_conversation(word: str, letter: str) -> Conversation:
    n = word.count(letter)
    return Conversation([Message.user(f"How many times does the letter '{letter}' appear in '{word}'?"),
                         Message.assistant(f"The letter '{letter}' appears {n} time{'s' if n != 1 else ''} in '{word}'.")])


SAMPLE_WORDS = ["strawberry", "banana", "mississippi", "programming", "algorithm", "necessary", "rhythm", "parallel"]


def create_spelling_task() -> LoadedTask:
    convs = []
    for w in SAMPLE_WORDS:
        convs.append(create_spelling_conversation(w))
        convs.append(create_letter_count_conversation(w, w[0]))
    return LoadedTask("spelling", convs)


def create_multiple_choice_conversation(question: str, choices: Sequence[str], correct_idx: int, explanation: str = "") -> Conversation:
    labels = "ABCD"
    full = question + "\n\n" + "\n".join(f"{labels[i]}. {c}" for i, c in enumerate(choices))
    ans = f"The answer is {labels[correct_idx]}. {choices[correct_idx]}" + (f"\n\n{explanation}" if explanation else "")
    return Conversation([Message.user(full), Message.assistant(ans)])


SAMPLE_MC = [("What is the capital of France?", ["London", "Paris", "Berlin", "Madrid"], 1, ""),
             ("Which planet is known as the Red Planet?", ["Venus", "Jupiter", "Mars", "Saturn"], 2, "Iron oxide gives Mars its colour."),
             ("What is the chemical symbol for water?", ["CO2", "H2O", "O2", "NaCl"], 1, "")]


def create_mc_task() -> LoadedTask:
    return LoadedTask("multiple_choice", [create_multiple_choice_conversation(*q) for q in SAMPLE_MC])


def create_midtraining_mixture(model_name: str) -> TaskMixture:
    return TaskMixture.create([MixtureEntry(create_identity_task(model_name, 50), 2), MixtureEntry(create_math_task(), 1),
                               MixtureEntry(create_spelling_task(), 1), MixtureEntry(create_mc_task(), 1)])


def create_sft_mixture(model_name: str) -> TaskMixture:
    return TaskMixture.create([MixtureEntry(create_identity_task(model_name, 20), 1), MixtureEntry(create_math_task(), 2),
                               MixtureEntry(create_mc_task(), 2)])


# ---- answer extraction / rendering ---------------------------------------------------------------------------------
def extract_hash_answer(response: str) -> Optional[str]:
    i = response.find("#### ")
    if i < 0:
        return None
    rest = response[i + 5:]
    for stop in ("\n", "\r"):
        j = rest.find(stop)
        if j >= 0:
            rest = rest[:j]
    rest = rest.strip().replace(",", "")
    return rest or None


def extract_letter_answer(response: str, valid=("A", "B", "C", "D")) -> Optional[str]:
    t = response.strip()
    if t in valid:
        return t
    for l in valid:
        if t.startswith(l):
            return l
    return None


def render_multiple_choice(question: str, letters: Sequence[str], choices: Sequence[str]) -> str:
    out = f"Multiple Choice question: {question}\n"
    for l, c in zip(letters, choices):
        out += f"- {c}={l}\n"
    return out + "\nRespond only with the letter of the correct answer."


def parse_gsm8k_answer(answer: str) -> List[ContentPart]:
    """Split on ``<<expr=result>>`` calculator annotations into text, tool-call and tool-result parts."""
    parts, rem = [], answer
    while True:
        i = rem.find("<<")
        if i < 0:
            if rem:
                parts.append(ContentPart("text", rem))
            return parts
        if rem[:i]:
            parts.append(ContentPart("text", rem[:i]))
        after = rem[i + 2:]
        j = after.find(">>")
        if j < 0:
            parts.append(ContentPart("text", rem[i:]))
            return parts
        inner = after[:j].split("=")
        expr, res = (inner[0], inner[1]) if len(inner) == 2 else (inner[0], "") if len(inner) == 1 else (after[:j], "")
        parts += [ContentPart("tool_call:calculator", expr), ContentPart("tool_result", res)]
        rem = after[j + 2:]


@dataclass
class SliceConfig:
    start: int = 0
    stop: Optional[int] = None
    step: int = 1

    def size(self, n: int) -> int:
        stop = n if self.stop is None else min(self.stop, n)
        return max(0, (stop - self.start + self.step - 1) // self.step)

    def physical(self, index: int) -> int:
        return self.start + index * self.step


class _RowTask(EvalTask):
    def __init__(self, rows: List[dict], config: Optional[SliceConfig] = None):
        self.rows, self.config = rows, config or SliceConfig()

    def size(self) -> int:
        return self.config.size(len(self.rows))

    def _row(self, idx: int) -> Optional[dict]:
        p = self.config.physical(idx)
        return self.rows[p] if 0 <= idx < self.size() and p < len(self.rows) else None


class _MCTask(_RowTask):
    def eval_type(self) -> str:
        return CATEGORICAL

    def evaluate(self, conv: Conversation, response: str) -> EvalResult:
        expected = conv.messages[-1].content if conv.messages else ""
        predicted = extract_letter_answer(response) or ""
        ok = bool(expected) and predicted == expected
        return EvalResult(ok, 1.0 if ok else 0.0, expected, predicted)


class ARCTask(_MCTask):
    name = "ARC"

    def get_example(self, idx):
        r = self._row(idx)
        if r is None:
            return None
        labels, texts = r["choices"]["label"], r["choices"]["text"]
        return Conversation([Message.user(render_multiple_choice(r["question"], labels, texts)), Message.assistant(r["answerKey"])])


class MMLUTask(_MCTask):
    name = "MMLU"
    letters = ("A", "B", "C", "D")

    def get_example(self, idx):
        r = self._row(idx)
        if r is None:
            return None
        return Conversation([Message.user(render_multiple_choice(r["question"], self.letters, r["choices"])),
                             Message.assistant(self.letters[int(r["answer"])])])


class GSM8KTask(_RowTask):
    name = "GSM8K"

    def get_example(self, idx):
        r = self._row(idx)
        if r is None:
            return None
        return Conversation([Message.user(r["question"]), Message(ASSISTANT, r["answer"], parse_gsm8k_answer(r["answer"]))])

    def evaluate(self, conv, response):
        expected = (extract_hash_answer(conv.messages[-1].content) or "") if conv.messages else ""
        predicted = extract_hash_answer(response) or ""
        ok = bool(expected) and predicted == expected
        return EvalResult(ok, 1.0 if ok else 0.0, expected, predicted)


def _parse_messages(raw) -> Optional[List[Message]]:
    msgs = []
    for m in raw:
        role = {"system": "system", "user": USER, "assistant": ASSISTANT, "tool": TOOL}.get(m.get("role"))
        if role is None or not isinstance(m.get("content"), str):
            return None
        msgs.append(Message(role, m["content"]))
    body = msgs[1:] if msgs and msgs[0].role == "system" else msgs
    if len(body) < 2 or any(m.role != (USER if i % 2 == 0 else ASSISTANT) for i, m in enumerate(body)):
        return None                                   # must alternate user / assistant
    return msgs


class SmolTalkTask(_RowTask):
    name = "SmolTalk"

    def __init__(self, rows, config=None):
        super().__init__([r for r in rows if _parse_messages(r.get("messages", [])) is not None], config)

    def get_example(self, idx):
        r = self._row(idx)
        return None if r is None else Conversation(_parse_messages(r["messages"]))

    def evaluate(self, conv, response):
        expected = conv.messages[-1].content if conv.messages else ""
        return EvalResult(response.strip() == expected.strip(), 1.0 if response.strip() == expected.strip() else 0.0, expected, response)


class CustomJSONTask(SmolTalkTask):
    """One JSON array of ``{"role", "content"}`` messages per line."""
    name = "CustomJSON"

    @staticmethod
    def from_file(path: str) -> "CustomJSONTask":
        return CustomJSONTask([{"messages": m if isinstance(m, list) else m.get("messages", [])} for m in load_jsonl_from_file(path)])


class SpellingBeeTask(EvalTask):
    """Count a letter in a word; generated from a word list with the reference's LCG."""
    name = "SpellingBee"

    def __init__(self, words: Sequence[str], size: int = 1000, seed: int = 42):
        self.words, self._size, self.seed = list(words), size, seed

    def size(self):
        return self._size

    def get_example(self, idx):
        if not self.words or not 0 <= idx < self._size:
            return None
        s = lcg_next(self.seed + idx)
        word = self.words[s % len(self.words)]
        s = lcg_next(s)
        letter = word[s % len(word)]
        return Conversation([Message.user(f"How many {letter} are in the word {word}?"),
                             Message.assistant(f"#### {word.count(letter)}")])

    def evaluate(self, conv, response):
        expected = extract_hash_answer(conv.messages[-1].content) or ""
        predicted = extract_hash_answer(response) or ""
        ok = bool(expected) and expected == predicted
        return EvalResult(ok, 1.0 if ok else 0.0, expected, predicted)


# ---- loaders ------------------------------------------------------------------------------------------------------------
def load_jsonl_from_file(path: str) -> List:
    with open(path, encoding="utf-8") as f:
        return [json.loads(l) for l in f if l.strip()]


def load_jsonl_from_url(url: str, cache_dir: str, filename: str, log=None, fetch=None) -> List:
    import os
    dest = os.path.join(dl.expand_home(cache_dir), filename)
    if not dl.download_with_retry(url, dest, log=log, fetch=fetch):
        raise IOError(f"failed to fetch {url}")
    return load_jsonl_from_file(dest)


def load_arc(subset: str, split: str, cache_dir="~/.cache/huggingface", log=None) -> List[dict]:
    return pq.read_parquet_to_json(dl.ensure_hf_parquet("allenai/ai2_arc", subset, split, cache_dir, log=log))


def load_gsm8k(subset: str = "main", split: str = "train", cache_dir="~/.cache/huggingface", log=None) -> List[dict]:
    return pq.read_parquet_to_json(dl.ensure_hf_parquet("openai/gsm8k", subset, split, cache_dir, log=log))


def load_mmlu(subset: str, split: str, cache_dir="~/.cache/huggingface", log=None) -> List[dict]:
    return pq.read_parquet_to_json(dl.ensure_hf_parquet("cais/mmlu", subset, split, cache_dir, log=log))


def load_smoltalk(split: str, cache_dir="~/.cache/huggingface", log=None) -> List[dict]:
    return pq.read_parquet_to_json(dl.ensure_hf_parquet("HuggingFaceTB/smol-smoltalk", "default", split, cache_dir, log=log))
