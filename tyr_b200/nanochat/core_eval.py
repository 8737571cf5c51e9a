"""CORE evaluation (DCLM): multiple-choice, schema and language-modelling tasks scored from token losses
(Examples/NanoChat/Eval/{CORE,COREData}.lean).

* multiple choice: one prompt per choice sharing a prefix; the choice with the lowest mean loss over its own
  continuation wins;
* schema: one prompt per context option sharing a suffix; lowest mean loss over the shared continuation wins;
* language modelling: the continuation must be the arg-max prediction at every one of its positions.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..data.task import lcg_next

MC, SCHEMA, LM = "multiple_choice", "schema", "language_modeling"


@dataclass
class TaskMeta:
    task_type: str
    num_fewshot: int = 0
    task_name: str = ""
    continuation_delimiter: str = " "


@dataclass
class MCItem:
    query: str
    choices: List[str]
    gold: int


@dataclass
class SchemaItem:
    context_options: List[str]
    continuation: str
    gold: int


@dataclass
class LMItem:
    context: str
    continuation: str


def render_fewshot_mc(examples: Sequence[MCItem], delim: str) -> str:
    return "".join(f"{e.query}{delim}{e.choices[e.gold]}\n\n" for e in examples)


def render_prompts_mc(item: MCItem, delim: str, fewshot: Sequence[MCItem] = ()) -> List[str]:
    pre = render_fewshot_mc(fewshot, delim)
    return [f"{pre}{item.query}{delim}{c}" for c in item.choices]


def render_fewshot_schema(examples: Sequence[SchemaItem], delim: str) -> str:
    return "".join(f"{e.context_options[e.gold]}{delim}{e.continuation}\n\n" for e in examples)


def render_prompts_schema(item: SchemaItem, delim: str, fewshot: Sequence[SchemaItem] = ()) -> List[str]:
    pre = render_fewshot_schema(fewshot, delim)
    return [f"{pre}{c}{delim}{item.continuation}" for c in item.context_options]


def render_fewshot_lm(examples: Sequence[LMItem], delim: str) -> str:
    return "".join(f"{e.context.strip()}{delim}{e.continuation}\n\n" for e in examples)


def render_prompts_lm(item: LMItem, delim: str, fewshot: Sequence[LMItem] = ()) -> Tuple[str, str]:
    without = render_fewshot_lm(fewshot, delim) + item.context.strip() + delim
    return without.strip(), without + item.continuation


def find_common_prefix_length(seqs: Sequence[Sequence[int]]) -> int:
    n = min(len(s) for s in seqs)
    for i in range(n):
        if any(s[i] != seqs[0][i] for s in seqs):
            return i
    return n


def find_common_suffix_length(seqs: Sequence[Sequence[int]]) -> int:
    n = min(len(s) for s in seqs)
    for i in range(1, n + 1):
        if any(s[-i] != seqs[0][-i] for s in seqs):
            return i - 1
    return n


@dataclass
class BatchInfo:
    tokens: List[List[int]]
    start_indices: List[int]
    end_indices: List[int]


def batch_sequences_mc(tokenize, prompts: Sequence[str], bos: int) -> BatchInfo:
    toks = [[bos] + list(tokenize(p)) for p in prompts]
    cp = find_common_prefix_length(toks)
    return BatchInfo(toks, [cp] * len(toks), [len(t) for t in toks])


def batch_sequences_schema(tokenize, prompts: Sequence[str], bos: int) -> BatchInfo:
    toks = [[bos] + list(tokenize(p)) for p in prompts]
    cs = find_common_suffix_length(toks)
    return BatchInfo(toks, [len(t) - cs for t in toks], [len(t) for t in toks])


def batch_sequences_lm(tokenize, prompt_without: str, prompt_with: str, bos: int) -> BatchInfo:
    a, b = [bos] + list(tokenize(prompt_without)), [bos] + list(tokenize(prompt_with))
    return BatchInfo([b], [len(a)], [len(b)])


def pad_sequences(seqs: Sequence[Sequence[int]], pad: int) -> torch.Tensor:
    L = max(len(s) for s in seqs)
    return torch.tensor([list(s) + [pad] * (L - len(s)) for s in seqs], dtype=torch.int64)


def compute_losses(logits: torch.Tensor, ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-position loss of predicting ids[:, t+1] from position t, and the arg-max predictions ([B, S-1] each)."""
    lg = logits[:, :-1].float()
    tgt = ids[:, 1:]
    loss = F.cross_entropy(lg.reshape(-1, lg.shape[-1]), tgt.reshape(-1), reduction="none").reshape(tgt.shape)
    return loss, lg.argmax(-1)


@dataclass
class EvalResult:
    correct: bool
    predicted: int = 0
    gold: int = 0
    losses: List[float] = field(default_factory=list)


ModelFn = Callable[[torch.Tensor], torch.Tensor]
"""ids int64 [B, S] -> logits [B, S, V]"""


@torch.no_grad()
def evaluate_mc(model: ModelFn, info: BatchInfo, gold: int, pad: int = 0, device="cpu") -> EvalResult:
    ids = pad_sequences(info.tokens, pad).to(device)
    loss, _ = compute_losses(model(ids), ids)
    means = [float(loss[i, s - 1:e - 1].mean()) if e > s else float("inf") for i, (s, e) in enumerate(zip(info.start_indices, info.end_indices))]
    pred = min(range(len(means)), key=lambda i: means[i])
    return EvalResult(pred == gold, pred, gold, means)


@torch.no_grad()
def evaluate_lm(model: ModelFn, info: BatchInfo, pad: int = 0, device="cpu") -> EvalResult:
    ids = pad_sequences(info.tokens, pad).to(device)
    _, preds = compute_losses(model(ids), ids)
    s, e = info.start_indices[0], info.end_indices[0]
    ok = bool((preds[0, s - 1:e - 1] == ids[0, s:e]).all()) if e > s else False
    return EvalResult(ok)


@dataclass
class EvalConfig:
    max_examples: int = 0          # 0 = all
    bos_token: int = 0
    pad_token: int = 0
    max_seq_len: int = 2048
    seed: int = 42


def get_fewshot_examples(items: Sequence, num_fewshot: int, exclude_idx: int, seed: int = 42) -> List:
    """Deterministic (LCG) sample of other items."""
    if num_fewshot == 0 or len(items) <= 1:
        return []
    out, state, seen = [], (seed + exclude_idx) & ((1 << 64) - 1), {exclude_idx}
    while len(out) < min(num_fewshot, len(items) - 1):
        state = lcg_next(state)
        j = state % len(items)
        if j not in seen:
            seen.add(j)
            out.append(items[j])
    return out


def evaluate_single_example(model: ModelFn, tokenize, meta: TaskMeta, items: Sequence, idx: int, cfg: EvalConfig, device="cpu") -> EvalResult:
    item = items[idx]
    few = get_fewshot_examples(items, meta.num_fewshot, idx, cfg.seed)
    d = meta.continuation_delimiter

    def crop(info: BatchInfo) -> BatchInfo:
        """Keep the last ``max_seq_len`` tokens of over-long prompts, shifting the scored span with them."""
        toks, st, en = [], [], []
        for t, s, e in zip(info.tokens, info.start_indices, info.end_indices):
            cut = max(0, len(t) - cfg.max_seq_len)
            toks.append(t[cut:]); st.append(max(1, s - cut)); en.append(e - cut)
        return BatchInfo(toks, st, en)
    if meta.task_type == MC:
        return evaluate_mc(model, crop(batch_sequences_mc(tokenize, render_prompts_mc(item, d, few), cfg.bos_token)), item.gold, cfg.pad_token, device)
    if meta.task_type == SCHEMA:
        return evaluate_mc(model, crop(batch_sequences_schema(tokenize, render_prompts_schema(item, d, few), cfg.bos_token)), item.gold, cfg.pad_token, device)
    a, b = render_prompts_lm(item, d, few)
    return evaluate_lm(model, crop(batch_sequences_lm(tokenize, a, b, cfg.bos_token)), cfg.pad_token, device)


def evaluate_task(model: ModelFn, tokenize, meta: TaskMeta, items: Sequence, cfg: EvalConfig, device="cpu", rank: int = 0,
                  world_size: int = 1) -> float:
    """Accuracy over the task (rank-strided examples; the caller averages across ranks)."""
    n = len(items) if cfg.max_examples == 0 else min(cfg.max_examples, len(items))
    idxs = range(rank, n, max(1, world_size))
    res = [evaluate_single_example(model, tokenize, meta, items, i, cfg, device).correct for i in idxs]
    return sum(res) / len(res) if res else 0.0


CORE_TASKS = [TaskMeta(MC, 0, "arc_easy"), TaskMeta(MC, 0, "arc_challenge"), TaskMeta(MC, 0, "hellaswag"), TaskMeta(SCHEMA, 0, "winogrande"),
              TaskMeta(MC, 0, "piqa"), TaskMeta(MC, 0, "mmlu"), TaskMeta(MC, 0, "boolq"), TaskMeta(LM, 0, "lambada")]


def compute_core_score(task_accuracies: Sequence[Tuple[str, float]]) -> float:
    return sum(a for _, a in task_accuracies) / len(task_accuracies) if task_accuracies else 0.0


# ---- bundle parsing (COREData.lean) --------------------------------------------------------------------------------------
def parse_mc_query_choices_gold(j: dict) -> Optional[MCItem]:
    if all(k in j for k in ("query", "choices", "gold")):
        return MCItem(j["query"], list(j["choices"]), int(j["gold"]))
    return None


def parse_arc_item(j: dict) -> Optional[MCItem]:
    try:
        labels, texts = j["choices"]["label"], j["choices"]["text"]
        return MCItem(f"Question: {j['question']}\nAnswer:", list(texts), labels.index(j["answerKey"]))
    except (KeyError, ValueError):
        return None


def parse_hellaswag_item(j: dict) -> Optional[MCItem]:
    try:
        return MCItem(j["ctx"], list(j["endings"]), int(j["label"]))
    except (KeyError, ValueError):
        return None


def parse_winogrande_item(j: dict) -> Optional[SchemaItem]:
    try:
        s = j["sentence"]
        k = s.index("_")
        return SchemaItem([s[:k] + j["option1"], s[:k] + j["option2"]], s[k + 1:], int(j["answer"]) - 1)
    except (KeyError, ValueError):
        return None


def parse_piqa_item(j: dict) -> Optional[MCItem]:
    try:
        return MCItem(f"Question: {j['goal']}\nAnswer:", [j["sol1"], j["sol2"]], int(j["label"]))
    except (KeyError, ValueError):
        return None


def parse_sciq_item(j: dict) -> Optional[MCItem]:
    try:
        return MCItem(f"Question: {j['question']}\nAnswer:", [j["distractor1"], j["distractor2"], j["distractor3"], j["correct_answer"]], 3)
    except KeyError:
        return None


def parse_boolq_item(j: dict) -> Optional[MCItem]:
    try:
        return MCItem(f"{j['passage']}\nQuestion: {j['question']}?\nAnswer:", ["no", "yes"], 1 if j["answer"] else 0)
    except KeyError:
        return None


def parse_lambada_item(j: dict) -> Optional[LMItem]:
    text = j.get("text")
    if not text or " " not in text.strip():
        return None
    ctx, last = text.strip().rsplit(" ", 1)
    return LMItem(ctx, " " + last)


PARSERS = {"arc_easy": parse_arc_item, "arc_challenge": parse_arc_item, "hellaswag": parse_hellaswag_item, "winogrande": parse_winogrande_item,
           "piqa": parse_piqa_item, "sciq": parse_sciq_item, "boolq": parse_boolq_item, "lambada": parse_lambada_item, "mmlu": parse_mc_query_choices_gold}


def load_core_task_data(bundle_dir: str, task_name: str, dataset_uri: Optional[str] = None) -> List:
    """Items of one task from ``<bundle>/eval_data/<uri>`` (jsonl).  Rows already in query/choices/gold form are used as is."""
    path = os.path.join(bundle_dir, "eval_data", dataset_uri or f"{task_name}.jsonl")
    out = []
    with open(path, encoding="utf-8") as f:
        for line in f:
            if not line.strip():
                continue
            j = json.loads(line)
            item = parse_mc_query_choices_gold(j) or PARSERS.get(task_name, lambda _: None)(j)
            if item is None and "context_options" in j:
                item = SchemaItem(list(j["context_options"]), j["continuation"], int(j["gold"]))
            if item is None and "context" in j and "continuation" in j:
                item = LMItem(j["context"], j["continuation"])
            if item is not None:
                out.append(item)
    return out


def evaluate_core(model: ModelFn, tokenize, bundle_dir: str, cfg: EvalConfig, device="cpu", tasks: Sequence[TaskMeta] = CORE_TASKS,
                  log=None) -> Tuple[float, List[Tuple[str, float]]]:
    accs = []
    for meta in tasks:
        try:
            items = load_core_task_data(bundle_dir, meta.task_name)
        except FileNotFoundError:
            if log:
                log(f"[CORE] {meta.task_name}: data not found, skipped")
            continue
        acc = evaluate_task(model, tokenize, meta, items, cfg, device)
        accs.append((meta.task_name, acc))
        if log:
            log(f"[CORE] {meta.task_name}: {acc:.4f} over {len(items)} examples")
    return compute_core_score(accs), accs
