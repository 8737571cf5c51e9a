"""CORE evaluation: prompt rendering, shared prefix/suffix spans, scoring with an oracle model."""
import json

import torch

from tyr_b200.nanochat import core_eval as C

tok = lambda s: [ord(c) for c in s]


def oracle_model(favourite: str):
    """Predicts the next character of ``favourite`` wherever the context ends inside it, else uniform."""
    fav = tok(favourite)

    def model(ids):
        B, S = ids.shape
        logits = torch.zeros(B, S, 256)
        for b in range(B):
            seq = ids[b].tolist()
            for t in range(S):
                for k in range(min(len(fav) - 1, t + 1), 0, -1):
                    if seq[t - k + 1:t + 1] == fav[:k]:
                        logits[b, t, fav[k]] = 10.0
                        break
                else:
                    logits[b, t, fav[0]] = 2.0
        return logits
    return model


def test_rendering_and_spans():
    it = C.MCItem("Q: 2+2?", ["three", "four"], 1)
    ps = C.render_prompts_mc(it, " ", [C.MCItem("Q: 1+1?", ["two", "one"], 0)])
    assert ps[1] == "Q: 1+1? two\n\nQ: 2+2? four"
    info = C.batch_sequences_mc(tok, ps, 1)
    assert info.start_indices == [1 + len("Q: 1+1? two\n\nQ: 2+2? ")] * 2 and info.end_indices[1] == len(info.tokens[1])
    sc = C.SchemaItem(["The cat", "The dog"], " barked.", 1)
    si = C.batch_sequences_schema(tok, C.render_prompts_schema(sc, "", []), 1)
    assert [e - s for s, e in zip(si.start_indices, si.end_indices)] == [len(" barked.")] * 2
    a, b = C.render_prompts_lm(C.LMItem("the quick brown ", "fox"), " ")
    li = C.batch_sequences_lm(tok, a, b, 1)
    assert li.end_indices[0] - li.start_indices[0] == len(" fox")        # trailing delimiter is trimmed off the prefix
    assert C.find_common_prefix_length([[1, 2, 3], [1, 2, 4]]) == 2 and C.find_common_suffix_length([[9, 2, 3], [1, 2, 3]]) == 2


def test_scoring_with_oracle_models():
    mc = C.MCItem("pick", [" zzz", " abc"], 1)
    r = C.evaluate_mc(oracle_model(" abc"), C.batch_sequences_mc(tok, C.render_prompts_mc(mc, ""), 1), mc.gold)
    assert r.correct and r.losses[1] < r.losses[0]
    assert not C.evaluate_mc(oracle_model(" zzz"), C.batch_sequences_mc(tok, C.render_prompts_mc(mc, ""), 1), mc.gold).correct
    lm = C.LMItem("say", " hello")
    a, b = C.render_prompts_lm(lm, "")
    assert C.evaluate_lm(oracle_model(" hello"), C.batch_sequences_lm(tok, a, b, 1)).correct
    assert not C.evaluate_lm(oracle_model(" world"), C.batch_sequences_lm(tok, a, b, 1)).correct
    items = [C.MCItem("q", [" abc", " zzz"], 0), C.MCItem("q", [" zzz", " abc"], 1), C.MCItem("q", [" abc", " zzz"], 1)]
    acc = C.evaluate_task(oracle_model(" abc"), tok, C.TaskMeta(C.MC, 0, "t", ""), items, C.EvalConfig(bos_token=1))
    assert abs(acc - 2 / 3) < 1e-9
    assert C.compute_core_score([("a", 0.5), ("b", 1.0)]) == 0.75 and len(C.CORE_TASKS) == 8
    assert len(C.get_fewshot_examples(items, 2, 0)) == 2 and items[0] not in C.get_fewshot_examples(items, 2, 0)


def test_bundle_parsers_and_loader(tmp_path):
    assert C.parse_arc_item({"question": "q", "choices": {"label": ["A", "B"], "text": ["x", "y"]}, "answerKey": "B"}).gold == 1
    w = C.parse_winogrande_item({"sentence": "The _ ran.", "option1": "cat", "option2": "dog", "answer": "2"})
    assert w.context_options == ["The cat", "The dog"] and w.continuation == " ran." and w.gold == 1
    assert C.parse_boolq_item({"passage": "p", "question": "q", "answer": True}).gold == 1
    assert C.parse_lambada_item({"text": "a b c"}).continuation == " c"
    d = tmp_path / "eval_data"
    d.mkdir()
    (d / "piqa.jsonl").write_text(json.dumps({"goal": "g", "sol1": " abc", "sol2": " zzz", "label": 0}) + "\n")
    score, accs = C.evaluate_core(oracle_model(" abc"), tok, str(tmp_path), C.EvalConfig(bos_token=1))
    assert accs == [("piqa", 1.0)] and score == 1.0
