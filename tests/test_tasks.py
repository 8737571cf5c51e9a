"""Task layer: deterministic shuffles, rendering masks, collation, token stream, eval tasks, parquet cursor, downloads."""
import os

import pytest
import torch

from tyr_b200.data import download as DL
from tyr_b200.data import parquet as PQ
from tyr_b200.data import task as T
from tyr_b200.data import task_class as TC
from tyr_b200.data import tasks as TS

CT = T.ChatTokens(bos=1, user_start=2, user_end=3, assistant_start=4, assistant_end=5, python_start=6, python_end=7,
                  output_start=8, output_end=9)
enc = lambda s: [100 + ord(c) % 50 for c in s]


def test_lcg_shuffle_is_deterministic_and_a_permutation():
    a = T.shuffle_indices(list(range(20)), 42)
    assert a == T.shuffle_indices(list(range(20)), 42) and sorted(a) == list(range(20)) and a != list(range(20))
    assert T.lcg_next(0) == 1442695040888963407
    mix = TS.create_midtraining_mixture("tyr")
    assert mix.size() == 2 * 50 + 5 + 16 + 3 and mix.get(0).messages


def test_render_masks_only_assistant_and_tool_calls():
    conv = T.Conversation([T.Message.system("sys"), T.Message.user("hi"),
                           T.Message(T.ASSISTANT, "x", [T.ContentPart("text", "ab"), T.ContentPart("tool_call:calculator", "1+1"),
                                                        T.ContentPart("tool_result", "2")]),
                           T.Message(T.TOOL, "z")])
    r = T.render_conversation(conv, CT, enc)
    assert r.tokens[:2] == [1, 2] and r.mask[:2] == [0, 0]
    n_sys_user = len(enc("sys\n\nhi"))                       # the system message merges into the first user turn
    assert r.tokens[2 + n_sys_user] == 3
    a0 = 3 + n_sys_user
    assert r.tokens[a0] == 4 and r.mask[a0] == 0
    body = r.mask[a0 + 1:]
    assert body[:2] == [1, 1] and body[2] == 1 and r.tokens[a0 + 3] == 6        # python_start trained
    out_start = r.tokens.index(8)
    assert r.mask[out_start] == 0 and r.mask[out_start + 1] == 0
    end = r.tokens.index(5)
    assert r.mask[end] == 1 and len(r.tokens) == len(r.mask)


def test_collate_pads_and_truncates():
    a = T.TokenizedConversation([1, 2, 3, 4, 5], [0, 1, 1, 1, 1], T.Conversation())
    b = T.TokenizedConversation([1, 2], [0, 1], T.Conversation())
    batch = T.collate([a, b], 4, pad_token=9)
    assert batch.tokens.tolist() == [[1, 2, 3, 4], [1, 2, 9, 9]] and batch.mask[1].tolist() == [0, 1, 0, 0] and batch.lengths == [4, 2]
    assert T.collate([], 4).batch_size == 0


def test_iterator_epochs_and_token_stream_windows():
    mix = TS.create_sft_mixture("tyr").to_conversation_mixture()
    it = T.TaskIterator(mix, 8, 64, CT, enc)
    n = 0
    while (b := it.next_batch()) is not None:
        n += b.batch_size
    assert n == mix.size() and it.epoch == 1 and it.progress() == 0.0
    s0 = T.TaskTokenStream(mix, 2, 16, CT, enc, rank=0, world_size=2)
    x, y = s0.next_gpt_batch()
    assert x.shape == (2, 16) and torch.equal(x.reshape(-1)[1:], y.reshape(-1)[:-1])
    x2, _ = s0.next_gpt_batch()
    assert x2[0, 0] == y[1, -1]                              # windows continue where the last one ended
    s1 = T.TaskTokenStream(mix, 2, 16, CT, enc, rank=1, world_size=2)
    assert not torch.equal(s1.next_gpt_batch()[0], x)


def test_eval_tasks_and_mixtures():
    arc = TS.ARCTask([{"question": "q?", "choices": {"label": ["A", "B"], "text": ["x", "y"]}, "answerKey": "B"}])
    c = arc.get_example(0)
    assert "- y=B" in c.messages[0].content and arc.evaluate(c, " B").correct and not arc.evaluate(c, "A").correct
    g = TS.GSM8KTask([{"question": "q", "answer": "3*4=<<3*4=12>>12\n#### 1,200"}] * 5, TS.SliceConfig(1, None, 2))
    assert g.size() == 2
    cg = g.get_example(0)
    kinds = [p.type for p in cg.messages[1].parts]
    assert kinds == ["text", "tool_call:calculator", "tool_result", "text"] and cg.messages[1].parts[1].content == "3*4"
    assert g.evaluate(cg, "so #### 1200").correct and g.reward(cg, "#### 7") == 0.0
    assert TS.extract_hash_answer("no marker") is None and TS.extract_letter_answer("C is right") == "C"
    mm = TS.MMLUTask([{"question": "q", "choices": ["a", "b", "c", "d"], "answer": 2}])
    assert mm.get_example(0).messages[1].content == "C" and mm.eval_type() == TC.CATEGORICAL
    st = TS.SmolTalkTask([{"messages": [{"role": "user", "content": "u"}, {"role": "assistant", "content": "a"}]},
                          {"messages": [{"role": "assistant", "content": "bad"}]}])
    assert st.size() == 1
    bee = TS.SpellingBeeTask(["banana", "kiwi"], size=10)
    e = bee.get_example(3)
    assert bee.evaluate(e, e.messages[1].content).correct
    mix = TC.mixture_weighted([TC.entry(arc, 2), TC.entry(g, 1)])
    assert mix.size() == 4 and mix.reward(0, "B") in (0.0, 1.0)
    assert mix.to_conversation_mixture_sharded(1, 2).size() == 2


def test_parquet_rows_and_resumable_cursor(tmp_path):
    import pyarrow as pa
    import pyarrow.parquet as pq
    paths = []
    for f in range(2):
        p = str(tmp_path / f"s{f}.parquet")
        pq.write_table(pa.table({"text": [f"f{f}d{i}" for i in range(10)], "n": list(range(10))}), p, row_group_size=3)
        paths.append(p)
    assert PQ.read_parquet_to_json(paths[0])[2] == {"text": "f0d2", "n": 2}
    assert len(list(PQ.read_parquet_to_json_streaming(paths[1]))) == 10 and PQ.num_row_groups(paths[0]) == 4
    s = PQ.ParquetDocumentStream(paths, rank=1, world_size=2)
    got = [next(s) for _ in range(9)]
    assert got[:8] == ["f0d3", "f0d4", "f0d5", "f0d9", "f1d3", "f1d4", "f1d5", "f1d9"] and got[8] == "f0d3" and s.cursor.epoch == 1
    resumed = PQ.ParquetDocumentStream(paths, rank=1, world_size=2, cursor=PQ.ParquetCursor.from_json(s.cursor.to_json()))
    assert next(resumed) == next(s)


def test_download_with_retry_backoff(tmp_path):
    calls, sleeps = [], []

    def fetch(url, dest):
        calls.append(url)
        if len(calls) < 3:
            raise IOError("boom")
        open(dest, "w").write("ok")
    dest = str(tmp_path / "a" / "f.txt")
    assert DL.download_with_retry("u", dest, 5, 10, fetch=fetch, sleep=sleeps.append)
    assert len(calls) == 3 and sleeps == [0.01, 0.02] and open(dest).read() == "ok" and not os.path.exists(dest + ".tmp")
    assert DL.download_with_retry("u", dest, fetch=lambda u, d: 1 / 0)            # already there: no fetch
    assert not DL.download_with_retry("u", str(tmp_path / "g"), 2, 1, fetch=lambda u, d: 1 / 0, sleep=lambda s: None)
