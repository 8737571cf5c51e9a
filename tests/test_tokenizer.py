"""BPE training / round trips / binary format, HF tokenizer.json loading, chat templates."""
import json

import pytest

from tyr_b200 import tokenizer as tk


def test_train_encode_decode_roundtrip():
    corpus = ["the quick brown fox jumps over the lazy dog " * 20, "hello world, hello there! 12345 naïve café"] * 5
    tok = tk.train_bpe(corpus, 256 + 40 + 2, ["<|bos|>", "<|assistant_start|>"])
    assert tok.vocab_size == 298 and len(tok.merges) == 40
    s = "hello there, the quick café 123"
    ids = tok.encode(s, prepend="<|bos|>")
    assert ids[0] == tok.get_bos_token_id() and tok.decode(ids[1:]) == s
    assert len(tok.encode_ordinary("the quick")) < len("the quick".encode())
    assert tok.encode("a<|assistant_start|>b")[1] == tok.encode_special("<|assistant_start|>")
    assert tok.encode("a<|assistant_start|>b", allowed_special=False) != tok.encode("a<|assistant_start|>b")
    tb = tok.token_bytes()
    assert tb[ord("a")] == 1 and tb[tok.get_bos_token_id()] == 0 and max(tb) > 1
    with pytest.raises(KeyError):
        tok.encode_special("<|nope|>")


def test_binary_format_roundtrip(tmp_path):
    tok = tk.train_bpe(["abababab cdcdcd abab"] * 3, 256 + 5 + 1, ["<|bos|>"])
    raw = tok.serialize()
    assert raw[:8] == b"TYR_BPE1"
    p = str(tmp_path / "tok.bin")
    tok.save(p)
    t2 = tk.BPETokenizer.load(p)
    assert t2.encode("abab cd<|bos|>") == tok.encode("abab cd<|bos|>") and t2.special_tokens == tok.special_tokens
    with pytest.raises(ValueError):
        tk.BPETokenizer.deserialize(b"NOPE" + raw[4:])
    with pytest.raises(ValueError):
        tk.BPETokenizer.deserialize(raw[:40])


def test_pretokenize_gpt4_pattern():
    assert tk.pretokenize("Hello world's 1234!") == ["Hello", " world", "'s", " ", "123", "4", "!"]


def test_hf_tokenizer_json(tmp_path):
    b2u = tk.hf.bytes_to_unicode()
    sp = b2u[ord(" ")]
    vocab = {b2u[i]: i for i in range(256)}
    vocab.update({"he": 256, "ll": 257, "hell": 258, "hello": 259, sp + "w": 260})
    merges = ["h e", "l l", "he ll", "hell o", f"{sp} w"]
    j = {"model": {"type": "BPE", "vocab": vocab, "merges": merges},
         "added_tokens": [{"content": "<|im_start|>", "id": 300}, {"content": "<|im_end|>", "id": 301}]}
    (tmp_path / "tokenizer.json").write_text(json.dumps(j))
    t = tk.load_qwen3(str(tmp_path))
    ids = t.encode("<|im_start|>hello world<|im_end|>")
    assert ids[0] == 300 and ids[1] == 259 and ids[2] == 260 and ids[-1] == 301
    assert t.decode(ids) == "<|im_start|>hello world<|im_end|>" and t.decode(ids, skip_special=True) == "hello world"
    assert t.vocab_size == 302


def test_chat_templates():
    msgs = [{"role": "user", "content": "hi"}]
    assert tk.chatml_prompt(msgs) == "<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
    assert tk.chatml_prompt(msgs, system="be brief").startswith("<|im_start|>system\nbe brief<|im_end|>\n")
    assert tk.chatml_prompt(msgs, enable_thinking=False).endswith("<think>\n\n</think>\n\n")
    assert tk.gemma_prompt(msgs) == "<bos><start_of_turn>user\nhi<end_of_turn>\n<start_of_turn>model\n"


def test_native_bpe_loops_equal_the_python_loops(monkeypatch):
    """Merge training and chunk encoding in csrc/host/bpe.cpp against the Python loops: same merges (ties included), same ids,
    on random corpora with multi-byte characters, runs of one character (overlapping pairs) and special tokens."""
    import random
    from tyr_b200.tokenizer import bpe
    if bpe._host() is None:
        pytest.skip("host library not built")
    rng = random.Random(3)
    alpha = "abcdeé中 \n0123,.!'xyzAB"
    def corpus(n, L):
        return ["".join(rng.choice(alpha) * rng.choice([1, 1, 1, 2, 3]) for _ in range(rng.randint(1, L))) for _ in range(n)]
    for trial in range(8):
        docs = corpus(rng.randint(1, 30), rng.randint(1, 50))
        vocab = 256 + 1 + rng.randint(0, 100)
        monkeypatch.setattr(bpe, "_NATIVE", True)
        a = bpe.train_bpe(docs, vocab, ["<|bos|>"])
        monkeypatch.setattr(bpe, "_NATIVE", False)
        b = bpe.train_bpe(docs, vocab, ["<|bos|>"])
        assert [(m.left, m.right, m.result) for m in a.merges] == [(m.left, m.right, m.result) for m in b.merges], trial
        assert a.id_to_bytes == b.id_to_bytes and a.special_tokens == b.special_tokens
        texts = corpus(12, 60) + ["", "<|bos|>x<|bos|>", "éé中中", "aaaaaaa"]
        monkeypatch.setattr(bpe, "_NATIVE", True)
        ids_native = [a.encode(t) for t in texts]
        assert a._handle is not None or not a.merges                     # the native table was really used
        monkeypatch.setattr(bpe, "_NATIVE", False)
        ids_python = [b.encode(t) for t in texts]
        assert ids_native == ids_python, trial
        assert all(a.decode(e) == t for e, t in zip(ids_native, texts))


def test_native_bpe_reports_a_byte_without_a_token(monkeypatch):
    from tyr_b200.tokenizer import bpe
    if bpe._host() is None:
        pytest.skip("host library not built")
    monkeypatch.setattr(bpe, "_NATIVE", True)
    tok = bpe.BPETokenizer([bytes([i]) if i != ord("q") else b"" for i in range(256)] + [b"ab"], [bpe.MergeRule(ord("a"), ord("b"), 256)])
    assert tok.encode("abab") == [256, 256]
    with pytest.raises(KeyError):
        tok.encode("aqb")
