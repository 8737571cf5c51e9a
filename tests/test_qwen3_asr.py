"""Qwen3-ASR: length rules, chunked/windowed audio encoder, placeholder splicing, prompt building, forced alignment
utilities, greedy transcription and streaming on a tiny random model."""
import pytest
import torch

from tyr_b200.models import qwen as Q
from tyr_b200.models import qwen3_asr as A


def tiny_cfg(aligner=False):
    audio = A.AudioEncoderConfig(num_mel_bins=16, encoder_layers=2, encoder_attention_heads=2, encoder_ffn_dim=32, d_model=16, n_window=4, output_dim=24,
                                 n_window_infer=16, downsample_hidden_size=6)
    text = Q.QwenConfig(vocab_size=64, hidden_size=24, intermediate_size=48, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1, half_head_dim=6)
    th = A.ThinkerConfig(audio, text, audio_token_id=60, model_type="qwen3_forced_aligner" if aligner else "qwen3_asr_thinker", classify_num=50 if aligner else 0)
    return A.Qwen3ASRConfig(th, timestamp_token_id=61, timestamp_segment_time=80.0)


def test_length_rules_and_config_validation():
    assert [A.feat_extract_output_length(n) for n in (0, 1, 7, 8, 100, 101, 250)] == [0, 1, 1, 1, 13, 14, 33]
    cfg = A.AudioEncoderConfig()
    assert A.build_chunk_lengths(cfg, [450, 0, 200]) == [200, 200, 50, 200]
    assert A.attention_window_lengths(cfg, 58, 26) == [52, 6]
    with pytest.raises(ValueError, match="whole number"):
        A.AudioEncoderConfig(n_window=100, n_window_infer=300)
    with pytest.raises(ValueError, match="classify_num"):
        A.ThinkerConfig(model_type="x_forced_aligner")
    j = {"thinker_config": {"audio_config": {"d_model": 1024, "encoder_attention_heads": 16, "output_dim": 2048}, "text_config": {"hidden_size": 2048, "num_hidden_layers": 4},
                            "audio_token_id": 7}, "timestamp_token_id": 9}
    c = A.Qwen3ASRConfig.from_json(j)
    assert c.thinker.audio.d_model == 1024 and c.thinker.text.hidden_size == 2048 and c.thinker.audio_token_id == 7 and c.timestamp_token_id == 9


def test_audio_encoder_token_counts_and_chunk_locality():
    cfg = tiny_cfg()
    enc = A.init_audio_encoder(cfg.thinker.audio)
    feats = torch.randn(2, 16, 37)
    out = A.encode_audio(enc, feats, [37, 20])
    assert [o.shape for o in out] == [(A.audio_token_count(cfg.thinker.audio, 37), 24), (A.audio_token_count(cfg.thinker.audio, 20), 24)]
    assert A.audio_token_count(A.AudioEncoderConfig(), 450) == A.feat_extract_output_length(450)
    # attention is confined to windows of n_window_infer frames: changing the audio after the first window leaves its tokens alone
    feats2 = feats.clone()
    feats2[0, :, 16:] += 1.0
    out2 = A.encode_audio(enc, feats2, [37, 20])
    first = A.feat_extract_output_length(8) * 2
    assert torch.allclose(out[0][:first], out2[0][:first], atol=1e-5) and not torch.allclose(out[0][first:], out2[0][first:], atol=1e-3)


def test_processor_prompt_and_expansion():
    p = A.Processor()
    assert p.build_asr_prompt("ctx", "English") == ("<|im_start|>system\nctx<|im_end|>\n<|im_start|>user\n<|audio_start|><|audio_pad|><|audio_end|><|im_end|>\n"
                                                   "<|im_start|>assistant\nlanguage English<asr_text>")
    assert p.replace_multimodal_special_tokens(["a<|audio_pad|>b", "<|audio_pad|>"], [2, 1]) == ["a<|audio_pad|><|audio_pad|>b", "<|audio_pad|>"]
    with pytest.raises(ValueError, match="Not enough"):
        p.replace_multimodal_special_tokens(["<|audio_pad|><|audio_pad|>"], [1])
    enc = lambda s: [ord(c) % 50 for c in s]
    ids = p.encode_with_expanded_audio_token_ids(enc, "x<|audio_pad|>y", [3], 60)
    assert ids == enc("x") + [60, 60, 60] + enc("y")
    assert A.Processor.get_chunked_index([0, 1, 5, 6, 11], 5) == [(0, 2), (2, 4), (4, 5)]


def test_forced_alignment_text_and_timestamp_repair():
    words, prompt = A.encode_timestamp_text("Hello, wor'ld 你好!", "English")
    assert words == ["Hello", "wor'ld", "你", "好"] and prompt.endswith("好<timestamp><timestamp>") and prompt.count("<timestamp>") == 8
    assert A.encode_timestamp_text("안녕 hi", "Korean")[0] == ["안", "녕", "hi"]
    assert A.fix_timestamp([10, 20, 5, 40, 50]) == [10, 20, 20, 40, 50]                    # one outlier snaps to the nearer neighbour
    assert A.fix_timestamp([10, 20, 900, 800, 700, 60, 70, 80]) == [10, 20, 30, 40, 50, 60, 70, 80]   # a run of three is interpolated
    items = A.parse_timestamp(["a", "b"], [100, 200, 300])
    assert (items[0].start_time, items[0].end_time, items[1].start_time, items[1].end_time) == (0.1, 0.2, 0.3, 0.3)
    cfg = tiny_cfg(aligner=True)
    ids = torch.tensor([[5, 61, 61, 7, 61, 61]])
    logits = torch.zeros(1, 6, 50)
    for pos, cls in ((1, 2), (2, 5), (4, 6), (5, 9)):
        logits[0, pos, cls] = 1.0
    out = A.align_from_logits(cfg, ids, logits, [["x", "y"]])[0]
    assert [(i.text, i.start_time, i.end_time) for i in out] == [("x", 0.16, 0.4), ("y", 0.48, 0.72)]


def test_splice_generation_and_aligner_forward():
    cfg = tiny_cfg()
    m = A.init(cfg)
    feats = torch.randn(1, 16, 30)
    n_audio = A.audio_token_count(cfg.thinker.audio, 30)
    ids = torch.tensor([[3, 4] + [60] * n_audio + [5, 6]])
    emb = A.build_inputs_embeds(m, ids, A.encode_audio(m.audio_tower, feats))
    assert torch.equal(emb[0, :2], m.lm.embed_tokens(ids[:, :2])[0]) and not torch.equal(emb[0, 2], m.lm.embed_tokens(ids[:, 2:3])[0, 0])
    with pytest.raises(ValueError, match="placeholders"):
        A.build_inputs_embeds(m, ids[:, 1:-3], A.encode_audio(m.audio_tower, feats))
    logits = A.forward(m, ids, feats)
    new = A.generate_greedy(m, ids, feats, max_new_tokens=5, eos_token_ids=(63,))[0]
    assert logits.shape == (1, ids.shape[1], 64) and len(new) <= 5 and new[0] == int(logits[0, -1].argmax())
    al = A.init(tiny_cfg(aligner=True))
    assert A.forward(al, ids, feats).shape == (1, ids.shape[1], 50)
    sd = A.state_dict(m)
    assert "thinker.audio_tower.layers.1.self_attn.out_proj.bias" in sd and "thinker.audio_tower.conv2d3.weight" in sd


def test_transcription_chunking_and_streaming(tmp_path):
    cfg = tiny_cfg()
    m = A.init(cfg)
    special = {"<|im_start|>": 50, "<|im_end|>": 51, "<|audio_start|>": 52, "<|audio_end|>": 53}

    def encode(s):
        out, i = [], 0
        while i < len(s):
            for k, v in special.items():
                if s.startswith(k, i):
                    out.append(v)
                    i += len(k)
                    break
            else:
                out.append(ord(s[i]) % 48)
                i += 1
        return out
    decode = lambda ids: " ".join(f"w{t}" for t in ids)
    wave = torch.randn(16000)
    r = A.transcribe_waveform(m, encode, decode, wave, language="english", max_new_tokens=4)
    assert r.language == "English" and len(r.text.split()) <= 4
    with pytest.raises(ValueError, match="Unsupported language"):
        A.transcribe_waveform(m, encode, decode, wave, language="Klingon")
    quiet = torch.cat([torch.randn(30000), torch.zeros(3000), torch.randn(30000)])
    chunks = A.split_audio_into_chunks(quiet, 1000, 35.0, search_seconds=6.0)                 # 63 s at 1 kHz, cut in the silent second
    assert len(chunks) == 2 and 30.0 <= chunks[1][1] <= 33.0 and sum(c.numel() for c, _ in chunks) == quiet.numel()
    assert A.parse_asr_output("language French<asr_text>bonjour") == ("French", "bonjour")
    st = A.StreamingTranscriber(m, encode, decode, chunk_seconds=0.5, language="English", max_new_tokens=3)
    for _ in range(3):
        st.push(torch.randn(8000))
    final = st.finish()
    assert st.decodes == 4 and isinstance(final, str)
