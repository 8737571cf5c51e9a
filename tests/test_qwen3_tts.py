"""Qwen3-TTS on tiny random models: config rules, sampling controls, frame generation, speaker encoder, speech decoder
(causality, chunked and streaming equivalence) and the end-to-end synthesis path."""
import pytest
import torch

from tyr_b200.models import qwen3_tts as T


def tiny_cfg(**kw):
    cp = T.CodePredictorConfig(vocab_size=32, hidden_size=16, intermediate_size=32, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1, half_head_dim=4)
    tk = T.TalkerConfig(cp, vocab_size=48, hidden_size=24, intermediate_size=32, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1, half_head_dim=6,
                        num_code_groups=4, text_hidden_size=20, text_vocab_size=64, codec_eos_token_id=40, codec_think_id=41, codec_nothink_id=42,
                        codec_think_bos_id=43, codec_think_eos_id=44, codec_pad_id=45, codec_bos_id=46, spk_id={"vivian": 39}, codec_language_id={"english": 38, "sichuan_dialect": 37})
    se = T.SpeakerEncoderConfig(mel_dim=8, enc_dim=24, enc_channels=(16, 16, 16, 16, 48), enc_attention_channels=8, enc_res2net_scale=4, enc_se_channels=8)
    base = dict(talker=tk, speaker_encoder=se, im_start_token_id=60, im_end_token_id=61, tts_pad_token_id=62, tts_bos_token_id=63, tts_eos_token_id=59)
    base.update(kw)
    return T.Qwen3TTSConfig(**base)


def tiny_decoder_cfg():
    return T.SpeechDecoderConfig(num_quantizers=3, codebook_size=32, codebook_dim=8, rvq_out_dim=12, latent_dim=16, hidden_size=12, num_layers=2, num_heads=2,
                                 head_dim=6, ffn_dim=16, sliding_window=5, upsample_stages=1, decoder_dim=16, decoder_rates=(2, 3))


def test_config_rules():
    c = tiny_cfg()
    assert c.supported_languages() == ["auto", "english"] and c.supported_speakers() == ["vivian"]
    with pytest.raises(ValueError, match="speaker embedding"):
        tiny_cfg(speaker_encoder=T.SpeakerEncoderConfig(mel_dim=8, enc_dim=10, enc_channels=(16, 16, 16, 16, 48), enc_res2net_scale=4))
    with pytest.raises(ValueError, match="codec embedding"):
        T.TalkerConfig(vocab_size=100)
    with pytest.raises(ValueError, match="same"):
        T.SpeakerEncoderConfig(enc_kernel_sizes=(4, 3, 3, 3, 1))
    assert T.SpeechDecoderConfig().upsample_rate == 1920 and tiny_decoder_cfg().upsample_rate == 12


def test_sampling_controls():
    logits = torch.zeros(1, 10)
    s = T.suppress_tail(logits, 4, eos=7)
    assert s[0, :6].eq(0).all() and s[0, 7] == 0 and s[0, [6, 8, 9]].lt(-1e8).all()
    l2 = torch.tensor([[2.0, -2.0, 1.0]])
    assert torch.allclose(T.repetition_penalty(l2, torch.tensor([[0, 1]]), 2.0), torch.tensor([[1.0, -4.0, 1.0]]))
    assert torch.equal(T.repetition_penalty(l2, None, 2.0), l2)
    with pytest.raises(ValueError, match="temperature"):
        T.apply_sampling(logits, 0.0, None, 1.0)
    peaked = torch.full((2, 10), -50.0)
    peaked[:, 3] = 50.0
    assert T.apply_sampling(peaked, 0.7, 3, 0.9).tolist() == [3, 3]


def test_frame_generation_and_stop_rules():
    cfg = tiny_cfg()
    m = T.init(cfg)
    text = torch.randint(0, 59, (2, 5))
    x = m.build_talker_inputs(text, speaker="vivian", language="english")
    assert x.shape == (2, 1 + 2 + 5, 24)
    assert torch.equal(x[:, 1], m.talker.embed_codec(torch.full((2, 1), 38))[:, 0]) and torch.equal(x[:, 2], m.talker.embed_codec(torch.full((2, 1), 39))[:, 0])
    with pytest.raises(ValueError, match="Unsupported speaker"):
        m.build_talker_inputs(text, speaker="bob")
    g = torch.Generator().manual_seed(0)
    codes, lengths = m.generate_from_text(text, max_frames=6, generator=g)
    assert codes.shape == (2, 6, 4) and len(lengths) == 2 and all(0 <= n <= 6 for n in lengths)
    for b, n in enumerate(lengths):
        assert n == 0 or int(codes[b, :n, 1:].max()) < 32                   # residual codebooks use the predictor's vocabulary
        assert bool((codes[b, min(n + 1, 6):] == 45).all())                 # padding after the end-of-sequence frame
    # forcing end-of-sequence: it is not allowed before min_new_tokens, then ends every row at that step
    m.talker.codec_head.zero_()
    m.talker.codec_head[40] = 0.0
    frames = []
    with torch.no_grad():
        big = torch.zeros(48)
        big[40] = 1.0
    orig = T.suppress_tail
    try:
        T.suppress_tail = lambda logits, n, eos: orig(logits, n, eos) + big * 1e4
        lengths = T.stream_codes(m.talker, x, lambda s, f: frames.append(f), max_frames=8, min_new_tokens=3)
    finally:
        T.suppress_tail = orig
    assert lengths == [3, 3] and len(frames) == 4 and all(int(f[0, 0]) != 40 for f in frames[:3]) and int(frames[3][0, 0]) == 40


def test_speaker_encoder_embedding():
    cfg = tiny_cfg()
    enc = T.init_speaker_encoder(cfg.speaker_encoder)
    mel = torch.randn(2, 30, 8)
    e = enc.forward(mel)
    assert e.shape == (2, 24) and torch.isfinite(e).all()
    e2 = enc.forward(torch.cat([mel, mel], 1))                              # pooled statistics: repeating the utterance barely moves the embedding
    assert torch.nn.functional.cosine_similarity(e, e2).min() > 0.9


def test_speech_decoder_is_causal_and_chunked_streaming_match():
    dc = tiny_decoder_cfg()
    dec = T.init_speech_decoder(dc)
    codes = torch.randint(0, 32, (1, 3, 14))
    wav = dec.decode(codes)
    assert wav.shape == (1, 1, 14 * 12) and wav.abs().max() <= 1.0
    codes2 = codes.clone()
    codes2[:, :, 9:] = (codes2[:, :, 9:] + 7) % 32
    wav2 = dec.decode(codes2)
    assert torch.allclose(wav[:, :, :9 * 12], wav2[:, :, :9 * 12], atol=1e-6) and not torch.allclose(wav[:, :, 9 * 12:], wav2[:, :, 9 * 12:], atol=1e-4)
    # with a left context at least as long as the receptive field (window 5 + conv taps) chunked decoding is exact
    chunked = dec.decode_chunked(codes, chunk_size=4, left_context=14)
    assert torch.allclose(chunked, wav, atol=1e-5)
    ds = T.DecodeStream(dec, 1, chunk_size=3, left_context=14)
    parts = [ds.push(codes[:, :, i:i + 2]) for i in range(0, 14, 2)] + [ds.flush()]
    assert torch.allclose(torch.cat(parts, 2), wav, atol=1e-5)


def test_synthesize_and_stream_end_to_end():
    m = T.init(tiny_cfg(), speech_decoder_cfg=tiny_decoder_cfg())
    text = torch.randint(0, 59, (1, 4))
    emb = m.extract_speaker_embedding(torch.randn(1, 20, 8))
    opt = T.SamplingOptions(suppress_tail=16)                             # codec ids >= 32 are control tokens in this tiny vocabulary
    wavs = m.synthesize(text, max_frames=5, opt=opt, generator=torch.Generator().manual_seed(1), speaker_embedding=emb)
    assert len(wavs) == 1 and wavs[0].numel() % 12 == 0 and wavs[0].numel() > 0
    chunks = []
    n = m.stream(text, chunks.append, max_frames=5, chunk_frames=2, opt=opt, generator=torch.Generator().manual_seed(1), speaker_embedding=emb)
    assert sum(c.numel() for c in chunks) == n * 12
