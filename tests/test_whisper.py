"""Whisper: front end, cached vs uncached decoding, timestamp rules, fallback heuristics, loader, transcription loop."""
import math
import struct

import pytest
import torch

from tyr_b200.audio import frontend as fe
from tyr_b200.io import safetensors as st
from tyr_b200.models import whisper as W


def tiny():
    return W.WhisperConfig(num_mel_bins=16, vocab_size=60, d_model=32, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=64,
                           decoder_layers=2, decoder_attention_heads=4, decoder_ffn_dim=64, max_source_positions=1500,
                           max_target_positions=40, eos_token_id=1, decoder_start_token_id=2)


def test_frontend_shapes_wav_roundtrip_and_filters(tmp_path):
    fb = fe.mel_filter_bank(80)
    assert fb.shape == (80, 201) and (fb >= 0).all() and (fb.sum(1) > 0).all()
    assert abs(float(fe.mel_to_hz(fe.hz_to_mel(440.0))) - 440.0) < 1e-6 and abs(float(fe.mel_to_hz(fe.hz_to_mel(4000.0))) - 4000.0) < 1e-6
    t = torch.arange(16000) / 16000.0
    wave = 0.5 * torch.sin(2 * math.pi * 1000.0 * t)
    feats = fe.log_mel_spectrogram(wave, 80, 3000)
    assert feats.shape == (80, 3000) and feats.max() <= 2.0 and float(feats[:, 2000:].max()) == float(feats.min())
    peak = feats[:, 50].argmax().item()
    centre = fe.mel_to_hz(torch.linspace(float(fe.hz_to_mel(0.0)), float(fe.hz_to_mel(8000.0)), 82))[peak + 1]
    assert abs(float(centre) - 1000.0) < 120.0
    p = str(tmp_path / "a.wav")
    pcm = (wave[:800] * 32767).to(torch.int16)
    hdr = b"RIFF" + struct.pack("<I", 36 + 1600) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 1, 1, 8000, 16000, 2, 16) + b"data" + struct.pack("<I", 1600)
    open(p, "wb").write(hdr + pcm.numpy().tobytes())
    x, rate = fe.load_mono_pcm16_wav(p)
    assert rate == 8000 and x.numel() == 800 and torch.allclose(x, pcm.float() / 32768)
    assert fe.resample_linear(x, 8000, 16000).numel() == 1600
    with pytest.raises(ValueError, match="RIFF"):
        open(p, "wb").write(b"nope" * 10); fe.load_mono_pcm16_wav(p)


def test_config_validation():
    assert W.WhisperConfig.conv2_output_seq(3000) == 1500
    with pytest.raises(ValueError, match="must divide d_model"):
        W.WhisperConfig(d_model=100, encoder_attention_heads=6)
    with pytest.raises(ValueError, match="unsupported activation"):
        W.WhisperConfig(activation_function="swish")


def test_cached_decoding_matches_full_and_loader_roundtrip(tmp_path):
    m = W.init(tiny())
    feats = torch.randn(1, 16, 200)
    enc = W.encode(m, feats)
    assert enc.shape == (1, 100, 32)
    toks = torch.randint(3, 60, (1, 9))
    full = W.decode(m, toks, enc)
    s = W.DecodeSession(m, enc)
    assert torch.allclose(s.step(toks[:, :4]), full[:, 3].float(), atol=1e-4)
    f = s.fork()
    for t in range(4, 9):
        assert torch.allclose(s.step(toks[:, t:t + 1]), full[:, t].float(), atol=1e-4)
    assert f.pos == 4 and torch.allclose(f.step(toks[:, 4:5]), full[:, 4].float(), atol=1e-4)
    d = tmp_path / "w"
    d.mkdir()
    st.save_file({k: v.contiguous() for k, v in W.state_dict(m).items()}, str(d / "model.safetensors"))
    m2 = W.load_sharded(str(d), tiny())
    assert torch.equal(W.decode(m2, toks, W.encode(m2, feats)), full) and m2.proj_out is m2.embed_tokens


def test_timestamp_rules_and_heuristics():
    rules = W.DecodeTokenRules(sot=2, eot=1, no_timestamps=5, timestamp_begin=40)
    lg = torch.zeros(60)
    first = W.apply_timestamp_rules(lg, [], rules, max_initial_ts=10)
    assert torch.isinf(first[:40]).all() and torch.isfinite(first[40:51]).all() and torch.isinf(first[51:]).all()
    opened = W.apply_timestamp_rules(lg, [40, 7, 8, 45], rules)           # text then a timestamp: must close with a timestamp >= 45
    assert torch.isinf(opened[:1]).all() and torch.isinf(opened[40:45]).all() and torch.isfinite(opened[45])
    closed = W.apply_timestamp_rules(torch.cat([torch.full((40,), 5.0), torch.zeros(20)]), [40, 7, 45, 45], rules)
    assert torch.isinf(closed[40:]).all() and torch.isfinite(closed[7])
    assert W.has_repetition_loop([1, 2] * 4) and W.has_repetition_loop([9] * 12) and not W.has_repetition_loop(list(range(20)))
    assert W.compression_ratio([7] * 200) > 2.4 > W.compression_ratio(list(range(100, 140)))
    assert W.WhisperDecodeOptions(no_fallback=False).temperatures() == [0.0, 0.2, 0.4, 0.6, 0.8, 1.0]
    assert W.token_overlap_length([1, 2, 3, 4], [3, 4, 5]) == 2 and W.append_with_token_stitch([1, 2, 3], [2, 3, 9]) == [1, 2, 3, 9]
    assert len(W.split_waveform_with_overlap(torch.zeros(100), 40, 10)) == 3
    c = W.DecodeCandidate([7] * 30, -2.0, 0.9, 0.0, 3.0)
    assert c.needs_fallback(W.WhisperDecodeOptions()) and c.is_no_speech(W.WhisperDecodeOptions())


def test_transcription_loop_greedy_and_beam():
    cfg = tiny()
    m = W.init(cfg, seed=3)
    rules = W.DecodeTokenRules(sot=2, eot=1, suppress=(0,))
    b = W.WhisperBundle(m, rules)
    wave = torch.randn(16000 * 2) * 0.1
    out = W.transcribe_waveform_16k(b, wave, W.WhisperDecodeOptions(max_new_tokens=6))
    assert 0 < len(out.tokens) <= 6 and all(t not in (0, 2) for t in out.tokens) and out.text
    enc = W.encode(m, fe.log_mel_spectrogram(wave, 16, 3000)[None])
    g = W.decode_at_temperature(m, enc, [2], rules, W.WhisperDecodeOptions(max_new_tokens=5), 0.0, False)
    bm = W.decode_at_temperature(m, enc, [2], rules, W.WhisperDecodeOptions(max_new_tokens=5, beam_size=3), 0.0, False)
    assert bm.avg_logprob >= g.avg_logprob - 1e-4
    s = W.decode_at_temperature(m, enc, [2], rules, W.WhisperDecodeOptions(max_new_tokens=5, top_k=5), 0.8, False, torch.Generator().manual_seed(0))
    assert len(s.tokens) <= 5
