"""Qwen3-TTS file-level bridge: speaker mel, code-row text format, wav -> codes (short and streamed), codes -> wav, speaker embedding."""
import json
import math
import os

import pytest
import torch

from tyr_b200.io import media
from tyr_b200.io import safetensors as st
from tyr_b200.models import qwen3_tts as T
from tyr_b200.models import qwen3_tts_bridge as B
from tyr_b200.models import qwen3_tts_encoder as E


def test_slaney_bank_and_speaker_mel_shapes():
    bank = B.slaney_mel_filter_bank(513, 128, 24000, 0.0, 12000.0)
    assert bank.shape == (513, 128) and float(bank.min()) >= 0 and int((bank.sum(0) > 0).sum()) == 128
    assert B.slaney_mel_filter_bank(1, 4, 24000, 0, 1).abs().sum() == 0
    t = torch.arange(24000) / 24000.0
    wave = 0.5 * torch.sin(2 * math.pi * 440.0 * t)
    mel = B.compute_speaker_mel(wave, 24000, 128)
    frames = (24000 + 2 * 384 - 1024) // 256 + 1
    assert mel.shape == (1, frames, 128) and float(mel.min()) >= math.log(1e-5) - 1e-6
    peak = int(mel[0].mean(0).argmax())
    centre = B.slaney_mel_filter_bank(513, 128, 24000, 0.0, 12000.0)[:, peak].argmax() * (12000.0 / 512)
    assert abs(float(centre) - 440.0) < 60.0                       # the energy sits in the filter around 440 Hz
    with pytest.raises(ValueError, match="empty"):
        B.compute_speaker_mel(torch.zeros(0), 24000, 128)
    with pytest.raises(ValueError, match="must be > 0"):
        B.compute_speaker_mel(wave, 24000, 128, hop=0)


def test_code_rows_roundtrip():
    text = B.format_code_rows([1, 2, 3, 4, 5, 6, 7], 3)
    assert text == "1 2 3\n4 5 6\n" and B.parse_code_rows(text).tolist() == [[1, 2, 3], [4, 5, 6]]
    assert B.format_code_rows([], 3) == "" and B.format_code_rows([1], 0) == "" and B.parse_code_rows("").shape == (0, 0)
    with pytest.raises(ValueError, match="different lengths"):
        B.parse_code_rows("1 2\n3\n")


def small12():
    return E.Encoder12HzConfig(channels=(8, 16, 16, 32, 32), hidden=32, heads=4, layers=2, ffn=64, window=6, codebook_size=32, codebook_dim=8,
                               semantic_codebooks=1, acoustic_codebooks=3, input_sample_rate=4000)


def test_encode_wave_short_and_streamed_agree_on_covered_context(tmp_path):
    enc = E.init_encoder_12hz(small12())
    wave = torch.randn(4000 * 3)
    a, b = str(tmp_path / "a.txt"), str(tmp_path / "b.txt")
    rows, groups = B.encode_wave_12hz(enc, wave, a, chunk_seconds=10)
    assert (rows, groups) == (E.encoded_frames(wave.numel()), 4)
    rows_s, _ = B.encode_wave_12hz(enc, wave, b, chunk_seconds=1, left_context_seconds=12)       # 3 streamed chunks, context covers everything
    assert rows_s <= rows
    full, streamed = B.parse_code_rows(open(a).read()), B.parse_code_rows(open(b).read())
    assert streamed.shape[1] == 4 and torch.equal(streamed[:2], full[:2])                       # rows whose windows end inside the first chunk agree


def test_encode_audio_file_and_decode_to_wav(tmp_path, monkeypatch):
    enc = E.init_encoder_12hz(small12())
    tok = tmp_path / "model" / "speech_tokenizer"
    tok.mkdir(parents=True)
    st.save_file({k: v.contiguous() for k, v in enc.p.items()}, str(tok / "model.safetensors"))
    json.dump({"model_type": "qwen3_tts_tokenizer_12hz", "encoder_valid_num_quantizers": 4}, open(tok / "config.json", "w"))
    monkeypatch.setattr(E.Encoder12HzConfig, "from_json", staticmethod(lambda j: small12()))
    wav = str(tmp_path / "in.wav")
    media.save_wav(wav, 0.3 * torch.sin(torch.arange(8000) / 20.0), 4000)
    assert not B.is_tokenizer_25hz(str(tok)) and B.resolve_speech_tokenizer_dir(str(tmp_path / "model")) == str(tok)
    rows, groups = B.encode_audio_to_codes(str(tmp_path / "model"), wav, str(tmp_path / "out" / "codes.txt"))
    codes = B.parse_code_rows(open(tmp_path / "out" / "codes.txt").read())
    assert codes.shape == (rows, groups) == (E.encoded_frames(8000), 4)
    dec = T.init_speech_decoder(_tiny_decoder_cfg())
    n = B.decode_codes_to_wav(dec, str(tmp_path / "out" / "codes.txt"), str(tmp_path / "out" / "speech.wav"), num_code_groups=4)
    assert n == rows * dec.cfg.upsample_rate and os.path.getsize(tmp_path / "out" / "speech.wav") == 44 + 2 * n
    with pytest.raises(ValueError, match="expected 5"):
        B.decode_codes_to_wav(dec, str(tmp_path / "out" / "codes.txt"), str(tmp_path / "x.wav"), num_code_groups=5)


def _tiny_decoder_cfg():
    import dataclasses
    fields = {f.name for f in dataclasses.fields(T.SpeechDecoderConfig)}
    want = dict(codebook_size=32, codebook_dim=8, num_quantizers=4, num_semantic_quantizers=1, hidden_size=16, num_hidden_layers=1, num_attention_heads=2,
                num_key_value_heads=2, head_dim=8, intermediate_size=32, latent_dim=16, decoder_dim=16)
    return T.SpeechDecoderConfig(**{k: v for k, v in want.items() if k in fields})


def test_speaker_mel_files_and_embedding(tmp_path):
    wav = str(tmp_path / "ref.wav")
    media.save_wav(wav, 0.2 * torch.sin(torch.arange(24000) / 9.0), 24000)
    frames = B.prepare_speaker_mel(wav, str(tmp_path / "m" / "mel.safetensors"), str(tmp_path / "m" / "frames.txt"))
    mel = st.Source.open(str(tmp_path / "m" / "mel.safetensors")).load("mel")
    assert mel.shape == (1, frames, 128) and open(tmp_path / "m" / "frames.txt").read() == f"{frames}\n"
    import types
    spk = T.SpeakerEncoderConfig(mel_dim=16, enc_dim=32, enc_channels=(8, 8, 8, 8, 24), enc_res2net_scale=2, enc_attention_channels=4, enc_se_channels=4)
    enc = T.init_speaker_encoder(spk)
    model = types.SimpleNamespace(cfg=types.SimpleNamespace(speaker_encoder=spk, talker=types.SimpleNamespace(hidden_size=32)),
                                  extract_speaker_embedding=lambda mel: enc.forward(mel))
    emb = B.extract_speaker_embedding_from_audio(model, wav, str(tmp_path / "e" / "mel.safetensors"), " ")
    assert emb.shape == (1, 1, 32) and torch.isfinite(emb).all() and os.path.exists(tmp_path / "e" / "mel.safetensors")
    model.cfg.talker.hidden_size = 48
    with pytest.raises(ValueError, match="dim mismatch"):
        B.extract_speaker_embedding_from_audio(model, wav)
