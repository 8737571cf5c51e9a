"""Qwen3-TTS speech-tokenizer encoders: frame arithmetic, causal padding, RVQ, streaming equivalence, 25 Hz chunking, loaders."""
import json
import os

import pytest
import torch

from tyr_b200.io import safetensors as st
from tyr_b200.models import qwen3_tts_encoder as E


def small12(**kw):
    return E.Encoder12HzConfig(channels=(8, 16, 16, 32, 32), hidden=32, heads=4, layers=2, ffn=64, window=6, codebook_size=32, codebook_dim=8,
                               semantic_codebooks=1, acoustic_codebooks=3, **kw)


def test_frame_arithmetic_and_causal_conv():
    assert E.encoded_frames(1920) == 1 and E.encoded_frames(1921) == 2 and E.frames_before_final_downsample(960) == 1 and E.encoded_frames(24000) == 13
    x, w = torch.randn(1, 2, 11), torch.randn(3, 2, 4)
    y = E.causal_conv(x, w, None, stride=2)
    assert y.shape == (1, 3, 6)
    x2 = x.clone()
    x2[..., 7:] += 1.0                                    # later samples must not change earlier frames
    assert torch.allclose(E.causal_conv(x2, w, None, stride=2)[..., :3], y[..., :3])
    rep = E.causal_conv(torch.full((1, 2, 5), 3.0), torch.ones(1, 2, 4) / 8, None, stride=2, replicate=True)
    assert torch.allclose(rep, torch.full_like(rep, 3.0))   # edge replication keeps a constant signal constant
    with pytest.raises(ValueError, match="no acoustic"):
        E.Encoder12HzConfig.from_json({"encoder_valid_num_quantizers": 1})
    assert E.Encoder12HzConfig.from_json({"encoder_valid_num_quantizers": 8}).acoustic_codebooks == 7


def test_encode_12hz_shapes_rvq_and_prefix_causality():
    m = E.init_encoder_12hz(small12())
    wave = torch.randn(2, 1, 5000)
    codes = m.encode(wave)
    assert codes.shape == (2, 4, E.encoded_frames(5000)) and codes.dtype == torch.long and int(codes.max()) < 32 and m.num_code_groups == 4
    # the stack is causal: a longer input leaves the codes of fully covered frames unchanged
    longer = torch.cat([wave, torch.randn(2, 1, 3000)], 2)
    full = E.encoded_frames(5000) - 1
    assert torch.equal(m.encode(longer)[:, :, :full], codes[:, :, :full])
    # residual quantisation: the second acoustic index is the nearest code of what the first left
    e0 = m.codebook("acoustic", 0)
    assert e0.shape == (32, 8) and torch.isfinite(e0).all()
    assert torch.equal(E.nearest_code(e0[[3, 7]].float() + 1e-4, e0.float()), torch.tensor([3, 7]))
    fm = m.encode_mono_frame_major(wave[0, 0])
    assert fm.shape == (E.encoded_frames(5000), 4) and torch.equal(fm.t(), codes[0])
    with pytest.raises(ValueError, match="at least one sample"):
        m.encode(torch.zeros(1, 1, 0))


def test_streaming_matches_offline_when_context_covers_the_window():
    m = E.init_encoder_12hz(small12())
    wave = torch.randn(1920 * 6).tolist()
    offline = m.encode_mono_frame_major(torch.tensor(wave)).reshape(-1).tolist()
    state, got = E.EncodeStreamState(left_context_samples=1920 * 6), []
    for s in range(0, len(wave), 1920 * 2):
        state, vals = E.push_encode_stream(m, state, wave[s:s + 1920 * 2])
        got += vals
    assert got == offline and state.offset_samples == len(wave)
    state2, vals = E.push_encode_stream(m, state, [])
    assert vals == [] and state2 is state
    # a short context re-encodes with the rotary offset of the retained history
    short = E.EncodeStreamState(left_context_samples=1920)
    for s in range(0, len(wave), 1920 * 2):
        short, vals = E.push_encode_stream(m, short, wave[s:s + 1920 * 2])
        assert len(vals) == 2 * 4
    assert len(short.history) == 1920 and short.offset_samples == len(wave)


def test_encoder_12hz_loader_roundtrip(tmp_path):
    cfg = small12()
    m = E.init_encoder_12hz(cfg, seed=3)
    d = str(tmp_path)
    st.save_file({k: v.contiguous() for k, v in m.p.items()}, os.path.join(d, "model.safetensors"))
    json.dump({"encoder_valid_num_quantizers": 4}, open(os.path.join(d, "config.json"), "w"))
    import unittest.mock as um
    with um.patch.object(E, "Encoder12HzConfig", wraps=E.Encoder12HzConfig) as C:
        C.from_json = lambda j: small12()
        loaded = E.load_encoder_12hz(d)
        wave = torch.randn(1, 1, 4000)
        assert torch.equal(loaded.encode(wave), m.encode(wave))
        with pytest.raises(ValueError, match="Fixed 16-group"):
            E.load_encoder_12hz(d, flexible=False)


def test_encoder_25hz_chunks_config_and_loader(tmp_path):
    cfg = E.Encoder25HzConfig(n_mels=16, n_ctx=64, n_state=32, n_head=4, n_blocks=2, codebook_size=50, chunk_mel_frames=40)
    m = E.init_encoder_25hz(cfg)
    ids = m.encode_mel_chunk(torch.randn(16, 37))
    assert ids.shape == (((37 + 1) // 2) // 2,) and int(ids.max()) < 50
    assert m.encode_mel_chunk(torch.randn(16, 1)).numel() == 0
    with pytest.raises(ValueError, match="learned positions"):
        m.encode_mel_chunk(torch.randn(16, 200))
    groups, flat = m.encode_wave_to_codes(torch.randn(24000))
    frames = 24000 // 160
    want = sum(((min(40, frames - s) + 1) // 2) // 2 for s in range(0, frames, 40) if min(40, frames - s) >= 2)
    assert groups == 1 and len(flat) == want
    with pytest.raises(ValueError, match="empty"):
        m.encode_wave_to_codes(torch.zeros(0))
    with pytest.raises(ValueError, match="model_type"):
        E.Encoder25HzConfig.from_json({"model_type": "other"})
    with pytest.raises(ValueError, match="n_head"):
        E.Encoder25HzConfig.from_json({"model_type": "qwen3_tts_tokenizer_25hz", "encoder_config": {"n_head": 8}})
    assert E.Encoder25HzConfig.from_json({"model_type": "qwen3_tts_tokenizer_25hz", "input_sample_rate": 16000}).input_sample_rate == 16000
    d = str(tmp_path)
    tensors = {k: v.contiguous() for k, v in m.p.items() if not k.endswith("blocks.0.attn.key.bias")}
    st.save_file(tensors, os.path.join(d, "model.safetensors"))
    json.dump({"model_type": "qwen3_tts_tokenizer_25hz"}, open(os.path.join(d, "config.json"), "w"))
    import unittest.mock as um
    with um.patch.object(E.Encoder25HzConfig, "from_json", staticmethod(lambda j: cfg)):
        loaded = E.load_encoder_25hz(d)
    mel = torch.randn(16, 30)
    assert torch.equal(loaded.encode_mel_chunk(mel), m.encode_mel_chunk(mel))
