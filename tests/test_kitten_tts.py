"""KittenTTS / Kokoro on a tiny random model: config rules, primitives, duration -> alignment, waveform length, loader."""
import math

import pytest
import torch

from tyr_b200.io import safetensors as st
from tyr_b200.models import kitten_tts as K


def tiny_cfg():
    return K.KittenTTSConfig(hidden_dim=16, max_conv_dim=16, max_dur=6, n_layer=2, n_token=20, style_dim=8, text_encoder_kernel_size=3, asr_res_dim=4,
                             plbert=K.AlbertConfig(num_hidden_layers=2, num_attention_heads=2, hidden_size=12, intermediate_size=24, max_position_embeddings=32, embedding_size=6),
                             generator=K.GeneratorConfig(resblock_kernel_sizes=(3, 5), upsample_rates=(3, 2), upsample_initial_channel=16,
                                                         resblock_dilation_sizes=((1, 2, 3), (1, 2, 3)), upsample_kernel_sizes=(5, 4), gen_istft_n_fft=8,
                                                         gen_istft_hop_size=2, harmonic_count=3))


def test_config_rules():
    g = K.GeneratorConfig()
    assert g.total_upsample == 60 and g.source_upsample == 300 and g.freq_bins == 11 and g.stage_out_channels(1) == 128
    with pytest.raises(ValueError, match="odd kernels"):
        K.GeneratorConfig(resblock_kernel_sizes=(3, 6, 11))
    with pytest.raises(ValueError, match="even amount"):
        K.GeneratorConfig(upsample_kernel_sizes=(21, 12))
    with pytest.raises(ValueError, match="even hidden"):
        K.KittenTTSConfig(hidden_dim=511)


def test_primitives():
    v = torch.randn(4, 3, 5)
    w = K.fuse_weight_norm(torch.full((4, 1, 1), 2.0), v)
    assert torch.allclose(w.flatten(1).norm(dim=1), torch.full((4,), 2.0), atol=1e-5)
    x = torch.randn(1, 6, 50)
    n = K.instance_norm(x)
    assert n.mean(2).abs().max() < 1e-5 and (n.var(2, unbiased=False) - 1).abs().max() < 1e-3
    assert K.duration_to_frames([0.2, 2.6, 5.0], 1.0) == [1, 3, 5] and K.duration_to_frames([4.0], 2.0) == [2]
    a = K.build_alignment([2, 1, 3], "cpu")
    assert a.shape == (3, 6) and a.sum(1).tolist() == [2, 1, 3] and a.sum(0).eq(1).all()
    # the hand-rolled BiLSTM against torch.nn.LSTM with the same weights
    lstm = torch.nn.LSTM(5, 4, batch_first=True, bidirectional=True)
    d = {"l." + k: p.detach() for k, p in lstm.named_parameters()}
    seq = torch.randn(1, 9, 5)
    assert torch.allclose(K.bilstm(K.P(d, "l."), seq), lstm(seq)[0], atol=1e-5)


def test_synthesis_shapes_and_speed():
    cfg = tiny_cfg()
    m = K.init(cfg, seed=3)
    ids = torch.randint(0, 20, (1, 7))
    style = torch.randn(1, 16)
    out = m.synthesize(ids, style, generator=torch.Generator().manual_seed(0))
    assert len(out.pred_durations) == 7 and out.alignment_frames == sum(out.pred_durations)
    assert out.audio.numel() == out.alignment_frames * 2 * cfg.generator.source_upsample and torch.isfinite(out.audio).all()
    fast = m.synthesize(ids, style, speed=3.0, generator=torch.Generator().manual_seed(0))
    assert fast.alignment_frames <= out.alignment_frames
    assert m.synthesize(ids[:, :0], style).audio.numel() == 0
    assert K.select_style(torch.randn(10, 1, 16), 4).shape == (1, 16) and K.select_style(torch.randn(16), 4).shape == (1, 16)


def test_loader_fuses_weight_norm_and_checks_shapes(tmp_path):
    cfg = tiny_cfg()
    m = K.init(cfg, seed=1)
    sd = {k: v.contiguous() for k, v in m.params.items()}
    w = sd.pop("decoder.asr_res.0.weight")
    sd["decoder.asr_res.0.weight_v"] = (w * 3.0).contiguous()
    sd["decoder.asr_res.0.weight_g"] = w.flatten(1).norm(dim=1).reshape(-1, 1, 1).contiguous()
    path = str(tmp_path / "kitten.safetensors")
    st.save_file(sd, path)
    m2 = K.load(cfg, path)
    assert torch.allclose(m2.params["decoder.asr_res.0.weight"], w, atol=1e-5)
    ids, style = torch.randint(0, 20, (1, 5)), torch.randn(1, 16)
    a = m.synthesize(ids, style, generator=torch.Generator().manual_seed(2)).audio
    b = m2.synthesize(ids, style, generator=torch.Generator().manual_seed(2)).audio
    assert torch.allclose(a, b, rtol=1e-3, atol=1e-3)
    del sd["bert_encoder.bias"]
    st.save_file(sd, path)
    with pytest.raises(st.SafeTensorsError, match="missing bert_encoder.bias"):
        K.load(cfg, path)
