"""KittenTTS / Kokoro config.json parsing, vocabulary, raw checkpoint conversion and the pretrained bundle; TTS CLI dispatch."""
import json
import os

import pytest
import torch

from tyr_b200.io import safetensors as st
from tyr_b200.models import kitten_tts as K
from tyr_b200.models import kitten_tts_io as KIO


def tiny_json():
    return {"hidden_dim": 16, "max_conv_dim": 16, "max_dur": 6, "n_layer": 2, "n_token": 20, "style_dim": 8, "text_encoder_kernel_size": 3, "dim_in": 4,
            "plbert": {"num_hidden_layers": 2, "num_attention_heads": 2, "hidden_size": 12, "intermediate_size": 24, "max_position_embeddings": 32, "embedding_size": 6,
                       "hidden_act": "gelu_new"},
            "istftnet": {"resblock_kernel_sizes": [3, 5], "upsample_rates": [3, 2], "upsample_initial_channel": 16, "resblock_dilation_sizes": [[1, 2, 3], [1, 2, 3]],
                         "upsample_kernel_sizes": [5, 4], "gen_istft_n_fft": 8, "gen_istft_hop_size": 2, "harmonic_num": 3},
            "vocab": {"a": 1, "b": 2, " ": 3, "ʃ": 19}}


def test_config_and_vocab_parsing(tmp_path):
    cfg = KIO.config_from_json(tiny_json())
    assert (cfg.hidden_dim, cfg.asr_res_dim, cfg.plbert.hidden_size, cfg.generator.harmonic_count, cfg.generator.upsample_rates) == (16, 4, 12, 3, (3, 2))
    bad = tiny_json()
    bad["plbert"]["num_attention_heads"] = 5
    with pytest.raises(ValueError, match="divide hidden_size"):
        KIO.config_from_json(bad)
    bad = tiny_json()
    bad["plbert"]["hidden_act"] = "relu"
    with pytest.raises(ValueError, match="hidden_act"):
        KIO.config_from_json(bad)
    bad = tiny_json()
    bad["decoder_out_dim"] = 7
    with pytest.raises(ValueError, match="decoder_out_dim"):
        KIO.config_from_json(bad)
    p = str(tmp_path / "config.json")
    json.dump(tiny_json(), open(p, "w"))
    vocab = KIO.load_vocab(p, 20)
    assert vocab["ʃ"] == 19 and KIO.encode_phoneme_ids(vocab, "ab?ʃ") == [0, 1, 2, 19, 0]
    with pytest.raises(ValueError, match="outside the embedding table"):
        KIO.load_vocab(p, 19)
    j = tiny_json()
    j["vocab"]["ab"] = 4
    json.dump(j, open(p, "w"))
    with pytest.raises(ValueError, match="expected one character"):
        KIO.load_vocab(p, 20)
    assert [KIO.voice_index_of_phoneme_count(n) for n in (0, 1, 10, 999)] == [0, 0, 9, 509]


def test_raw_checkpoint_conversion_bundle_and_cli(tmp_path, capsys):
    cfg = KIO.config_from_json(tiny_json())
    model = K.init(cfg, seed=2)
    d = tmp_path / "kokoro"
    (d / "voices").mkdir(parents=True)
    json.dump(tiny_json(), open(d / "config.json", "w"))
    # a raw checkpoint: {module: state_dict} with DataParallel prefixes, and a .pt voicepack
    payload = {}
    for name, t in model.params.items():
        top, rest = name.split(".", 1)
        payload.setdefault(top, {})["module." + rest] = t
    torch.save(payload, str(d / "kokoro-v1_0.pth"))
    torch.save(torch.randn(510, 1, cfg.full_style_dim), str(d / "voices" / "af.pt"))
    bundle = KIO.load_from_pretrained(str(d))
    assert os.path.exists(d / "model.safetensors") and set(st.Source.open(str(d / "model.safetensors")).names()) == set(model.params)
    style = bundle.load_voice_style("af", 4)
    assert style.shape == (1, cfg.full_style_dim) and os.path.exists(d / "voices" / "af.safetensors")
    table = st.Source.open(str(d / "voices" / "af.safetensors")).load("voice")
    assert torch.equal(style[0], table[3, 0])
    out = bundle.synthesize_phonemes_to_file("ab a", "af", str(tmp_path / "o" / "x.wav"), 1.0, torch.Generator().manual_seed(0))
    assert out.audio.numel() > 0 and os.path.getsize(tmp_path / "o" / "x.wav") == 44 + 2 * out.audio.numel()
    bundle.synthesize_phonemes_to_file("ab", "af", str(tmp_path / "o" / "x.safetensors"))
    assert st.Source.open(str(tmp_path / "o" / "x.safetensors")).load("audio").dim() == 1
    with pytest.raises(FileNotFoundError, match="voicepack"):
        bundle.load_voice_style("nobody", 3)
    from tyr_b200.cli import run_tts
    assert run_tts.main(["kitten", str(d), "ab a", "af", str(tmp_path / "cli.wav"), "1.25"]) == 0
    text = capsys.readouterr().out
    assert "saved_audio=" in text and "pred_durations=" in text and os.path.exists(tmp_path / "cli.wav")
    assert run_tts.main(["kitten", str(d)]) == 1 and run_tts.main(["kitten", str(d), "a", "af", "x.wav", "fast"]) == 1 and run_tts.main([]) == 1
    empty = tmp_path / "empty"
    empty.mkdir()
    json.dump(tiny_json(), open(empty / "config.json", "w"))
    with pytest.raises(FileNotFoundError, match="raw .pth"):
        KIO.resolve_pretrained_dir(str(empty))
