"""Qwen3-TTS config.json parsing and checkpoint round trip (talker, code predictor, speaker encoder)."""
import json
import os

import pytest
import torch

from tyr_b200.io import safetensors as st
from tyr_b200.models import qwen3_tts as T
from tyr_b200.models import qwen3_tts_io as IO


def tiny_json(**over):
    j = {"tts_model_type": "base", "im_start_token_id": 10, "im_end_token_id": 11, "tts_pad_token_id": 12, "tts_bos_token_id": 13, "tts_eos_token_id": 14,
         "talker_config": {"vocab_size": 96, "hidden_size": 32, "intermediate_size": 48, "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2,
                           "head_dim": 8, "num_code_groups": 3, "text_hidden_size": 24, "text_vocab_size": 64, "codec_eos_token_id": 70, "codec_think_id": 71,
                           "codec_nothink_id": 72, "codec_think_bos_id": 73, "codec_think_eos_id": 74, "codec_pad_id": 75, "codec_bos_id": 76,
                           "spk_id": {"vivian": 80}, "spk_is_dialect": {"vivian": False}, "codec_language_id": {"english": 81},
                           "code_predictor_config": {"vocab_size": 40, "hidden_size": 16, "intermediate_size": 24, "num_hidden_layers": 1, "num_attention_heads": 2,
                                                     "num_key_value_heads": 1, "head_dim": 8}},
         "speaker_encoder_config": {"mel_dim": 16, "enc_dim": 32, "enc_channels": [8, 8, 8, 8, 24], "enc_res2net_scale": 2, "enc_attention_channels": 4, "enc_se_channels": 4}}
    j.update(over)
    return j


def test_config_parsing_and_rejections():
    cfg = IO.config_from_json(tiny_json())
    t = cfg.talker
    assert (t.hidden_size, t.half_head_dim, t.num_code_groups, t.code_predictor.hidden_size, t.code_predictor.half_head_dim) == (32, 4, 3, 16, 4)
    assert t.spk_id == {"vivian": 80} and t.spk_is_dialect == {"vivian": "false"} and cfg.speaker_encoder.enc_channels == (8, 8, 8, 8, 24)
    assert cfg.supported_speakers() == ["vivian"] and cfg.supported_languages() == ["auto", "english"]
    bad = tiny_json()
    bad["talker_config"]["rope_scaling"] = {"rope_type": "yarn", "factor": 2}
    with pytest.raises(ValueError, match="plain RoPE"):
        IO.config_from_json(bad)
    bad = tiny_json()
    bad["talker_config"]["num_key_value_heads"] = 3
    with pytest.raises(ValueError, match="must be positive and divide"):
        IO.config_from_json(bad)
    bad = tiny_json()
    bad["talker_config"]["code_predictor_config"]["head_dim"] = 7
    with pytest.raises(ValueError, match="positive and even"):
        IO.config_from_json(bad)
    bad = tiny_json()
    bad["talker_config"]["spk_id"] = {"x": -1}
    with pytest.raises(ValueError, match="non-negative integer"):
        IO.config_from_json(bad)
    bad = tiny_json()
    bad["speaker_encoder_config"]["enc_dim"] = 48
    with pytest.raises(ValueError, match="speaker embedding"):
        IO.config_from_json(bad)
    assert IO.config_from_json(tiny_json(tts_model_type="custom_voice")).tts_model_type == "custom_voice"


def test_checkpoint_roundtrip_and_identity_projection(tmp_path):
    cfg = IO.config_from_json(tiny_json())
    m = T.init(cfg, seed=4)
    d = str(tmp_path)
    json.dump(tiny_json(), open(os.path.join(d, "config.json"), "w"))
    st.save_file({k: v.contiguous() for k, v in IO.state_dict(m).items()}, os.path.join(d, "model.safetensors"))
    logs = []
    loaded = IO.load_sharded(d, log=logs.append)
    assert loaded.speaker_encoder is not None and loaded.speech_decoder is None and any("real checkpoint tensors" in l for l in logs)
    ids = torch.tensor([[3, 5, 7, 9]])
    g1, g2 = torch.Generator().manual_seed(1), torch.Generator().manual_seed(1)
    a, la = m.generate_from_text(ids, max_frames=4, generator=g1, speaker="vivian")
    b, lb = loaded.generate_from_text(ids, max_frames=4, generator=g2, speaker="vivian")
    assert torch.equal(a, b) and la == lb
    mel = torch.randn(1, 30, 16)
    assert torch.allclose(loaded.extract_speaker_embedding(mel), m.extract_speaker_embedding(mel))
    # the projection may be omitted only when the predictor has the talker's width
    def variant(name, tensors):
        v = tmp_path / name
        v.mkdir()
        json.dump(tiny_json(), open(v / "config.json", "w"))
        st.save_file(tensors, str(v / "model.safetensors"))
        return str(v)
    tensors = {k: v.contiguous() for k, v in IO.state_dict(m).items() if "small_to_mtp_projection" not in k}
    with pytest.raises(st.SafeTensorsError, match="hidden sizes differ"):
        IO.load_sharded(variant("no_proj", tensors))
    tensors["talker.code_predictor.small_to_mtp_projection.weight"] = m.talker.code_predictor.input_projection.contiguous()
    with pytest.raises(st.SafeTensorsError, match="both be present"):
        IO.load_sharded(variant("half_proj", tensors))
    tensors["talker.code_predictor.small_to_mtp_projection.bias"] = m.talker.code_predictor.input_projection_bias.contiguous()
    del tensors["talker.codec_head.weight"]
    with pytest.raises(st.SafeTensorsError, match="codec_head"):
        IO.load_sharded(variant("no_head", tensors))


def test_cli_text_to_codes_and_wav(tmp_path, capsys):
    """run_tts qwen3tts: token ids -> codes file -> wav through a tiny speech decoder stored next to the model."""
    from tyr_b200.cli import run_tts
    from tyr_b200.models import qwen3_tts_bridge as B
    cfg = IO.config_from_json(tiny_json())
    m = T.init(cfg, seed=1)
    d = tmp_path / "model"
    (d / "speech_tokenizer").mkdir(parents=True)
    json.dump(tiny_json(), open(d / "config.json", "w"))
    st.save_file({k: v.contiguous() for k, v in IO.state_dict(m).items()}, str(d / "model.safetensors"))
    ids = tmp_path / "ids.txt"
    ids.write_text("3 5 7 9 11")
    codes = tmp_path / "out" / "codes.txt"
    rc = run_tts.main(["qwen3tts", "--model-dir", str(d), "--token-ids-path", str(ids), "--speaker", "vivian", "--max-frames", "5", "--codes-path", str(codes),
                       "--skip-decode", "--device", "cpu", "--seed", "3"])
    assert rc == 0 and B.parse_code_rows(codes.read_text()).shape[1] == 3
    assert "saved_codes=" in capsys.readouterr().out
    with pytest.raises(SystemExit):
        run_tts.main(["qwen3tts", "--model-dir", str(d), "--encode-only"])
    with pytest.raises(SystemExit, match="no speech_tokenizer"):
        run_tts.main(["qwen3tts", "--model-dir", str(d), "--token-ids-path", str(ids), "--max-frames", "3", "--codes-path", str(codes), "--device", "cpu"])
    with pytest.raises(ValueError, match="Unsupported speaker"):
        run_tts.main(["qwen3tts", "--model-dir", str(d), "--token-ids-path", str(ids), "--speaker", "nobody", "--skip-decode", "--device", "cpu",
                      "--codes-path", str(codes)])
