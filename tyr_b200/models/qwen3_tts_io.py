"""Qwen3-TTS ``config.json`` parsing and checkpoint loading (talker, code predictor, ECAPA speaker encoder).

Contract: Tyr/Model/Qwen3TTS/ConfigIO.lean (field names, the checks on heads / head_dim / rope / special ids, plain-RoPE only)
and Tyr/Model/Qwen3TTS/Weights.lean (tensor names under ``talker.*`` and ``speaker_encoder.*``, identity projection when the code
predictor has the talker's width and the checkpoint omits ``small_to_mtp_projection``).
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Optional

import torch

from ..io import safetensors as st
from . import qwen as Q
from . import qwen3_tts as T


def _check_decoder_fields(j: dict, what: str):
    if j.get("hidden_act", "silu") != "silu":
        raise ValueError(f"Invalid Qwen3-TTS {what} config: hidden_act must be silu")
    if j.get("attention_bias", False) or j.get("use_sliding_window", False):
        raise ValueError(f"Invalid Qwen3-TTS {what} config: attention_bias and use_sliding_window must be false")
    scaling = j.get("rope_scaling")
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type"))
        if kind != "default":
            raise ValueError(f"unsupported 'rope_scaling' = {json.dumps(scaling)}; this model implements plain RoPE")


def _heads(j: dict, d, what: str):
    heads, kv = int(j.get("num_attention_heads", d.num_attention_heads)), int(j.get("num_key_value_heads", d.num_key_value_heads))
    if kv <= 0 or heads % kv:
        raise ValueError(f"Invalid Qwen3-TTS {what} config: num_key_value_heads={kv} must be positive and divide num_attention_heads={heads}")
    head_dim = int(j.get("head_dim", 2 * d.half_head_dim))
    if head_dim <= 0 or head_dim % 2:
        raise ValueError(f"Invalid Qwen3-TTS {what} config: head_dim={head_dim} must be positive and even")
    theta, eps = float(j.get("rope_theta", d.rope_theta)), float(j.get("rms_norm_eps", d.rms_norm_eps))
    if theta <= 0:
        raise ValueError(f"Invalid Qwen3-TTS {what} config: rope_theta={theta} must be positive")
    if eps <= 0:
        raise ValueError(f"Invalid Qwen3-TTS {what} config: rms_norm_eps={eps} must be positive")
    return heads, kv, head_dim // 2, theta, eps


def code_predictor_config_from_json(j: dict) -> T.CodePredictorConfig:
    d = T.CodePredictorConfig()
    _check_decoder_fields(j, "code predictor")
    heads, kv, half, theta, eps = _heads(j, d, "code predictor")
    g = lambda k: int(j.get(k, getattr(d, k)))
    return T.CodePredictorConfig(g("vocab_size"), g("hidden_size"), g("intermediate_size"), g("num_hidden_layers"), heads, kv, half, eps, theta)


def _id_map(j: dict, key: str) -> Dict[str, int]:
    out = {}
    for name, v in (j.get(key) or {}).items():
        if isinstance(v, bool) or not isinstance(v, int) or v < 0:
            raise ValueError(f"invalid '{key}.{name}' = {json.dumps(v)}: expected a non-negative integer")
        out[name] = v
    return out


def talker_config_from_json(j: dict) -> T.TalkerConfig:
    d = T.TalkerConfig()
    _check_decoder_fields(j, "talker")
    cp = code_predictor_config_from_json(j["code_predictor_config"]) if isinstance(j.get("code_predictor_config"), dict) else d.code_predictor
    heads, kv, half, theta, eps = _heads(j, d, "talker")
    g = lambda k: int(j.get(k, getattr(d, k)))
    dialect = {}
    for name, v in (j.get("spk_is_dialect") or {}).items():
        if not isinstance(v, (str, bool)):
            raise ValueError(f"invalid 'spk_is_dialect.{name}' = {json.dumps(v)}: expected a string or boolean")
        dialect[name] = ("true" if v else "false") if isinstance(v, bool) else v
    return T.TalkerConfig(cp, g("vocab_size"), g("hidden_size"), g("intermediate_size"), g("num_hidden_layers"), heads, kv, half, eps, theta, g("num_code_groups"),
                          g("text_hidden_size"), g("text_vocab_size"), g("codec_eos_token_id"), g("codec_think_id"), g("codec_nothink_id"), g("codec_think_bos_id"),
                          g("codec_think_eos_id"), g("codec_pad_id"), g("codec_bos_id"), _id_map(j, "spk_id"), dialect, _id_map(j, "codec_language_id"))


def speaker_encoder_config_from_json(j: dict) -> T.SpeakerEncoderConfig:
    d = T.SpeakerEncoderConfig()
    g = lambda k: j.get(k, getattr(d, k))
    if int(g("sample_rate")) <= 0:
        raise ValueError("Invalid speaker encoder config: sample_rate must be positive")
    return T.SpeakerEncoderConfig(int(g("mel_dim")), int(g("enc_dim")), tuple(g("enc_channels")), tuple(g("enc_kernel_sizes")), tuple(g("enc_dilations")),
                                  int(g("enc_attention_channels")), int(g("enc_res2net_scale")), int(g("enc_se_channels")), int(g("sample_rate")))


def config_from_json(root: dict) -> T.Qwen3TTSConfig:
    d = T.Qwen3TTSConfig()
    talker = talker_config_from_json(root["talker_config"]) if isinstance(root.get("talker_config"), dict) else d.talker
    spk = speaker_encoder_config_from_json(root["speaker_encoder_config"]) if isinstance(root.get("speaker_encoder_config"), dict) else d.speaker_encoder
    g = lambda k: int(root.get(k, getattr(d, k)))
    return T.Qwen3TTSConfig(talker, spk, root.get("tts_model_type", d.tts_model_type), g("im_start_token_id"), g("im_end_token_id"), g("tts_pad_token_id"),
                            g("tts_bos_token_id"), g("tts_eos_token_id"))


def load_config(model_dir: str) -> T.Qwen3TTSConfig:
    with open(os.path.join(model_dir, "config.json"), encoding="utf-8") as f:
        return config_from_json(json.load(f))


# ---- weights ---------------------------------------------------------------------------------------------------------------
def _tensor(src, name: str, shape, device, dtype, required=True) -> Optional[torch.Tensor]:
    if src.find(name) is None:
        if required:
            raise st.SafeTensorsError(f"Qwen3TTS tensor '{name}': missing")
        return None
    t = src.load(name)
    if tuple(t.shape) != tuple(shape):
        raise st.SafeTensorsError(f"Qwen3TTS tensor '{name}': expected shape {list(shape)}, got {list(t.shape)}")
    return t.to(device=device, dtype=dtype)


def _prefix_map(model_prefix: str, embedding: str) -> Callable[[str], str]:
    def m(name: str) -> str:
        if name == "model.embed_tokens.weight":
            return embedding
        return model_prefix + name[len("model."):] if name.startswith("model.") else name
    return m


def load_talker(src, cfg: T.TalkerConfig, device, dtype) -> T.Talker:
    cp, n = cfg.code_predictor, cfg.num_code_groups - 1
    t = lambda name, *shape, **kw: _tensor(src, name, shape, device, dtype, **kw)
    codec = t("talker.model.codec_embedding.weight", cfg.vocab_size, cfg.hidden_size)
    model = Q.load_qwen3_model(cfg.qwen(), src, device, dtype, name_map=_prefix_map("talker.model.", "talker.model.codec_embedding.weight"))
    pw = t("talker.code_predictor.small_to_mtp_projection.weight", cp.hidden_size, cfg.hidden_size, required=False)
    pb = t("talker.code_predictor.small_to_mtp_projection.bias", cp.hidden_size, required=False)
    if (pw is None) != (pb is None):
        raise st.SafeTensorsError("Incomplete talker.code_predictor.small_to_mtp_projection: weight and bias must both be present or both absent.")
    if pw is None:
        if cp.hidden_size != cfg.hidden_size:
            raise st.SafeTensorsError("Missing talker.code_predictor.small_to_mtp_projection.* and hidden sizes differ; cannot build projection.")
        pw, pb = torch.eye(cp.hidden_size, device=device, dtype=dtype), torch.zeros(cp.hidden_size, device=device, dtype=dtype)
    predictor = T.CodePredictor(
        [t(f"talker.code_predictor.model.codec_embedding.{i}.weight", cp.vocab_size, cfg.hidden_size) for i in range(n)], pw, pb,
        Q.load_qwen3_model(cp.qwen(), src, device, dtype, name_map=_prefix_map("talker.code_predictor.model.", "talker.code_predictor.model.codec_embedding.0.weight")),
        [t(f"talker.code_predictor.lm_head.{i}.weight", cp.vocab_size, cp.hidden_size) for i in range(n)])
    return T.Talker(cfg, codec, t("talker.model.text_embedding.weight", cfg.text_vocab_size, cfg.text_hidden_size),
                    t("talker.text_projection.linear_fc1.weight", cfg.text_hidden_size, cfg.text_hidden_size), t("talker.text_projection.linear_fc1.bias", cfg.text_hidden_size),
                    t("talker.text_projection.linear_fc2.weight", cfg.hidden_size, cfg.text_hidden_size), t("talker.text_projection.linear_fc2.bias", cfg.hidden_size),
                    model, predictor, t("talker.codec_head.weight", cfg.vocab_size, cfg.hidden_size))


def load_speaker_encoder(src, cfg: T.SpeakerEncoderConfig, device, dtype) -> T.SpeakerEncoder:
    c, k, d = cfg.enc_channels, cfg.enc_kernel_sizes, cfg.enc_dilations
    part = c[0] // cfg.enc_res2net_scale

    def conv(name, o, i, kk):
        return _tensor(src, name + ".weight", (o, i, kk), device, dtype), _tensor(src, name + ".bias", (o,), device, dtype)
    blocks = []
    for b in (1, 2, 3):
        p = f"speaker_encoder.blocks.{b}"
        blocks.append(T.SERes2Block(conv(p + ".tdnn1.conv", c[b], c[b - 1], 1),
                                    [conv(f"{p}.res2net_block.blocks.{i}.conv", part, part, k[b]) for i in range(cfg.enc_res2net_scale - 1)],
                                    conv(p + ".tdnn2.conv", c[b], c[b], 1), conv(p + ".se_block.conv1", cfg.enc_se_channels, c[b], 1),
                                    conv(p + ".se_block.conv2", c[b], cfg.enc_se_channels, 1), d[b]))
    return T.SpeakerEncoder(cfg, conv("speaker_encoder.blocks.0.conv", c[0], cfg.mel_dim, k[0]), blocks, conv("speaker_encoder.mfa.conv", c[4], c[1] + c[2] + c[3], k[4]),
                            conv("speaker_encoder.asp.tdnn.conv", cfg.enc_attention_channels, 3 * c[4], 1), conv("speaker_encoder.asp.conv", c[4], cfg.enc_attention_channels, 1),
                            conv("speaker_encoder.fc", cfg.enc_dim, 2 * c[4], 1))


def load_sharded(model_dir: str, cfg: Optional[T.Qwen3TTSConfig] = None, device="cpu", dtype: Optional[torch.dtype] = None, log=None,
                 with_speech_decoder: bool = True) -> T.Qwen3TTS:
    """Talker (+ speaker encoder for ``base`` models, + the 12 Hz speech decoder when ``speech_tokenizer/`` is present).  Every part
    keeps its checkpoint dtype unless ``dtype`` is given."""
    info = log or (lambda s: None)
    cfg = cfg or load_config(model_dir)
    info(f"Loading Qwen3TTS weights from {model_dir}...")
    src = st.Source.open(model_dir)
    anchor = src.load("talker.model.codec_embedding.weight")
    if not anchor.dtype.is_floating_point:
        raise st.SafeTensorsError("talker.model.codec_embedding.weight is not a floating tensor")
    talker = load_talker(src, cfg.talker, device, dtype or anchor.dtype)
    enc = None
    if cfg.tts_model_type == "base":
        first = src.load("speaker_encoder.blocks.0.conv.weight")
        enc = load_speaker_encoder(src, cfg.speaker_encoder, device, dtype or first.dtype)
    dec = None
    tok_dir = os.path.join(model_dir, "speech_tokenizer")
    if with_speech_decoder and os.path.exists(os.path.join(tok_dir, "model.safetensors")):
        dec = T.load_speech_decoder(tok_dir, device=device, dtype=dtype or torch.float32)
    info("Loaded Qwen3TTS weights (real checkpoint tensors).")
    return T.Qwen3TTS(cfg, talker, enc, dec)


def state_dict(m: T.Qwen3TTS) -> Dict[str, torch.Tensor]:
    """Checkpoint-named tensors of the talker and speaker encoder (the inverse of :func:`load_sharded`)."""
    t, out = m.talker, {}
    out["talker.model.codec_embedding.weight"], out["talker.model.text_embedding.weight"] = t.codec_embedding, t.text_embedding
    out["talker.text_projection.linear_fc1.weight"], out["talker.text_projection.linear_fc1.bias"] = t.text_fc1, t.text_fc1_b
    out["talker.text_projection.linear_fc2.weight"], out["talker.text_projection.linear_fc2.bias"] = t.text_fc2, t.text_fc2_b
    out["talker.codec_head.weight"] = t.codec_head

    def stack(prefix, model):
        out[prefix + "norm.weight"] = model.norm
        for i, l in enumerate(model.layers):
            p = f"{prefix}layers.{i}."
            out[p + "input_layernorm.weight"], out[p + "post_attention_layernorm.weight"] = l.input_layernorm, l.post_attention_layernorm
            for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
                out[p + f"self_attn.{n}.weight"] = getattr(l.self_attn, n)
            for n in ("q_norm", "k_norm"):
                if getattr(l.self_attn, n) is not None:
                    out[p + f"self_attn.{n}.weight"] = getattr(l.self_attn, n)
            for n in ("gate_proj", "up_proj", "down_proj"):
                out[p + f"mlp.{n}.weight"] = getattr(l.mlp, n)
    stack("talker.model.", t.model)
    cp = t.code_predictor
    stack("talker.code_predictor.model.", cp.model)
    for i, (e, h) in enumerate(zip(cp.input_embeddings, cp.lm_heads)):
        out[f"talker.code_predictor.model.codec_embedding.{i}.weight"], out[f"talker.code_predictor.lm_head.{i}.weight"] = e, h
    out["talker.code_predictor.small_to_mtp_projection.weight"], out["talker.code_predictor.small_to_mtp_projection.bias"] = cp.input_projection, cp.input_projection_bias
    s = m.speaker_encoder
    if s is not None:
        def conv(name, wb):
            out[name + ".weight"], out[name + ".bias"] = wb
        conv("speaker_encoder.blocks.0.conv", s.tdnn0)
        for b, blk in enumerate(s.blocks, 1):
            p = f"speaker_encoder.blocks.{b}"
            conv(p + ".tdnn1.conv", blk.tdnn1), conv(p + ".tdnn2.conv", blk.tdnn2), conv(p + ".se_block.conv1", blk.se1), conv(p + ".se_block.conv2", blk.se2)
            for i, wb in enumerate(blk.res2):
                conv(f"{p}.res2net_block.blocks.{i}.conv", wb)
        conv("speaker_encoder.mfa.conv", s.mfa), conv("speaker_encoder.asp.tdnn.conv", s.asp_tdnn), conv("speaker_encoder.asp.conv", s.asp_conv), conv("speaker_encoder.fc", s.fc)
    return out
