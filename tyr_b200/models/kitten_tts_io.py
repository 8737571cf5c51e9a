"""KittenTTS / Kokoro: ``config.json`` parsing, phoneme vocabulary, checkpoint / voicepack conversion and the pretrained bundle
(phonemes + voice -> audio file).

Contract: Tyr/Model/KittenTTS/ConfigIO.lean (field names and checks, vocabulary of single-character keys below ``n_token``) and
Tyr/Model/KittenTTS/Pretrained.lean (raw ``.pth`` / ``.pt`` files converted once to safetensors, voice lookup under ``voices/``,
style row ``min(509, phoneme count - 1)``, ids ``0, ..., 0``).  The reference converts with an external Python script
(scripts/kokoro_to_safetensors.py); here the conversion runs in-process.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..io import hub, media
from ..io import safetensors as st
from . import kitten_tts as K

DEFAULT_REPO_ID = "hexgrad/Kokoro-82M"


def albert_config_from_json(j: dict) -> K.AlbertConfig:
    d = K.AlbertConfig()
    g = lambda k: j.get(k, getattr(d, k))
    layers, groups = int(g("num_hidden_layers")), int(j.get("num_hidden_groups", 1))
    if groups <= 0 or layers % groups:
        raise ValueError(f"Invalid KittenTTS plbert config: num_hidden_groups={groups} must be positive and divide num_hidden_layers={layers}")
    heads, hidden = int(g("num_attention_heads")), int(g("hidden_size"))
    if heads <= 0 or hidden % heads:
        raise ValueError(f"Invalid KittenTTS plbert config: num_attention_heads={heads} must be positive and divide hidden_size={hidden}")
    eps, types = float(g("layer_norm_eps")), int(g("type_vocab_size"))
    if eps <= 0:
        raise ValueError(f"Invalid KittenTTS plbert config: layer_norm_eps={eps} must be positive")
    if types <= 0:
        raise ValueError(f"Invalid KittenTTS plbert config: type_vocab_size={types} must hold token type 0")
    if j.get("hidden_act", "gelu_new") not in ("gelu_new", "gelu_pytorch_tanh"):
        raise ValueError(f"Invalid KittenTTS plbert config: hidden_act={j.get('hidden_act')!r} must be gelu_new or gelu_pytorch_tanh")
    if groups != 1 or int(j.get("inner_group_num", 1)) != 1:
        raise ValueError("Invalid KittenTTS plbert config: this implementation shares one ALBERT layer group (num_hidden_groups = inner_group_num = 1)")
    return K.AlbertConfig(layers, heads, hidden, int(g("intermediate_size")), int(g("max_position_embeddings")), int(g("embedding_size")), types, eps)


def generator_config_from_json(j: dict) -> K.GeneratorConfig:
    d = K.GeneratorConfig()
    g = lambda k: j.get(k, getattr(d, k))
    return K.GeneratorConfig(tuple(g("resblock_kernel_sizes")), tuple(g("upsample_rates")), int(g("upsample_initial_channel")),
                             tuple(tuple(x) for x in g("resblock_dilation_sizes")), tuple(g("upsample_kernel_sizes")), int(g("gen_istft_n_fft")),
                             int(g("gen_istft_hop_size")), int(j.get("harmonic_num", d.harmonic_count)))


def config_from_json(root: dict) -> K.KittenTTSConfig:
    d = K.KittenTTSConfig()
    plbert = albert_config_from_json(root["plbert"]) if isinstance(root.get("plbert"), dict) else d.plbert
    gen = generator_config_from_json(root["istftnet"]) if isinstance(root.get("istftnet"), dict) else d.generator
    g = lambda k: int(root.get(k, getattr(d, k)))
    out_dim = int(root.get("decoder_out_dim", 0))
    if out_dim not in (0, gen.upsample_initial_channel):
        raise ValueError(f"Invalid KittenTTS config: decoder_out_dim={out_dim} must match upsample_initial_channel={gen.upsample_initial_channel}")
    return K.KittenTTSConfig(g("hidden_dim"), g("max_conv_dim"), g("max_dur"), g("n_layer"), g("n_token"), g("style_dim"), g("text_encoder_kernel_size"),
                             int(root.get("dim_in", d.asr_res_dim)), g("sample_rate"), plbert, gen)


def load_config(model_dir: str) -> K.KittenTTSConfig:
    with open(os.path.join(model_dir, "config.json"), encoding="utf-8") as f:
        return config_from_json(json.load(f))


def load_vocab(path: str, n_token: int) -> Dict[str, int]:
    """Phoneme vocabulary from ``config.json``: single-character keys mapped to ids below ``n_token``."""
    with open(path, encoding="utf-8") as f:
        root = json.load(f)
    vocab = root.get("vocab")
    if not isinstance(vocab, dict):
        raise ValueError(f"Missing or invalid vocab object in {path}")
    out = {}
    for key, value in vocab.items():
        if len(key) != 1:
            raise ValueError(f'Invalid vocab key "{key}" in {path}: expected one character')
        if isinstance(value, bool) or not isinstance(value, int) or value < 0:
            raise ValueError(f'Invalid vocab id for "{key}" in {path}: {value!r}')
        if value >= n_token:
            raise ValueError(f'Vocab id {value} for "{key}" in {path} is outside the embedding table (n_token={n_token})')
        out[key] = value
    return out


def encode_phoneme_ids(vocab: Dict[str, int], phonemes: str) -> List[int]:
    """``[0, ids of the known characters..., 0]``; characters outside the vocabulary are dropped."""
    return [0] + [vocab[c] for c in phonemes if c in vocab] + [0]


def voice_index_of_phoneme_count(count: int) -> int:
    return min(509, 0 if count == 0 else count - 1)


# ---- raw checkpoint / voicepack conversion ----------------------------------------------------------------------------------------
def convert_checkpoint(src: str, dst: str) -> None:
    """``{module: state_dict}`` payload of a Kokoro ``.pth`` -> flat ``module.name`` safetensors (a ``module.`` prefix left by
    DataParallel is dropped)."""
    payload = torch.load(src, map_location="cpu", weights_only=True)
    if not isinstance(payload, dict):
        raise TypeError(f"expected dict checkpoint, got {type(payload).__name__}")
    tensors = {}
    for top, state in payload.items():
        if isinstance(state, dict):
            for name, t in state.items():
                if isinstance(t, torch.Tensor):
                    tensors[f"{top}.{name[7:] if name.startswith('module.') else name}"] = t.detach().cpu().contiguous()
    if not tensors:
        raise RuntimeError(f"no tensors found in checkpoint {src}")
    os.makedirs(os.path.dirname(dst) or ".", exist_ok=True)
    st.save_file(tensors, dst)


def convert_voice(src: str, dst: str) -> None:
    t = torch.load(src, map_location="cpu", weights_only=True)
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"expected tensor voicepack, got {type(t).__name__}")
    os.makedirs(os.path.dirname(dst) or ".", exist_ok=True)
    st.save_file({"voice": t.detach().cpu().contiguous()}, dst)


def find_raw_model_file(model_dir: str) -> Optional[str]:
    for name in ("kokoro-v1_0.pth", "kokoro-v1_1-zh.pth"):
        if os.path.exists(os.path.join(model_dir, name)):
            return os.path.join(model_dir, name)
    if os.path.isdir(model_dir):
        for name in sorted(os.listdir(model_dir)):
            if name.endswith(".pth"):
                return os.path.join(model_dir, name)
    return None


def resolve_pretrained_dir(source: str, revision: Optional[str] = None) -> str:
    """A local directory with ``config.json`` and ``model.safetensors`` (converted from the raw checkpoint when only that exists)."""
    src = os.path.expanduser(source)
    model_dir = src if os.path.isdir(src) else hub.resolve_pretrained_dir(source, revision)
    if not os.path.exists(os.path.join(model_dir, "config.json")):
        raise FileNotFoundError(f"Missing config.json in {model_dir}")
    if not os.path.exists(os.path.join(model_dir, "model.safetensors")):
        raw = find_raw_model_file(model_dir)
        if raw is None:
            raise FileNotFoundError(f"No model.safetensors or raw .pth checkpoint found in {model_dir}")
        convert_checkpoint(raw, os.path.join(model_dir, "model.safetensors"))
    return model_dir


def ensure_voice_safetensors(model_dir: str, voice: str) -> str:
    """Path of the voice's safetensors file: ``voice`` is a name under ``voices/`` or a path to a ``.safetensors`` / ``.pt`` file."""
    if voice.endswith(".safetensors") or voice.endswith(".pt"):
        rel = voice
    else:
        rel = f"voices/{voice}.safetensors" if os.path.exists(os.path.join(model_dir, f"voices/{voice}.safetensors")) else f"voices/{voice}.pt"
    path = os.path.expanduser(rel if rel.startswith("/") or rel.startswith("~") else os.path.join(model_dir, rel))
    if rel.endswith(".safetensors"):
        if not os.path.exists(path):
            raise FileNotFoundError(f"Missing voice safetensors file at {path}")
        return path
    if not os.path.exists(path):
        raise FileNotFoundError(f"Missing voicepack file at {path}")
    out = path[:-3] + ".safetensors"
    if not os.path.exists(out):
        convert_voice(path, out)
    return out


@dataclass
class PretrainedBundle:
    cfg: K.KittenTTSConfig
    model: K.KittenTTS
    vocab: Dict[str, int]
    model_dir: str

    def input_ids_from_phonemes(self, phonemes: str) -> List[int]:
        return encode_phoneme_ids(self.vocab, phonemes)

    def load_voice_style(self, voice: str, phoneme_count: int) -> torch.Tensor:
        """[1, 2 * style_dim] row of the voice table for an utterance of ``phoneme_count`` characters."""
        table = st.Source.open(ensure_voice_safetensors(self.model_dir, voice)).load("voice").float()
        full = self.cfg.full_style_dim
        if table.dim() == 1:
            table = table[None]
        table = table.reshape(table.shape[0], -1)
        if table.shape[1] != full:
            raise st.SafeTensorsError(f"voice table has rows of {table.shape[1]} values, expected {full}")
        idx = min(voice_index_of_phoneme_count(phoneme_count), table.shape[0] - 1)
        return table[idx][None].to(self.model.device)

    def synthesize_phonemes(self, phonemes: str, voice: str, speed: float = 1.0, generator=None) -> K.KittenTTSOutput:
        ids = torch.tensor([self.input_ids_from_phonemes(phonemes)], dtype=torch.long, device=self.model.device)
        return self.model.synthesize(ids, self.load_voice_style(voice, len(phonemes)), speed, generator)

    def synthesize_phonemes_to_file(self, phonemes: str, voice: str, out_path: str, speed: float = 1.0, generator=None) -> K.KittenTTSOutput:
        out = self.synthesize_phonemes(phonemes, voice, speed, generator)
        out_path = os.path.expanduser(out_path)
        os.makedirs(os.path.dirname(out_path) or ".", exist_ok=True)
        audio = out.audio.reshape(-1).float().cpu()
        if out_path.endswith(".safetensors"):
            st.save_file({"audio": audio.contiguous()}, out_path)
        else:
            media.save_wav(out_path, audio, self.cfg.sample_rate)
        return out


def load_from_pretrained(source: str = DEFAULT_REPO_ID, revision: Optional[str] = None, device="cpu", log=None) -> PretrainedBundle:
    info = log or (lambda s: None)
    model_dir = resolve_pretrained_dir(source, revision)
    cfg = load_config(model_dir)
    info(f"Loading KittenTTS weights from {model_dir}...")
    model = K.load(cfg, os.path.join(model_dir, "model.safetensors"), device)
    return PretrainedBundle(cfg, model, load_vocab(os.path.join(model_dir, "config.json"), cfg.n_token), model_dir)
