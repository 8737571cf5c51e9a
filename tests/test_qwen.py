"""Qwen3 base blocks, causal LM cached/uncached parity, Flux embedder, loaders (Tests/TestQwen3Model.lean)."""
import json

import pytest
import torch

from tyr_b200.io import safetensors as st
from tyr_b200.models import qwen as Q


def tiny():
    return Q.QwenConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
                        num_key_value_heads=2, half_head_dim=4, eos_token_ids=(1,))


def test_config_presets_and_json():
    assert Q.QwenConfig.qwen3_4b().head_dim == 128
    f = Q.QwenConfig.flux_klein_text_encoder()
    assert (f.num_hidden_layers, f.num_attention_heads, f.num_key_value_heads, f.intermediate_size) == (36, 32, 8, 9728)
    c = Q.QwenConfig.from_json({"hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
                                "rope_theta": 1e6, "eos_token_id": 7})
    assert c.half_head_dim == 8 and c.rope_theta == 1e6 and c.eos_token_ids == (7,)
    with pytest.raises(ValueError, match="whole groups"):
        Q.QwenConfig(num_attention_heads=5, num_key_value_heads=2)


def test_cached_and_uncached_greedy_agree():
    lm = Q.Qwen3ForCausalLM.init(tiny())
    ids = torch.randint(2, 64, (2, 5))
    a = Q.generate_greedy(lm, ids, 6, eos_token_ids=())
    b = Q.generate_greedy_uncached(lm, ids, 6, eos_token_ids=())
    assert torch.equal(a, b) and a.shape == (2, 11)
    logits, hs = lm.forward_with_hidden_states(ids)
    assert len(hs) == 4 and torch.allclose(logits, lm.forward(ids))


def test_flux_embedder_concatenates_layers_and_respects_mask():
    m = Q.init_model(tiny())
    e = Q.QwenFluxEmbedder.from_model(m, 16, (0, 2))
    ids = torch.randint(2, 64, (2, 7))
    out = e.encode(ids)
    hs = Q.forward_with_hidden_states(m, ids)
    assert out.shape == (2, 7, 64) and torch.allclose(out[..., :32], hs[0]) and torch.allclose(out[..., 32:], hs[2])
    mask = torch.ones(2, 7)
    mask[0, 5:] = 0
    om = e.encode_masked(ids, mask)
    assert torch.allclose(om[1], out[1], atol=1e-5) and torch.allclose(om[0, :5], out[0, :5], atol=1e-5)
    with pytest.raises(ValueError, match="exceed"):
        Q.QwenFluxEmbedder.from_model(m, 16, (9,)).encode(ids)


def test_loader_roundtrip_fp8_blocks_and_omni_names(tmp_path):
    cfg = tiny()
    lm = Q.Qwen3ForCausalLM.init(cfg, tie_word_embeddings=False)
    sd = {k: v.contiguous() for k, v in Q.state_dict(lm).items()}
    p = str(tmp_path / "m.safetensors")
    st.save_file(sd, p)
    lm2 = Q.load_qwen3_causal_lm(cfg, p, dtype=torch.float32)
    ids = torch.randint(2, 64, (1, 4))
    assert torch.equal(lm.forward(ids), lm2.forward(ids))
    # thinker-prefixed checkpoint
    d = tmp_path / "omni"
    d.mkdir()
    st.save_file({Q.qwen25_omni_name_map(k): v for k, v in sd.items()}, str(d / "model.safetensors"))
    json.dump({"thinker_config": {"text_config": {"vocab_size": 64, "hidden_size": 32, "intermediate_size": 64,
               "num_hidden_layers": 3, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 8}}}, open(d / "config.json", "w"))
    lm3 = Q.load_qwen25_omni_thinker(str(d), dtype=torch.float32)
    assert torch.equal(lm.forward(ids), lm3.forward(ids))
    # fp8 block scales
    w = torch.randn(128, 256)
    src_p = str(tmp_path / "q.safetensors")
    st.save_file({"x.weight": w.to(torch.float8_e4m3fn), "x.weight_scale_inv": torch.tensor([[2.0, 0.5]])}, src_p)
    got = Q._load_linear(st.Source.open(src_p), "x", 128, 256, "cpu", torch.float32)
    ref = w.to(torch.float8_e4m3fn).float()
    assert torch.equal(got[:, :128], ref[:, :128] * 2.0) and torch.equal(got[:, 128:], ref[:, 128:] * 0.5)


@pytest.mark.gpu
def test_gpu_qwen3_graph_decode_step_matches_eager_session(monkeypatch):
    """Decode steps replayed from one CUDA graph (device-side position, fused KV append) against the eager cached step."""
    from tyr_b200.models import qwen as Q
    cfg = Q.QwenConfig(vocab_size=200, hidden_size=256, intermediate_size=512, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                       half_head_dim=64, rope_theta=10000.0, rms_norm_eps=1e-6)
    lm = Q.Qwen3ForCausalLM.init(cfg, device="cuda", dtype=torch.bfloat16, seed=3)
    ids = torch.randint(0, 200, (3, 37), device="cuda")
    toks = torch.randint(0, 200, (6, 3), device="cuda")
    graph = Q.Qwen3Session(lm, 3, 64)
    assert graph.device_step_supported()
    outs = [graph.prefill(ids)] + [graph.step(t).clone() for t in toks]          # a replay returns the graph's static output tensor
    assert graph._graph.replays == 6 and graph.pos == 43
    monkeypatch.setenv("TYR_DECODE_GRAPH", "0")
    eager = Q.Qwen3Session(lm, 3, 64)
    refs = [eager.prefill(ids)] + [eager.step(t) for t in toks]
    for a, b in zip(outs, refs):
        assert (a.float() - b.float()).abs().max() < 0.06 * max(1.0, b.float().abs().max().item())
    assert torch.equal(outs[-1].argmax(-1), refs[-1].argmax(-1)) or (outs[-1].float() - refs[-1].float()).abs().max() < 0.05
