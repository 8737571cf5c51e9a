"""Gemma 4: config rules, KV sharing, cached vs uncached parity, MoE branch, per-layer inputs, loader padding."""
import pytest
import torch

from tyr_b200.io import safetensors as st
from tyr_b200.models import gemma4 as G


def tiny(**kw):
    base = dict(vocab_size=70, hidden_size=32, intermediate_size=48, num_hidden_layers=6, num_attention_heads=4, num_key_value_heads=2,
                num_global_key_value_heads=1, half_head_dim=4, global_half_head_dim=8, sliding_window=5, half_full_rotary_dim=2,
                layer_types=[G.SLIDING, G.SLIDING, G.FULL, G.SLIDING, G.SLIDING, G.FULL], num_kv_shared_layers=2, use_double_wide_mlp=True,
                hidden_size_per_layer_input=8, vocab_size_per_layer_input=70, eos_token_id=(1,))
    base.update(kw)
    return G.Gemma4Config(**base)


def test_config_rules():
    c = G.Gemma4Config()
    assert c.layer_types[5] == G.FULL and c.layer_types[-1] == G.FULL and c.full_head_dim == 512 and c.head_dim == 256
    t = tiny()
    assert t.first_kv_shared_layer == 4 and t.shared_source_layer(4) == 3 and t.shared_source_layer(5) == 2 and t.shared_source_layer(1) is None
    assert t.layer_intermediate_size(5) == 96 and t.layer_intermediate_size(0) == 48 and t.geometry(2) == (1, 16) and t.geometry(0) == (2, 8)
    with pytest.raises(ValueError, match="last layer must be full"):
        tiny(layer_types=[G.SLIDING] * 6)
    with pytest.raises(ValueError, match="top_k_experts"):
        tiny(enable_moe_block=True, num_experts=4, top_k_experts=0, moe_intermediate_size=8)
    j = {"text_config": {"num_hidden_layers": 6, "head_dim": 8, "global_head_dim": 16, "hidden_size": 32, "num_attention_heads": 4, "num_key_value_heads": 2,
                         "layer_types": tiny().layer_types, "rope_parameters": {"full_attention": {"partial_rotary_factor": 0.25, "rope_theta": 5e5}},
                         "final_logit_softcapping": None}}
    cj = G.Gemma4Config.from_json(j)
    assert cj.half_full_rotary_dim == 2 and cj.full_rope_theta == 5e5 and cj.final_logit_softcapping is None


def test_full_rotary_passes_tail_channels():
    (sc, ss), (fc, fs) = G.rotary_tables(tiny(), 7, "cpu")
    assert sc.shape == (7, 4) and fc.shape == (7, 8) and torch.equal(fc[:, 2:], torch.ones(7, 6)) and torch.equal(fs[:, 2:], torch.zeros(7, 6))


@pytest.mark.parametrize("moe", [False, True])
def test_cached_matches_uncached(moe):
    cfg = tiny(enable_moe_block=moe, num_experts=4 if moe else 0, top_k_experts=2 if moe else 0, moe_intermediate_size=8 if moe else 0)
    m = G.init(cfg)
    for l in m.layers:
        l.layer_scalar.fill_(0.9)
    ids = torch.randint(2, 70, (2, 12))
    full = G.forward(m, ids)
    assert full.shape == (2, 12, 70) and full.abs().max() <= 30.0
    c = G.Gemma4Cache(m, 2, 16)
    assert sum(x is not None for x in c.caches) == 4
    assert torch.allclose(c.prefill(ids[:, :7]), full[:, 6], atol=1e-4)
    for t in range(7, 12):
        assert torch.allclose(c.step(ids[:, t]), full[:, t], atol=1e-4), t
    out = G.generate_greedy(m, ids[:, :3], 4, eos_token_ids=())
    assert out.shape == (2, 7) and torch.equal(out[:, 3], G.forward(m, ids[:, :3])[:, -1].argmax(-1))


def test_edge_mask_makes_attention_bidirectional():
    m = G.init(tiny(num_kv_shared_layers=0, hidden_size_per_layer_input=0, use_double_wide_mlp=False))
    ids = torch.randint(2, 70, (1, 6))
    causal = torch.tril(torch.ones(6, 6, dtype=torch.bool))[None]
    assert not torch.allclose(G.forward(m, ids, edge_mask=causal)[:, 0], G.forward(m, ids, edge_mask=torch.ones(1, 6, 6, dtype=torch.bool))[:, 0])


def test_loader_pads_smaller_geometry(tmp_path):
    cfg = tiny(enable_moe_block=True, num_experts=4, top_k_experts=2, moe_intermediate_size=8)
    m = G.init(cfg)
    p = str(tmp_path / "g.safetensors")
    sd = {k: v.contiguous() for k, v in G.state_dict(m).items()}
    assert sd["model.language_model.layers.0.self_attn.q_proj.weight"].shape == (4 * 8, 32)
    assert sd["model.language_model.layers.2.self_attn.q_proj.weight"].shape == (4 * 16, 32)
    st.save_file(sd, p)
    m2 = G.load(cfg, p, dtype=torch.float32)
    assert m2.layers[0].self_attn.q_proj.shape == (64, 32) and m2.layers[0].mlp.gate_proj.shape == (96, 32)
    ids = torch.randint(2, 70, (1, 5))
    assert torch.allclose(G.forward(m, ids), G.forward(m2, ids), atol=1e-5)
