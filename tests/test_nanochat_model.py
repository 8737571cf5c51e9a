"""NanoChat model: fused training path vs the op-for-op reference restatement
(the reference's own model tests: Tests/TestModdedGPT.lean:43-293)."""
import pytest
import torch

from tyr_b200.models import nanochat as nc


def tiny_cfg(**kw):
    base = dict(vocab_size=128, n_layer=7, n_head=2, half_head_dim=32, max_seq_len=32)
    base.update(kw)
    return nc.Config(**base)


def randomize(params, seed=0):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for k, v in params.master.items():
            if k == "scalars":
                v.copy_(1.1 + 0.3 * torch.randn(v.shape, generator=g))
            else:
                v.copy_(torch.randn(v.shape, generator=g) * 0.05)
    params.sync_work_from_master()
    params.refresh_leaves()


def test_config_defaults_and_d20():
    c = nc.Config()
    assert (c.vocab_size, c.n_layer, c.n_head, c.head_dim, c.model_dim) == (50304, 11, 6, 128, 768)
    d20 = nc.depth_config(20)
    assert (d20.model_dim, d20.n_head, d20.head_dim, d20.vocab_size, d20.max_seq_len) == (1280, 10, 128, 65536, 2048)
    assert nc.Config.from_json(d20.to_json()) == d20
    with pytest.raises(ValueError):
        nc.Config(vocab_size=0)


def test_window_pattern_and_value_embed_routing():
    assert nc.get_window_size_for_layer("SL", 0, 4, 64) == 32
    assert nc.get_window_size_for_layer("SL", 1, 4, 64) is None
    assert nc.get_window_size_for_layer("S", 3, 4, 64) is None  # final layer is always full
    c = nc.depth_config(20)
    got = [nc.layer_value_embed_index(c, i) for i in range(20)]
    assert got[:3] == [0, 1, 2] and got[17:] == [0, 1, 2] and all(g is None for g in got[3:17])


@pytest.mark.parametrize("pattern", ["L", "SL"])
def test_fused_matches_reference_cpu_fp32(pattern):
    cfg = tiny_cfg(window_pattern=pattern)
    params = nc.ModdedGPTParams(cfg, device="cpu", compute_dtype=torch.float32, seed=1)
    randomize(params)
    B, T = 2, 32
    g = torch.Generator().manual_seed(3)
    x = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    y = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    params.zero_grads()
    loss = nc.loss_fused(params, x, y, ce_chunk_rows=24)
    loss.backward()
    ref_p = {k: v.detach().clone().requires_grad_(True) for k, v in params.named_parameters("master").items()}
    ref_loss = nc.loss_reference(ref_p, cfg, x, y, params.cos, params.sin)
    ref_loss.backward()
    assert torch.allclose(loss, ref_loss, rtol=1e-4, atol=1e-5), (loss.item(), ref_loss.item())
    grads = params.named_parameters("grad")
    for name, rp in ref_p.items():
        if name == "scalars.values":
            got = params.work["scalars"].grad
        elif name == "smearGate.weight":
            got = params.work["smear_gate"].grad
        else:
            got = grads[name]
        assert got is not None, name
        err = (got - rp.grad).abs().max().item()
        scale = rp.grad.abs().max().item() + 1e-8
        assert err <= 2e-3 * scale + 1e-6, (name, err, scale)


def test_initialisation_matches_reference_rules():
    cfg = tiny_cfg()
    p = nc.ModdedGPTParams(cfg, seed=0, compute_dtype=torch.float32)
    named = p.named_parameters()
    assert torch.count_nonzero(named["blocks.0.attn.wO"]) == 0
    assert torch.count_nonzero(named["blocks.0.mlp.cProj"]) == 0
    assert "blocks.5.attn.wQ" not in named and "blocks.5.mlp.cFc" in named
    assert torch.allclose(named["scalars.values"], torch.full((cfg.n_layer * 4 + 8,), 1.1))
    assert named["smearGate.weight"].shape == (1, 12)
