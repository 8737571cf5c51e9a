"""Qwen3.5: gated delta rule (chunked vs recurrent), hybrid cache parity, MoE block, loader
(Tests/TestQwen35Model.lean:150-264)."""
import pytest
import torch

from tyr_b200.io import safetensors as st
from tyr_b200.models import qwen35 as Q
from tyr_b200.ops import delta_rule as D


def tiny(moe=0, **kw):
    base = dict(vocab_size=80, hidden_size=32, intermediate_size=64, num_hidden_layers=4, num_attention_heads=4,
                num_key_value_heads=2, head_dim=16, half_rotary_dim=4, linear_key_head_dim=8, linear_value_head_dim=8,
                linear_num_key_heads=2, linear_num_value_heads=4, moe_intermediate_size=16,
                shared_expert_intermediate_size=16, num_experts_per_tok=2, num_experts=moe)
    base.update(kw)
    return Q.Qwen35Config(**base)


def _gdr_inputs(B=2, S=150, H=3, dk=16, dv=24, device="cpu", dtype=torch.float32):
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g)
    return (r(B, S, H, dk).to(device, dtype), r(B, S, H, dk).to(device, dtype), r(B, S, H, dv).to(device, dtype),
            (-torch.nn.functional.softplus(r(B, S, H))).to(device), torch.sigmoid(r(B, S, H)).to(device))


def test_chunked_matches_recurrent_and_chains_state():
    q, k, v, g, beta = _gdr_inputs()
    o1, s1 = D.recurrent_gated_delta_rule(q, k, v, g, beta)
    o2, s2 = D.chunk_gated_delta_rule(q, k, v, g, beta)
    assert torch.allclose(o1, o2, atol=1e-5) and torch.allclose(s1, s2, atol=1e-5)
    o3, s3 = D.chunk_gated_delta_rule(q[:, :100], k[:, :100], v[:, :100], g[:, :100], beta[:, :100])
    o4, s4 = D.chunk_gated_delta_rule(q[:, 100:], k[:, 100:], v[:, 100:], g[:, 100:], beta[:, 100:], state=s3)
    assert torch.allclose(torch.cat([o3, o4], 1), o1, atol=1e-5) and torch.allclose(s4, s1, atol=1e-5)


def test_decode_step_updates_state_in_place_cpu():
    q, k, v, g, beta = _gdr_inputs(S=5, H=4)
    qk, kk = q[:, :, :2], k[:, :, :2]                       # 2 key heads repeated onto 4 value heads
    ref, sref = D.recurrent_gated_delta_rule(qk.repeat_interleave(2, 2), kk.repeat_interleave(2, 2), v, g, beta)
    state = torch.zeros(2, 4, 16, 24)
    outs = [D.gdr_decode_step(qk[:, i:i + 1], kk[:, i:i + 1], v[:, i:i + 1], g[:, i:i + 1], beta[:, i:i + 1], state) for i in range(5)]
    assert torch.allclose(torch.cat(outs, 1), ref, atol=1e-5) and torch.allclose(state, sref, atol=1e-5)


def test_config_presets_and_validation():
    assert Q.Qwen35Config.qwen35_35b_a3b().num_experts == 256 and Q.Qwen35Config.qwen36_35b_a3b().eos_token_id == 248044
    c = Q.Qwen35Config()
    assert c.layer_types[:4] == [Q.LINEAR, Q.LINEAR, Q.LINEAR, Q.FULL] and c.linear_conv_dim == 2 * 2048 + 4096
    j = {"text_config": {"num_hidden_layers": 4, "hidden_size": 64, "head_dim": 32, "partial_rotary_factor": 0.25,
                         "layer_types": ["linear_attention", "full_attention"] * 2, "eos_token_id": [5, 6]}}
    c2 = Q.Qwen35Config.from_json(j)
    assert c2.half_rotary_dim == 4 and c2.is_full(1) and c2.eos_token_id == 5
    with pytest.raises(ValueError, match="whole multiple of key heads"):
        tiny(linear_num_value_heads=3)
    assert "Qwen/Qwen3.5-27B" in Q.PRETRAINED_REPOS


@pytest.mark.parametrize("moe", [0, 8])
def test_cached_generation_matches_uncached(moe):
    m = Q.init(tiny(moe))
    ids = torch.randint(0, 80, (2, 9))
    assert torch.equal(Q.generate_greedy(m, ids, 5), Q.generate_uncached(m, ids, 5))
    c = Q.HybridCache(m, 2, 20)
    full = Q.forward(m, ids)
    assert torch.allclose(c.prefill(ids[:, :2]), full[:, 1], atol=1e-4)        # prompt shorter than the conv kernel
    for t in range(2, 9):
        assert torch.allclose(c.step(ids[:, t]), full[:, t], atol=1e-4), t
    assert c.state_bytes() > 0


def test_padding_mask_zeroes_padded_inputs_of_linear_layers():
    m = Q.init(tiny())
    ids = torch.randint(0, 80, (1, 6))
    mask = torch.ones(1, 6, dtype=torch.long)
    out = Q.forward(m, ids, attn_mask=mask)
    assert torch.allclose(out, Q.forward(m, ids), atol=1e-5)


def test_loader_roundtrip(tmp_path):
    for moe in (0, 4):
        cfg = tiny(moe)
        m = Q.init(cfg)
        p = str(tmp_path / f"m{moe}.safetensors")
        st.save_file({k: v.contiguous() for k, v in Q.state_dict(m).items()}, p)
        m2 = Q.load(cfg, p, dtype=torch.float32)
        ids = torch.randint(0, 80, (1, 5))
        assert torch.equal(Q.forward(m, ids), Q.forward(m2, ids))


@pytest.mark.gpu
@pytest.mark.parametrize("tile,dk", [(True, 128), (False, 128), (True, 64), (False, 64)])
def test_gpu_gdr_decode_kernel_matches_recurrence(tile, dk, monkeypatch):
    """Both forms of the decode step (state tile staged in shared memory by bulk copies; state columns held in registers)."""
    monkeypatch.setattr(D, "_GDR_TILE", tile)
    monkeypatch.setattr(D, "_GDR_TILE_MIN_TILES", 0)
    q, k, v, g, beta = _gdr_inputs(B=3, S=6, H=8, dk=dk, dv=128, device="cuda", dtype=torch.bfloat16)
    qk, kk = q[:, :, :4].contiguous(), k[:, :, :4].contiguous()
    ref, sref = D.recurrent_gated_delta_rule(qk.float().repeat_interleave(2, 2), kk.float().repeat_interleave(2, 2), v.float(), g, beta)
    state = torch.zeros(3, 8, dk, 128, device="cuda")
    outs = []
    for i in range(6):
        outs.append(D.gdr_decode_step(qk[:, i:i + 1].contiguous(), kk[:, i:i + 1].contiguous(), v[:, i:i + 1].contiguous(),
                                      g[:, i:i + 1], beta[:, i:i + 1], state))
    out = torch.cat(outs, 1).float()
    assert torch.allclose(out, ref, atol=2e-2, rtol=2e-2), (out - ref).abs().max().item()
    assert torch.allclose(state, sref, atol=1e-3, rtol=1e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("tile", [True, False])
def test_gpu_gdn_decode_fused_matches_library_op_sequence(tile, monkeypatch):
    """Conv + gates kernel and the recurrent kernel with the gated-norm epilogue against the op-by-op decode branch, on column
    windows of one projection output, over several tokens (conv window and recurrent state carried in place)."""
    cfg = tiny(0, hidden_size=256, intermediate_size=512, head_dim=128, half_rotary_dim=32, linear_key_head_dim=128, linear_value_head_dim=128,
               num_attention_heads=4, num_key_value_heads=1)
    m = Q.init(cfg, device="cuda", dtype=torch.bfloat16)
    monkeypatch.setattr(D, "_GDR_TILE", tile)
    monkeypatch.setattr(D, "_GDR_TILE_MIN_TILES", 0)
    layer = next(l for i, l in enumerate(m.layers) if not cfg.is_full(i))
    mix = layer.mixer
    mix.conv1d_bias = (torch.randn(cfg.linear_conv_dim, device="cuda") * 0.1).bfloat16()
    B, cd, vd, Hv, K = 5, cfg.linear_conv_dim, cfg.linear_value_dim, cfg.linear_num_value_heads, cfg.linear_conv_kernel_dim
    g = torch.Generator(device="cuda").manual_seed(2)

    def fresh():
        gs = torch.Generator(device="cuda").manual_seed(9)
        return Q.LinearState(torch.randn(B, cd, K, device="cuda", generator=gs).bfloat16(),
                             torch.randn(B, Hv, cfg.linear_key_head_dim, cfg.linear_value_head_dim, device="cuda", generator=gs) * 0.1)
    s_ref, s_fused = fresh(), fresh()
    for t in range(4):
        proj = torch.randn(B, 1, cd + vd + 2 * Hv + 8, device="cuda", generator=g).bfloat16()
        assert D._tile_ok(128, proj[..., cd:cd + vd], proj[..., cd:cd + vd], B * Hv) == tile      # the z window is 8-byte aligned
        views = (proj[..., :cd], proj[..., cd:cd + vd], proj[..., cd + vd:cd + vd + Hv], proj[..., cd + vd + Hv:cd + vd + 2 * Hv])
        D._GDN_FUSED = False
        try:
            ref = Q.gated_delta_net_core(cfg, mix, *views, s_ref)
        finally:
            D._GDN_FUSED = True
        assert D.gdn_decode_fused_supported(views[0], s_fused.conv, s_fused.rec, 128, 128)
        got = Q.gated_delta_net_core(cfg, mix, *views, s_fused)
        assert got.shape == ref.shape
        assert (got.float() - ref.float()).abs().max().item() < 2e-2 * max(1.0, ref.float().abs().max().item()), t
        assert torch.equal(s_fused.conv, s_ref.conv)
        assert torch.allclose(s_fused.rec, s_ref.rec, atol=2e-3, rtol=2e-3)


@pytest.mark.gpu
def test_gpu_qwen35_moe_bf16_cached_matches_full_forward():
    cfg = tiny(8, hidden_size=256, head_dim=128, half_rotary_dim=32, linear_key_head_dim=128, linear_value_head_dim=128,
               moe_intermediate_size=128, shared_expert_intermediate_size=128, num_attention_heads=2, num_key_value_heads=1)
    m = Q.init(cfg, device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, 80, (2, 140), device="cuda")
    with torch.no_grad():
        full = Q.forward(m, ids).float()
        c = Q.HybridCache(m, 2, 160)
        scale = full.abs().max().item()
        errs = [(c.prefill(ids[:, :130]).float() - full[:, 129]).abs().amax(dim=1)]
        for t in range(130, 140):
            errs.append((c.step(ids[:, t]).float() - full[:, t]).abs().amax(dim=1))
        # a router near-tie (top-2 of 8 random experts) can pick a different expert once the arithmetic differs in the last
        # bf16 bit; that moves the row discretely and, through the recurrent state, the next few steps of that row while the
        # gate decays it.  A wrong cache or state update would instead break every step of every row.
        ok = torch.stack(errs) < 0.06 * scale
        assert bool(ok[0].all()) and ok.float().mean().item() >= 0.5 and bool(ok[-2:].all())


def test_device_position_decode_step_matches_host_position_step():
    m = Q.init(tiny())
    ids = torch.randint(0, 80, (2, 12))
    a, b = Q.HybridCache(m, 2, 16), Q.HybridCache(m, 2, 16)
    a.prefill(ids[:, :7]), b.prefill(ids[:, :7])
    b.pos_t = torch.tensor([b.pos], dtype=torch.int32)
    for t in range(7, 12):
        want = a.step(ids[:, t])
        with torch.no_grad():
            got = b._device_step(ids[:, t])
        b._advance_host()
        assert int(b.pos_t) == b.pos == a.pos and torch.allclose(got, want, atol=2e-4), t


@pytest.mark.gpu
def test_gpu_qwen35_dense_graph_decode_matches_full_forward():
    cfg = tiny(0, hidden_size=256, intermediate_size=512, head_dim=128, half_rotary_dim=32, linear_key_head_dim=128, linear_value_head_dim=128,
               num_attention_heads=4, num_key_value_heads=1)
    m = Q.init(cfg, device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, 80, (2, 140), device="cuda")
    with torch.no_grad():
        full = Q.forward(m, ids).float()
        c = Q.HybridCache(m, 2, 160)
        scale = full.abs().max().item()
        assert c.device_step_supported()
        assert (c.prefill(ids[:, :130]).float() - full[:, 129]).abs().max().item() < 0.06 * scale
        for t in range(130, 140):
            assert (c.step(ids[:, t]).float() - full[:, t]).abs().max().item() < 0.06 * scale, t
        assert c._graph.replays == 10 and int(c.pos_t) == 140
