"""Gemma 4 multimodal wrapper: patch grid, 2-D rotary, clipped linears, pooled features, bidirectional image spans, generation."""
import pytest
import torch

from tyr_b200.models import gemma4 as G
from tyr_b200.models import gemma4_vl as V


def tiny(bidir=""):
    text = G.Gemma4Config(vocab_size=70, hidden_size=32, intermediate_size=48, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                          half_head_dim=4, global_half_head_dim=8, sliding_window=4, half_full_rotary_dim=2, layer_types=[G.SLIDING, G.SLIDING, G.FULL],
                          hidden_size_per_layer_input=8, vocab_size_per_layer_input=70, use_bidirectional_attention=bidir, eos_token_id=(1,))
    vis = V.VisionConfig(hidden_size=16, intermediate_size=32, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=2, quarter_head_dim=2, patch_size=2,
                         pooling_kernel_size=2, position_embedding_size=16)
    return V.VLConfig(text, vis, image_token_id=60, boi_token_id=61, eoi_token_id=62, video_token_id=63, audio_token_id=64, vision_soft_tokens_per_image=4)


def test_config_patch_grid_and_masks():
    with pytest.raises(ValueError, match="heads of 4"):
        V.VisionConfig(hidden_size=100)
    assert V.ImageProcessorConfig(max_soft_tokens=0).soft_token_count() == 280
    img = torch.arange(3 * 4 * 6, dtype=torch.float32).reshape(3, 4, 6)
    g = V.patch_grid(img, 2)
    assert g.shape == (2, 3, 12) and torch.equal(g[0, 1].reshape(3, 2, 2), img[:, 0:2, 2:4])
    ids = torch.tensor([[0, 5, 60, 60, 7, 60, 60, 60, 8]])
    sliding, full = V.vision_group_masks(ids, 60, 0, sliding_window=2)
    assert bool(full[0, 2, 3]) and bool(full[0, 5, 7]) and not bool(full[0, 2, 5]) and not bool(full[0, 4, 5])     # bidirectional inside a span only
    assert not bool(full[0, 1, 0]) and bool(full[0, 4, 1]) and not bool(sliding[0, 4, 1]) and bool(sliding[0, 5, 7])  # pad is never attended; window on sliding layers
    x = torch.randn(1, 6, 2, 8)
    r = V.rotary_2d(x, 2, 3, 100.0)
    assert torch.allclose(r[0, 0], x[0, 0], atol=1e-6) and not torch.allclose(r[0, 4], x[0, 4])                    # patch (0,0) is not rotated
    assert torch.allclose(r[0, 3, :, :4], x[0, 3, :, :4], atol=1e-6)                                               # column 0: the x half stays


def test_vision_features_clipping_and_standardisation():
    cfg = tiny()
    m = V.init(cfg)
    grid = V.patch_grid(torch.rand(3, 8, 8), 2)
    feats = m.get_image_features(grid)
    assert feats.shape == (4, 32)
    m.vision_tower.clip["encoder.layers.0.mlp.down_proj"] = (None, None, -0.01, 0.01)
    assert not torch.allclose(m.get_image_features(grid), feats)
    m.vision_tower.clip.clear()
    m.vision_tower.p["std_bias"], m.vision_tower.p["std_scale"] = torch.full((16,), 0.5), torch.full((16,), 2.0)
    assert not torch.allclose(m.get_image_features(grid), feats)
    assert V.Gemma4VL.repeat_features_for_batch(feats, 3).shape == (12, 32)


@pytest.mark.parametrize("bidir", ["", "vision"])
def test_forward_and_cached_generation_agree(bidir):
    cfg = tiny(bidir)
    m = V.init(cfg)
    feats = m.get_image_features(V.patch_grid(torch.rand(3, 8, 8), 2))
    ids = torch.tensor([[5, 61, 60, 60, 60, 60, 62, 9, 11]])
    logits = m.forward(ids, feats)
    assert logits.shape == (1, 9, 70) and not torch.allclose(logits, m.forward(ids))
    out = m.generate(ids, 3, eos_token_ids=(), image_features=feats)
    assert out.shape == (1, 12) and int(out[0, 9]) == int(logits[0, -1].argmax())
    with pytest.raises(ValueError, match="count mismatch"):
        m.forward(ids[:, :5], feats)
    if bidir:
        causal = tiny("")
        m2 = V.Gemma4VL(causal, m.vision_tower, m.embedding_projection, m.language_model)
        assert not torch.allclose(m2.forward(ids, feats)[0, 2], logits[0, 2], atol=1e-5)        # the first image token now sees the later ones
