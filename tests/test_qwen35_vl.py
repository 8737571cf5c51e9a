"""Qwen3.5 multimodal wrapper: patchify layout, vision tower shapes, placeholder scatter, cached generation."""
import pytest
import torch

from tyr_b200.models import qwen35 as Q
from tyr_b200.models import qwen35_vl as V


def tiny():
    text = Q.Qwen35Config(vocab_size=90, hidden_size=32, intermediate_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                          half_rotary_dim=4, linear_key_head_dim=8, linear_value_head_dim=8, linear_num_key_heads=2, linear_num_value_heads=4)
    vis = V.VisionConfig(depth=2, hidden_size=24, intermediate_size=48, num_heads=2, half_head_dim=6, in_channels=3, patch_size=4, spatial_merge_size=2,
                         temporal_patch_size=2, out_hidden_size=32, num_position_embeddings=64)
    return V.VLConfig(text, vis, image_token_id=80, video_token_id=81, vision_start_token_id=82, vision_end_token_id=83)


def test_config_rules_and_json():
    with pytest.raises(ValueError, match="heads of even width"):
        V.VisionConfig(hidden_size=100, num_heads=3, half_head_dim=16)
    with pytest.raises(ValueError, match="text hidden size"):
        V.VLConfig(Q.Qwen35Config.qwen35_0_8b(), V.VisionConfig())
    c = V.VisionConfig.from_json({"hidden_size": 768, "num_heads": 12, "depth": 3, "out_hidden_size": 1024})
    assert c.half_head_dim == 32 and c.patch_dim == 3 * 2 * 16 * 16 and c.merge_unit == 4


def test_patchify_groups_two_by_two_neighbours():
    c = tiny().vision_config
    img = torch.arange(2 * 3 * 16 * 8, dtype=torch.float32).reshape(2, 3, 16, 8)
    p = V.patchify(img, c)
    assert p.shape == (8, c.patch_dim)                      # (16/4) x (8/4) patches, one temporal group
    first = p[0].reshape(3, 2, 4, 4)
    assert torch.equal(first, img[:, :, :4, :4].permute(1, 0, 2, 3))
    second = p[1].reshape(3, 2, 4, 4)                       # right-hand neighbour inside the same 2x2 group
    assert torch.equal(second, img[:, :, :4, 4:8].permute(1, 0, 2, 3))
    third = p[2].reshape(3, 2, 4, 4)                        # then the row below
    assert torch.equal(third, img[:, :, 4:8, :4].permute(1, 0, 2, 3))
    with pytest.raises(ValueError):
        V.patchify(torch.zeros(1, 3, 16, 8), c)


def test_features_replace_placeholders_and_generation_uses_them():
    cfg = tiny()
    m = V.init(cfg)
    patches = V.patchify(torch.randn(2, 3, 16, 8), cfg.vision_config)
    feats = m.get_image_features(patches)
    assert feats.shape == (2, 32)
    ids = torch.tensor([[5, 82, 80, 80, 83, 7, 9]])
    emb = m.build_inputs_embeds(ids, feats)
    assert torch.allclose(emb[0, 2:4], feats) and torch.equal(emb[0, 0], m.language_model.embed_tokens[5])
    with pytest.raises(ValueError, match="count mismatch"):
        m.build_inputs_embeds(ids[:, :3], feats)
    with pytest.raises(ValueError, match="exceeds"):
        m.visual.forward(torch.zeros(68, cfg.vision_config.patch_dim))
    logits = m.forward(ids, image_patches=patches)
    assert logits.shape == (1, 7, 90) and not torch.allclose(logits, m.forward(ids))
    out = m.generate(ids, 3, image_features=feats)
    assert out.shape == (1, 10) and int(out[0, 7]) == int(logits[0, -1].argmax())
