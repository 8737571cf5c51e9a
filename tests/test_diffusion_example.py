"""Masked discrete diffusion example: schedule, loss, samplers, training and exact resume."""
import pytest
import torch

from tyr_b200.examples import diffusion as D


def test_schedule_masks_more_at_later_steps_and_never_the_context():
    cfg = D.Config.tiny()
    s = D.MaskedDiffusionSchedule.init(cfg.diffusion_steps, cfg.mask_token_id, cfg.context_len)
    assert torch.allclose(s.mask_probs[0], torch.tensor(1.0 / 16)) and s.mask_probs[-1] == 1.0
    x0 = torch.randint(1, 128, (64, cfg.seq_len))
    early = s.add_masks(x0, torch.zeros(64, dtype=torch.int64))
    late = s.add_masks(x0, torch.full((64,), 15))
    assert (early == 0).float().mean() < 0.15 and bool((late[:, cfg.context_len:] == 0).all())
    assert torch.equal(late[:, :cfg.context_len], x0[:, :cfg.context_len])


def test_masked_loss_counts_only_masked_positions():
    logits = torch.zeros(1, 4, 8)
    logits[0, 0, 3] = 10.0
    targets = torch.tensor([[3, 1, 2, 5]])
    x_t = torch.tensor([[0, 1, 2, 5]])
    assert D.masked_cross_entropy_loss(logits, targets, x_t, 0) < 1e-3
    assert abs(D.masked_cross_entropy_loss(logits, targets, torch.tensor([[3, 0, 2, 5]]), 0).item() - torch.log(torch.tensor(8.0)).item()) < 1e-3


def test_config_validation_and_samplers_fill_every_position():
    with pytest.raises(ValueError):
        D.Config(context_len=300)
    cfg = D.Config.tiny()
    p = D.init(cfg, seed=1)
    with torch.no_grad():
        p["output_head"].copy_(torch.randn_like(p["output_head"]) * 0.5)
    ctx = torch.randint(1, 128, (2, cfg.context_len))
    x = D.sample_confidence(p, cfg, 2, threshold=0.9, context=ctx, max_steps=cfg.seq_len)
    assert not bool((x == 0).any()) and torch.equal(x[:, :cfg.context_len], ctx)
    y = D.sample_top_k(p, cfg, 8, 2, max_steps=8)
    assert not bool((y == 0).any())                                             # 64 positions in 8 steps of 8
    with pytest.raises(ValueError, match="top-k"):
        D.sample_top_k(p, cfg, 0)
    with pytest.raises(ValueError, match="temperature"):
        D.sample_confidence(p, cfg, 1, temperature=0.0)
    assert D.decode_ascii(torch.tensor([72, 105, 0, 10])) == "Hi_\n"


def test_training_reduces_loss_and_resume_is_exact(tmp_path):
    cfg = D.Config(seq_len=32, n_layer=1, n_head=2, half_head_dim=8, diffusion_steps=8, context_len=0)
    data = D.encode_ascii("abcdefgh" * 200)
    lines = []
    tc = D.TrainConfig(iterations=60, batch_size=8, lr=3e-3, warmup=5, log_interval=10, checkpoint_interval=30)
    ck = str(tmp_path / "ck")
    p_full, loss_full = D.train(cfg, data, tc, checkpoint_dir=ck, log=lines.append)
    first = float(lines[0].split("loss ")[1].split()[0])
    assert loss_full < first * 0.7
    # interrupted at 30 and resumed to 60: the same weights as the uninterrupted run
    ck2 = str(tmp_path / "ck2")
    quiet = D.TrainConfig(iterations=60, batch_size=8, lr=3e-3, warmup=5, log_interval=0, checkpoint_interval=0)
    D.train(cfg, data, quiet, checkpoint_dir=ck2, stop_at=30)
    assert D.load_checkpoint(ck2)[2] == 30
    p_res, _ = D.train(cfg, data, quiet, checkpoint_dir=ck2, resume=True, log=lines.append)
    assert "resumed at step 30" in lines
    for k in p_full:
        assert torch.allclose(p_full[k], p_res[k], atol=1e-6), k
    assert D.main(["--sample", "--checkpoint-dir", ck, "--method", "topk", "--top-k", "4", "--device", "cpu"]) == 0
