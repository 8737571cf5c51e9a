"""Training engine: schedules and a few optimisation steps on CPU
(Tests/TestModdedGPT.lean, Tests/TestNorMuon*.lean style checks)."""
import math
import os

import pytest
import torch

from tyr_b200.models import nanochat as nc
from tyr_b200.train import nanochat_engine as eng


def test_lr_schedule_and_momentum():
    hp = eng.Hyperparameters(num_iterations=100, cooldown_frac=0.4)
    assert eng.get_learning_rate(0, hp, 1.0) == 1.0
    assert eng.get_learning_rate(60, hp, 1.0) == 1.0
    assert abs(eng.get_learning_rate(80, hp, 1.0) - 0.5) < 1e-9
    assert eng.get_learning_rate(100, hp, 1.0) == 0.0
    hpw = eng.Hyperparameters(num_iterations=100, warmup_frac=0.1)
    assert abs(eng.get_learning_rate(0, hpw, 1.0) - 0.1) < 1e-9
    assert eng.get_muon_momentum(0) == 0.85 and eng.get_muon_momentum(300) == 0.95
    assert abs(eng.get_muon_momentum(150) - 0.90) < 1e-9
    assert eng.get_batch_size(0) == 8 and eng.get_batch_size(999) == 16 and eng.get_batch_size(1000) == 24
    assert eng.get_window_sizes(1500) == (3, 11)


def test_grad_accum_rules():
    hp = eng.Hyperparameters()
    assert eng.effective_grad_accum_steps(hp, 8) == 1
    assert eng.effective_grad_accum_steps(hp, 1) == 8
    eng.validate_grad_accum_config(hp, 8)
    bad = eng.Hyperparameters(total_batch_size_tokens=524288 + 1)
    try:
        eng.validate_grad_accum_config(bad, 8)
        assert False
    except ValueError:
        pass
    assert abs(eng.d_model_lr_scale(nc.depth_config(20)) - (1280 / 768) ** -0.5) < 1e-12
    assert eng.aspect_ratio_scale((5120, 1280)) == 2.0 and eng.aspect_ratio_scale((1280, 5120)) == 1.0


def test_training_reduces_loss_cpu():
    cfg = nc.Config(vocab_size=64, n_layer=3, n_head=2, half_head_dim=16, max_seq_len=16)
    hp = eng.Hyperparameters(num_iterations=50, device_batch_size=4, max_seq_len=16,
                             total_batch_size_tokens=64)
    tr = eng.NanoChatTrainer(cfg, hp, device="cpu", compute_dtype=torch.float32, seed=0, ce_chunk_rows=32)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, 64, (4, 17), generator=g)
    losses = []
    for _ in range(12):
        losses.append(tr.train_step_from_host(tok))
    assert all(math.isfinite(l) for l in losses)
    assert losses[-1] < losses[0] - 0.3, losses
    assert tr.step_index == 12
    sd = tr.optimizer_state_dict()
    assert int(sd["adam.embed.step"][0]) == 12
    # the zero-initialised projections must have moved (Muon update applied)
    assert tr.params.master["attn_w"][:, 3].abs().sum() > 0
    assert tr.params.master["mlp_w"][:, 1].abs().sum() > 0


def test_restated_reference_arm_steps_on_cpu():
    """The comparison arm (library ops only, fp32 as the reference trains) takes steps and lowers the loss on a repeated batch."""
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from baseline.restated_reference import RestatedTrainer
    cfg = nc.Config(vocab_size=256, n_layer=4, n_head=2, half_head_dim=8, max_seq_len=32)
    hp = eng.Hyperparameters(device_batch_size=2, max_seq_len=32, total_batch_size_tokens=64)
    tr = RestatedTrainer(cfg, hp, device="cpu", precision="fp32")
    tok = torch.randint(0, 256, (2, 33), generator=torch.Generator().manual_seed(0))
    losses = [float(tr.step([(tok[:, :-1], tok[:, 1:])]).loss) for _ in range(4)]
    assert all(l == l for l in losses) and losses[-1] < losses[0]
    with pytest.raises(ValueError):
        RestatedTrainer(cfg, hp, device="cpu", precision="fp16")
