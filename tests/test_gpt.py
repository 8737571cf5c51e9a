"""Char GPT through the typed API (Tests/TestGPTTyped.lean; BASELINE config 1 plumbing)."""
import torch

from tyr_b200.models import gpt
from tyr_b200.struct import tree as ts
from tyr_b200.train import gpt_train
from tyr_b200.typed import Tensor


def test_presets_and_param_tree():
    assert gpt.Config.nanogpt_gpu_shakespeare() == gpt.Config(65, 256, 384, 6, 6, 0.2)
    cfg = gpt.Config.tiny_shakespeare()
    p = gpt.GPTParams.init(cfg, seed=0)
    assert ts.count(p) == 4 + 13 * cfg.n_layer
    n = sum(t.raw.numel() for t in ts.leaves(p))
    assert n == 65 * 64 + 64 * 64 + 2 * (12 * 64 * 64 + 10 * 64) + 128


def test_forward_is_causal_and_weight_tied():
    cfg = gpt.Config.tiny_shakespeare()
    p = gpt.GPTParams.init(cfg, seed=1)
    x = torch.randint(0, 65, (2, 16))
    a = gpt.forward(p, Tensor.of_tensor(x)).raw
    x2 = x.clone()
    x2[:, 10:] = (x2[:, 10:] + 1) % 65
    b = gpt.forward(p, Tensor.of_tensor(x2)).raw
    assert a.shape == (2, 16, 65)
    assert torch.allclose(a[:, :10], b[:, :10], atol=1e-5) and not torch.allclose(a[:, 10:], b[:, 10:])
    gpt.loss(p, Tensor.of_tensor(x), Tensor.of_tensor(x)).raw.backward()
    assert p.wte.raw.grad is not None and p.wte.raw.grad.abs().sum() > 0   # gradient from the tied head too


def test_training_reduces_loss_and_lr_schedule():
    cfg = gpt.Config(vocab_size=16, block_size=16, n_embd=32, n_head=2, n_layer=2)
    p = gpt.GPTParams.init(cfg, seed=2)
    data = torch.arange(4000) % 16
    tc = gpt_train.TrainConfig(max_iters=40, batch_size=8, block_size=16, warmup_iters=5, lr_decay_iters=40,
                               learning_rate=3e-3)
    p, st, losses = gpt_train.train_loop(tc, p, data, generator=torch.Generator().manual_seed(0))
    assert losses[-1] < losses[0] - 0.5
    assert gpt_train.get_lr(tc, 0) == 0.0 and abs(gpt_train.get_lr(tc, 5) - 3e-3) < 1e-12
    assert gpt_train.get_lr(tc, 100) == tc.min_lr
    out = gpt.generate(p, Tensor.of_tensor(torch.zeros(1, 1, dtype=torch.int64)), 5, top_k=3)
    assert out.shape == (1, 6)
