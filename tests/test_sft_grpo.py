"""ChatSFT and GRPO on a toy bigram policy: masked loss algebra, accumulation count, learning actually happens."""
import pytest
import torch

from tyr_b200.data import task as T
from tyr_b200.data import tasks as TS
from tyr_b200.rl import grpo as G
from tyr_b200.train import chat_sft as S
from tyr_b200.train import run_ledger as RL

V = 32


def bigram_forward(params, inputs):
    return params["table"][inputs]                       # [B, S, V]


def test_masked_ce_and_batch_shift():
    logits = torch.randn(2, 3, V)
    targets = torch.randint(0, V, (2, 3))
    mask = torch.tensor([[1.0, 0, 1], [0, 0, 0]])
    ref = torch.nn.functional.cross_entropy(logits[0, [0, 2]], targets[0, [0, 2]])
    assert torch.allclose(S.masked_cross_entropy(logits, targets, mask), ref, atol=1e-6)
    assert S.masked_cross_entropy(logits, targets, torch.zeros(2, 3)).item() == 0.0
    cb = T.collate([T.TokenizedConversation([1, 2, 3, 4], [0, 0, 1, 1], T.Conversation())], 8)
    b = S.SFTBatch.of_conversation_batch(cb)
    assert b.inputs.tolist() == [[1, 2, 3]] and b.targets.tolist() == [[2, 3, 4]] and b.mask.tolist() == [[0, 1, 1]] and b.num_valid_tokens == 2
    assert S.SFTConfig(device_batch_size=4, target_examples_per_step=32).grad_accum_steps(2) == 4
    with pytest.raises(ValueError, match="smaller than"):
        S.SFTConfig(device_batch_size=8, target_examples_per_step=8).grad_accum_steps(2)
    assert S.linear_lr_multiplier(5, 10) == 0.5


def test_sft_learns_assistant_tokens_and_logs(tmp_path):
    ct = T.ChatTokens(1, 2, 3, 4, 5, 6, 7, output_start=8, output_end=9)
    enc = lambda s: [10 + ord(c) % 20 for c in s]
    mix = TS.create_sft_mixture("tyr").to_conversation_mixture()
    cfg = S.SFTConfig(num_iterations=30, device_batch_size=4, target_examples_per_step=8, embedding_lr=1.0, init_lr_frac=0.2,
                      max_seq_len=64, eval_every=10, eval_steps=2, log_interval=5)
    params = {"table": torch.zeros(V, V)}
    art = RL.RunArtifacts.of_base_dir(str(tmp_path))
    RL.prepare(art, cfg)
    losses = []
    cb = S.artifact_callbacks(art).combine(S.Callbacks(on_train_step=lambda s, l, m, n: losses.append(l)))
    it = T.TaskIterator(mix, 4, 64, ct, enc)
    p, _, st = S.train_sft(cfg, params, bigram_forward, it, T.TaskIterator(mix, 4, 64, ct, enc), cb)
    assert losses[-1] < losses[0] * 0.8 and st.total_tokens > 0 and st.best_val_loss < 1e9
    rows = RL.read_events(art.metrics_path)
    assert any("val_loss" in r["metrics"] for r in rows) and any("train_loss" in r["metrics"] for r in rows)
    assert not torch.equal(p["table"], torch.zeros(V, V))


def test_grpo_algebra():
    assert G.compute_advantages([1.0, 0.0, 0.0, 1.0]) == [0.5, -0.5, -0.5, 0.5] and G.compute_advantages([]) == []
    assert G.math_reward("42", "so #### 42").reward == 1.0 and G.math_reward("42", "42").reward == 0.0
    assert G.exact_match_reward(" a ", "a").reward == 1.0
    lp = torch.log(torch.tensor([[0.5, 0.25], [0.5, 0.5]]))
    loss = G.compute_pg_loss(lp, torch.tensor([1.0, -1.0]), torch.tensor([[1.0, 1.0], [1.0, 0.0]]), 2, 3)
    ref = -((lp[0].sum() - lp[1, 0]) / 3.0) / 6.0
    assert torch.allclose(loss, ref, atol=1e-6)
    rb = G.RolloutBatch([1, 2, 3], "p", [G.Sample([4, 5], "", 1.0), G.Sample([6], "", 0.0)], "x")
    b = G.prepare_batched_rollouts([rb])
    assert b.inputs.tolist() == [[1, 2, 3, 4], [1, 2, 3, 6]][0:1] + [[1, 2, 3, 0]] and b.targets[0].tolist() == [2, 3, 4, 5]
    assert b.mask.tolist() == [[0, 0, 1, 1], [0, 0, 1, 0]] and b.advantages.tolist() == [0.5, -0.5]
    pk = G.compute_pass_k([rb, G.RolloutBatch([1], "", [G.Sample([2], "", 0.0), G.Sample([2], "", 1.0)], "")], 2)
    assert pk.pass1 == 0.5 and pk.pass_k == 1.0
    assert abs(G.get_lr_multiplier(5, 10, 0.1) - 0.05) < 1e-12


def test_grpo_improves_reward_on_toy_policy():
    torch.manual_seed(0)
    params = {"table": torch.zeros(V, V)}
    good = 7

    def make_gen(p):
        def gen(prompt, cfg, seed):
            g = torch.Generator().manual_seed(seed)
            probs = torch.softmax(p["table"][prompt[-1]], -1)
            return [int(torch.multinomial(probs, 1, generator=g))]
        return gen
    decode = lambda toks: "#### 1" if toks and toks[0] == good else "#### 0"
    cfg = G.GRPOConfig(num_samples=16, examples_per_step=2, device_batch_size=16, embedding_lr=3.0, init_lr_frac=1.0, log_every=1,
                       eval_every=0, weight_decay=0.0)
    res = G.train_loop_with_updates(cfg, params, bigram_forward, make_gen, lambda s: [3], decode, [("q", "1")], 25)
    first, last = sum(r.mean_reward for r in res.history[:5]) / 5, sum(r.mean_reward for r in res.history[-5:]) / 5
    assert last > first + 0.2, (first, last)
    assert torch.softmax(res.params["table"][3], -1)[good] > 0.3
