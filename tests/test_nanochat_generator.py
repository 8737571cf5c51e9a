"""NanoChat inference session parity, calculator tool, generation engine state machine."""
import pytest
import torch

from tyr_b200.models import nanochat as nc
from tyr_b200.nanochat import generator as GEN
from tyr_b200.nanochat import tools as TL
from tyr_b200.nanochat.inference import NanoChatSession
from tyr_b200.ops import rope as rope_ops


def test_calculator_parser():
    assert TL.eval_calc("2+3*4") == 14 and TL.eval_calc("(2+3)*4") == 20 and TL.eval_calc("2^3^2") == 512
    assert TL.eval_calc("-3 + 10 / 4") == -0.5 and TL.format_float(12.0) == "12" and TL.format_float(0.5) == "0.5"
    assert TL.calculator_tool.execute("144/12").output == "12"
    assert not TL.calculator_tool.execute("1/0").success and not TL.calculator_tool.can_execute("__import__('os')")
    assert not TL.calculator_tool.can_execute("2**3")
    for bad in ("2+", "(1", "1 2", "."):
        with pytest.raises(ValueError):
            TL.eval_calc(bad)
    reg = TL.ToolRegistry()
    assert reg.dispatch("6*7").output == "42" and reg.execute("nope", "1").error == "Unknown tool: nope"
    assert reg.dispatch("theorem foo").error == "Prover not yet implemented" and reg.dispatch("hello!").error == "No tool matched input"


def test_row_state_transitions():
    r = GEN.RowState.from_prompt([1, 2])
    assert r.exit_tool_block([9]) is None and r.accumulate_tool_token(3) is None      # invalid outside a tool block
    assert r.enter_tool_block("calculator") is r and r.enter_tool_block("x") is None
    r.accumulate_tool_token(5)
    r.exit_tool_block([7, 8])
    assert r.forced_tokens == [7, 8] and not r.in_tool_block and r.pop_forced_token() == 7
    bs = GEN.BatchState([r, GEN.RowState.from_prompt([4])])
    assert bs.get_next_tokens([100, 200]) == [8, 200] and bs.completed_count() == 0


def test_engine_runs_calculator_and_forces_output_tokens():
    # vocabulary: digits/operators as their ord, specials above 200
    st = GEN.SpecialTokens(eot=201, bot=202, tool_start=203, tool_end=204, output_start=205, output_end=206)
    enc = lambda s: [ord(c) for c in s]
    dec = lambda ts: "".join(chr(t) for t in ts if t < 200)
    script = [203] + enc("6*7") + [204] + [0, 0, 0, 0] + [ord("!"), 201]             # zeros are overridden by forced tokens
    calls = []

    def run_model(last):
        i = len(calls)
        calls.append(last)
        logits = torch.full((1, 256), -1e9)
        logits[0, script[min(i, len(script) - 1)]] = 0.0
        return logits
    eng = GEN.Engine(st, sampling_config=GEN.SamplingConfig(temperature=0.0, max_tokens=40))
    out = eng.generate_one([202], run_model, dec, enc)
    assert out == [202, 203] + enc("6*7") + [204, 205] + enc("42") + [206, ord("!"), 201]
    assert calls[6] == [205]                                     # the model is fed the forced tokens as well
    assert eng.generate_text("", lambda last: run_model(last), dec, enc) is not None


def test_sampling_config_filters():
    logits = torch.tensor([[0.0, 3.0, 2.9, -5.0]])
    g = torch.Generator().manual_seed(0)
    draws = {GEN.sample_with_config(logits, GEN.SamplingConfig(temperature=1.0, top_p=0.9, top_k=2), g)[0] for _ in range(40)}
    assert draws <= {1, 2} and GEN.sample_with_config(logits, GEN.SamplingConfig(temperature=0.0))[0] == 1


def test_cached_session_matches_full_forward():
    cfg = nc.Config(vocab_size=64, n_layer=7, n_head=2, half_head_dim=8, max_seq_len=16)
    params = nc.ModdedGPTParams(cfg, device="cpu", compute_dtype=torch.float32, seed=3)
    p = params.named_parameters()
    # training init zeroes the output projections; perturb so that attention and MLP matter
    g = torch.Generator().manual_seed(1)
    p = {k: (v + 0.02 * torch.randn(v.shape, generator=g)).float() if v.is_floating_point() else v for k, v in p.items()}
    ids = torch.randint(0, 64, (2, 16))
    cos, sin = rope_ops.rotary_freqs(16, cfg.head_dim, cfg.rope_base)
    full = nc.forward_reference(p, cfg, ids, cos, sin).float()
    s = NanoChatSession(p, cfg, 2, 16)
    assert torch.allclose(s.prefill(ids[:, :9]), full[:, 8], atol=1e-4)
    for t in range(9, 16):
        assert torch.allclose(s.step(ids[:, t]), full[:, t], atol=1e-4), t
