"""The static gates of ci/run.py: they pass on the tree and they catch what they are meant to catch."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ci():
    spec = importlib.util.spec_from_file_location("ci_run", os.path.join(ROOT, "ci", "run.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def test_source_gates_pass_on_the_tree():
    res = _ci().stage_gates()
    assert res["rc"] == 0, res["tail"]


def test_gate_patterns_catch_closed_calls_and_shared_bulk_loads():
    ci = _ci()
    bad = {
        "batched memcpy": "cudaMemcpyBatch" + "Async(dst, src, n, stream);",
        "bulk load shared by several CTAs": "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes." + "multi" + "cast" + "::" + "cluster [%0]",
        "GPU clock / power setting": "nvidia-smi " + "-lgc 1500",
        "device-side trap": "if (bad) __tr" + "ap();",
    }
    for what, rx in ci.FORBIDDEN:
        assert rx.search(bad[what]), what
    ok = "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];  cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global"
    for _, rx in ci.FORBIDDEN:
        assert not rx.search(ok)
