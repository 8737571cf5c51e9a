"""SafeTensors validation, sharded index safety, checkpoint snapshot protocol, media writers
(Tests/TestCheckpointPersistence.lean:13-152, safetensors fixtures single/sharded/provider_errors)."""
import json
import os
import struct

import pytest
import torch

from tyr_b200.io import checkpoint as ck
from tyr_b200.io import hub, media
from tyr_b200.io import safetensors as st
from tyr_b200.struct import Frozen, Static, tensor_struct
from tyr_b200.typed import DType


def test_roundtrip_and_typed_loads(tmp_path):
    p = str(tmp_path / "a.safetensors")
    t = {"w.0": torch.randn(3, 4), "b": torch.arange(5, dtype=torch.int64), "h": torch.randn(2, 2).bfloat16()}
    st.save_file(t, p, {"k": "v"})
    src = st.Source.open(p)
    assert src.names() == ["b", "h", "w.0"]
    for k, v in t.items():
        assert torch.equal(src.load(k), v)
    assert src.spec("h") == ((2, 2), DType.BFloat16)
    with pytest.raises(ValueError):
        src.load_as("w.0", (4, 3), DType.Float32)
    with pytest.raises(TypeError):
        src.load_as("w.0", (3, 4), DType.Float64)
    W = st.safetensors_type_provider(p, "W")
    assert torch.equal(W.load_w_0(), t["w.0"]) and W.tree()["w"]["0"] == "w.0"


def _write_raw(path, header: dict, data: bytes):
    hb = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)) + hb + data)


def test_header_validation(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    _write_raw(p, {"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 4)
    with pytest.raises(st.SafeTensorsError, match="truncated"):
        st.read_header(p)
    _write_raw(p, {"x": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(st.SafeTensorsError, match="size mismatch"):
        st.read_header(p)
    _write_raw(p, {"x": {"dtype": "Q9", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(st.SafeTensorsError, match="unsupported dtype"):
        st.read_header(p)
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", 1 << 40))
    with pytest.raises(st.SafeTensorsError, match="limit"):
        st.read_header(p)
    with open(p, "wb") as f:
        f.write(b"\1\2")
    with pytest.raises(st.SafeTensorsError, match="8-byte"):
        st.read_header(p)


def test_sharded_index_and_path_traversal(tmp_path):
    d = tmp_path / "model"
    d.mkdir()
    st.save_file({"a": torch.ones(2)}, str(d / "m-1.safetensors"))
    st.save_file({"b": torch.zeros(3)}, str(d / "m-2.safetensors"))
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "m-1.safetensors", "b": "m-2.safetensors"}}))
    src = st.Source.open(str(d))
    assert torch.equal(src.load("a"), torch.ones(2)) and torch.equal(src.load("b"), torch.zeros(3))
    assert hub.shard_files(str(d)) == ["m-1.safetensors", "m-2.safetensors"]
    st.clear_caches()
    for bad in ("../x.safetensors", "/abs.safetensors", "c:\\x.safetensors", "./m-1.safetensors", "m-1.bin"):
        (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": bad}}))
        with pytest.raises(st.SafeTensorsError):
            st.open_model_dir(str(d))
        st.clear_caches()


@tensor_struct
class Tiny:
    w: torch.Tensor
    f: Frozen
    cfg: Static


def test_checkpoint_snapshot_protocol(tmp_path):
    root = str(tmp_path / "ckpt")
    os.makedirs(root)
    assert not ck.has_checkpoint(root)
    tree = Tiny(torch.randn(2, 3), Frozen(torch.arange(4)), Static({"a": 1}))
    ck.save_training_checkpoint(root, tree, None, None, ck.CheckpointMeta.with_loss(7, 1.25))
    first = ck.resolve_snapshot(root)
    # an interrupted save: snapshot written but never published -> readers still see the first one
    snap = ck.begin_snapshot(root)
    ck.save_tree(snap, "param", Tiny(torch.zeros(2, 3), Frozen(torch.arange(4)), Static(None)))
    assert ck.resolve_snapshot(root) == first
    got, _, _, meta = ck.load_training_checkpoint(root, tree)
    assert torch.equal(got.w, tree.w) and meta.step == 7 and meta.loss == 1.25
    # count / shape / dtype mismatches are rejected
    with pytest.raises(ck.CheckpointError, match="shape"):
        ck.load_tree(first, "param", Tiny(torch.zeros(3, 2), Frozen(torch.arange(4)), Static(None)))
    with pytest.raises(ck.CheckpointError, match="dtype"):
        ck.load_tree(first, "param", Tiny(torch.zeros(2, 3).double(), Frozen(torch.arange(4)), Static(None)))
    with open(os.path.join(first, "param_count.txt"), "w") as f:
        f.write("9\n")
    with pytest.raises(ck.CheckpointError, match="holds 9"):
        ck.load_tree(first, "param", tree)
    # pointer that escapes the root is refused
    with open(os.path.join(root, ck.CURRENT), "w") as f:
        f.write("../elsewhere\n")
    with pytest.raises(ck.CheckpointError):
        ck.resolve_snapshot(root)


def test_checkpoint_on_disk_forms_match_the_reference(tmp_path):
    """Pointer = bare snapshot name, meta.txt = version-2 JSON with loss bits, flat directories, legacy key=value
    metadata, a second pointer for optimizer state, and removal of a snapshot whose save failed
    (Tyr/Checkpoint.lean:42-157)."""
    import json
    import struct as _struct
    root = str(tmp_path / "ckpt")
    os.makedirs(root)
    tree = Tiny(torch.randn(2, 3), Frozen(torch.arange(4)), Static(None))
    snap = ck.save_training_checkpoint(root, tree, None, None, ck.CheckpointMeta.with_loss(12, 0.75, best_val_loss=0.5, optim_count=12))
    name = open(os.path.join(root, "CURRENT")).read()
    assert name == os.path.basename(snap) and name.startswith("snapshot-") and "/" not in name and "." not in name
    j = json.load(open(os.path.join(snap, "meta.txt")))
    assert j == {"version": 2, "iteration": 12, "optimCount": 12,
                 "trainLossBits": _struct.unpack("<Q", _struct.pack("<d", 0.75))[0],
                 "bestValLossBits": _struct.unpack("<Q", _struct.pack("<d", 0.5))[0]}
    m = ck.load_meta(snap)
    assert (m.step, m.loss, m.best_val_loss, m.optim_count) == (12, 0.75, 0.5, 12)
    assert ck.has_checkpoint(root)
    # a pointer in the form earlier versions of this module wrote still resolves
    with open(os.path.join(root, "CURRENT"), "w") as f:
        f.write(".snapshots/" + name + "\n")
    assert ck.resolve_snapshot(root) == snap
    # flat legacy directory: no pointer -> the directory itself; key=value metadata
    flat = str(tmp_path / "flat")
    os.makedirs(flat)
    assert ck.resolve_snapshot(flat) == flat
    with open(os.path.join(flat, "meta.txt"), "w") as f:
        f.write("iteration=40\nbestValLoss=1.5\ntrainLoss=2.25\n")
    m = ck.load_meta(flat)
    assert (m.step, m.best_val_loss, m.loss, m.optim_count) == (40, 1.5, 2.25, 0)
    with open(os.path.join(flat, "meta.txt"), "w") as f:
        f.write("iteration=40\niteration=41\nbestValLoss=1\ntrainLoss=2\n")
    with pytest.raises(ck.CheckpointError, match="Duplicate"):
        ck.load_meta(flat)
    # a separate pointer for optimizer state
    osnap = ck.write_snapshot(root, lambda d: ck.save_tree(d, "mu", tree), pointer="OPTIMIZER_CURRENT")
    assert ck.resolve_snapshot(root, "OPTIMIZER_CURRENT") == osnap and ck.resolve_snapshot(root) == snap
    # a failed save leaves no partial snapshot behind and does not move the pointer
    before = set(os.listdir(os.path.join(root, ".snapshots")))

    def boom(d):
        ck.save_tree(d, "param", tree)
        raise RuntimeError("disk full")
    with pytest.raises(RuntimeError, match="disk full"):
        ck.write_snapshot(root, boom)
    assert set(os.listdir(os.path.join(root, ".snapshots"))) == before
    assert ck.resolve_snapshot(root) == snap
    for bad in ("snapshot-1.2", "snapshot-1/x", "other-1"):
        with open(os.path.join(root, "CURRENT"), "w") as f:
            f.write(bad)
        with pytest.raises(ck.CheckpointError):
            ck.resolve_snapshot(root)


def test_checkpoint_reads_tensor_files_written_by_libtorch_vector_save():
    """tests/fixtures/reference_pt/param_{0,1,2}.pt were written by a C++ program with the call the reference makes for
    every leaf, ``torch::save(std::vector<torch::Tensor>{t}, path)`` (cc/src/tyr.cpp:2149-2151): arange(6).reshape(2, 3)
    fp32, 0.5 * arange(4) fp32, 1.5 * ones(3, 2) bf16."""
    d = os.path.join(os.path.dirname(__file__), "fixtures", "reference_pt")

    @tensor_struct
    class Three:
        a: torch.Tensor
        b: torch.Tensor
        c: torch.Tensor
    tmpl = Three(torch.zeros(2, 3), torch.zeros(4), torch.zeros(3, 2, dtype=torch.bfloat16))
    got = ck.load_reference_pt_layout(d, "param", tmpl)
    assert torch.equal(got.a, torch.arange(6.).reshape(2, 3))
    assert torch.equal(got.b, torch.arange(4.) * 0.5)
    assert got.c.dtype == torch.bfloat16 and torch.equal(got.c.float(), torch.full((3, 2), 1.5))
    with pytest.raises(ck.CheckpointError, match="shape"):
        ck.load_reference_pt_layout(d, "param", Three(torch.zeros(3, 2), torch.zeros(4), torch.zeros(3, 2, dtype=torch.bfloat16)))
    with pytest.raises(ck.CheckpointError, match="dtype"):
        ck.load_reference_pt_layout(d, "param", Three(torch.zeros(2, 3), torch.zeros(4), torch.zeros(3, 2)))


def test_media_writers_and_float_buffer(tmp_path):
    img = torch.rand(3, 4, 5)
    p = str(tmp_path / "x.ppm")
    media.save_ppm(p, img)
    raw = open(p, "rb").read()
    assert raw.startswith(b"P6\n5 4\n255\n") and len(raw) == len(b"P6\n5 4\n255\n") + 60
    w = str(tmp_path / "x.wav")
    media.save_wav(w, torch.linspace(-1, 1, 100), 16000)
    assert os.path.getsize(w) == 44 + 200 and open(w, "rb").read(4) == b"RIFF"
    s = media.WavStream(str(tmp_path / "s.wav"), 8000)
    s.append(torch.zeros(10)); s.append(torch.ones(6)); s.finalize()
    assert struct.unpack("<I", open(str(tmp_path / "s.wav"), "rb").read()[40:44])[0] == 32
    fb = media.FloatBuffer()
    fb.append([3.0, 4.0]); fb.push(0.0)
    assert len(fb) == 3 and abs(fb.rms() - (25 / 3) ** 0.5) < 1e-6 and fb.get(1) == 4.0
    fb.keep_last(2)
    assert fb.to_tensor().tolist() == [4.0, 0.0]
    with pytest.raises(IOError, match="macOS"):
        media.load_image_patchified("x.png")


def test_hub_cache_lookup(tmp_path, monkeypatch):
    monkeypatch.setenv("HF_HUB_CACHE", str(tmp_path))
    snap = tmp_path / "models--org--name" / "snapshots" / "abc"
    snap.mkdir(parents=True)
    (tmp_path / "models--org--name" / "refs").mkdir()
    (tmp_path / "models--org--name" / "refs" / "main").write_text("abc")
    assert hub.find_cached_snapshot("org/name") == str(snap)
    assert hub.resolve_pretrained_dir("org/name", allow_download=False) == str(snap)
    with pytest.raises(hub.HubError):
        hub.resolve_pretrained_dir("org/missing", allow_download=False)
