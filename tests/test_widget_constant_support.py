"""Inspection data models (Tyr/Widget.lean) and constant-support witnesses (Tyr/ConstantSupport.lean)."""
import pytest
import torch

from tyr_b200.struct.tree import Frozen, Static, tensor_struct
from tyr_b200.typed import constant_support as cs
from tyr_b200.typed.device import Device
from tyr_b200.typed.dtype import DType
from tyr_b200.typed.tensor import Tensor
from tyr_b200.utils import widget


@tensor_struct
class Lin:
    weight: torch.Tensor
    bias: torch.Tensor
    cfg: Static


@tensor_struct
class Net:
    layers: list
    table: Frozen
    head: object


def test_module_tree_text_and_html():
    w = torch.arange(6.).reshape(2, 3).requires_grad_(True)
    w.grad = torch.ones(2, 3)
    net = Net([Lin(w, torch.zeros(2), Static({"act": "relu"})), Lin(torch.ones(2, 2), torch.zeros(2), Static(None))],
              Frozen(torch.arange(4)), None)
    props = widget.to_module_display_props(net, "net")
    root = props.root
    assert root.kind == "group" and root.name == "net: Net"
    names = [k for k, _ in root.children]
    assert names == ["layers", "table", "head"]
    layers = root.children[0][1]
    assert layers.name == "layers [2]" and [k for k, _ in layers.children] == ["[0]", "[1]"]
    t = layers.children[0][1].children[0][1].tensor
    assert t.shape == [2, 3] and t.dtype == "float32" and t.requires_grad and t.numel == 6
    assert t.values == [0.0, 1.0, 2.0, 3.0, 4.0, 5.0] and t.grad_values == [1.0] * 6
    assert "min=0" in t.stats and "max=5" in t.stats
    assert root.children[2][1].name == "head (none)"
    assert widget.count_parameters(props) == 6 + 2 + 4 + 2 + 4
    text = widget.render_text(props)
    assert "weight: float32[2, 3]" in text and "cfg = {'act': 'relu'}" in text and "table (frozen)" in text
    page = widget.render_html(props)
    assert page.startswith("<details") and "<table" in page and "18 elements" in page
    d = widget.show(net, "net")
    assert repr(d) == text and d._repr_html_() == page


def test_typed_tensor_html_repr_and_large_tensor_sampling():
    t = Tensor.of_tensor(torch.linspace(-1, 1, 12).reshape(3, 4))
    assert "float32[3, 4]" in t.describe()
    assert "<table" in t._repr_html_()
    big = widget.tensor_to_props(torch.zeros(300, 100), "big")
    assert len(big.values) == widget.MAX_VALUES and big.numel == 30000
    assert "<table" not in widget.render_html(widget.to_module_node(torch.zeros(300, 100), "big"))


def test_constant_support_static_and_runtime():
    cpu = Device.CPU
    for d in (DType.Float32, DType.Int64, DType.Bool, DType.BFloat16, DType.Float64, DType.Float8E4M3FN):
        assert cs.static_constant_support(d, cpu)
        assert cs.acquire_constant_support(d, cpu).static
    # formats outside the static table are probed: quantised dtypes cannot be built without parameters
    assert not cs.static_constant_support(DType.QInt8, cpu)
    with pytest.raises(IOError):
        cs.acquire_constant_support(DType.QInt8, cpu)
    with pytest.raises(IOError):
        cs.acquire_constant_support(DType.Bits8, cpu)
    w = cs.acquire_constant_support(DType.Float32, cpu)
    assert cs.acquire_constant_support(DType.Float32, cpu) is w
    cs.require(w, DType.Float32, cpu)
    with pytest.raises(TypeError):
        cs.require(w, DType.Float64, cpu)
    with pytest.raises(TypeError):
        cs.ConstantSupported(DType.Float32, cpu, True)


@pytest.mark.gpu
def test_constant_support_probe_on_cuda():
    dev = Device.cuda(0)
    assert not cs.static_constant_support(DType.BFloat16, dev)
    w = cs.acquire_constant_support(DType.BFloat16, dev)
    assert not w.static and w.device == dev
    assert cs.acquire_constant_support(DType.Float8E4M3FN, dev).dtype is DType.Float8E4M3FN
