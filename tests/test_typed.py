"""Typed core: dtype algebra, shape algebra, device rules, spec-checked ops
(Tests/TestShapeProofs.lean, TestTensorConstruction.lean, dtype promotion native tests)."""
import itertools

import pytest
import torch

from tyr_b200.typed import DType, Device, DeviceKind, StaticSpec, Tensor, SpecMismatch, promote, promote_scalar
from tyr_b200.typed import ops as O
from tyr_b200.typed import neural as N
from tyr_b200.typed import shape as sh
from tyr_b200.typed import dtype as dt
from tyr_b200.typed import device as dv


def test_dtype_table_has_46_members_in_reference_order():
    assert len(dt.ALL) == 46
    assert [d.name for d in dt.ALL[:12]] == ["UInt8", "Int8", "Int16", "Int32", "Int64", "Float16", "BFloat16",
                                             "Float32", "Float64", "Bool", "Float8E4M3FN", "Float8E5M2"]
    assert dt.ALL[-1] is DType.Float4E2M1FNX2


def test_dtype_names_and_safetensors_tags():
    assert DType.of_string("torch.bfloat16") is DType.BFloat16
    assert DType.of_string("Half") is DType.Float16
    assert DType.of_string("F8_E4M3") is DType.Float8E4M3FN
    assert DType.of_string("nonsense") is None
    assert DType.BFloat16.safetensor_format == ("BF16", 2)
    assert DType.Complex64.safetensor_tag is None
    assert DType.of_safetensor_tag("I64") is DType.Int64
    assert DType.Float4E2M1FNX2.bit_width == 4 and DType.Complex128.bit_width == 128
    for d in dt.ALL:
        assert DType.of_string(d.canonical_name) is d


def test_promotion_matches_torch_for_standard_types():
    std = [d for d in dt.ALL if d.is_standard]
    for a, b in itertools.product(std, std):
        assert promote(a, b).torch == torch.promote_types(a.torch, b.torch), (a, b)
    assert promote(DType.Float8E5M2, DType.Float32) is None
    assert promote(DType.QInt8, DType.QInt8) is DType.QInt8
    assert promote(DType.UInt16, DType.Float32) is DType.Float32
    assert promote(DType.UInt16, DType.Int32) is None


def test_weak_scalar_promotion_and_result_dtypes():
    assert promote_scalar(DType.Float16, DType.Float64) is DType.Float16
    assert promote_scalar(DType.Int32, DType.Float32) is DType.Float32
    assert promote_scalar(DType.Int32, DType.Int64) is DType.Int32
    assert promote_scalar(DType.Float32, DType.Complex64) is DType.Complex64
    assert promote_scalar(DType.Bool, DType.Int64) is DType.Int64
    assert DType.Int32.sum_result is DType.Int64 and DType.Float16.sum_result is DType.Float16
    assert DType.Int8.divide_result is DType.Float32 and DType.Complex64.abs_result is DType.Float32


def test_shape_algebra():
    assert sh.broadcast_shapes_opt((3, 1, 5), (4, 5)) == (3, 4, 5)
    assert sh.broadcast_shapes_opt((3, 2), (4, 5)) is None
    assert sh.matmul_shape_opt((7, 2, 3), (3, 4)) == (7, 2, 4)
    assert sh.matmul_shape_opt((3,), (3,)) == ()
    assert sh.matmul_shape_opt((2, 3), (4, 5)) is None
    assert sh.squeeze_shape((2, 1, 3), 1) == (2, 3) and sh.squeeze_shape((2, 1, 3), 0) == (2, 1, 3)
    assert sh.squeeze_shape((), 0) == ()
    assert sh.transpose_shape((2, 3, 4), 0, 2) == (4, 3, 2)
    assert sh.reduce_shape((2, 3), 1, True) == (2, 1) and sh.reduce_shape((2, 3), 1, False) == (2,)
    assert sh.cat_compatible((2, 3), (5, 3), 0) and not sh.cat_compatible((2, 3), (5, 4), 0)
    assert sh.cat_shape((2, 3), (5, 3), 0) == (7, 3)
    assert sh.is_permutation([2, 0, 1], 3) and not sh.is_permutation([0, 0, 1], 3)
    assert sh.conv2d_shape((1, 3, 32, 32), 8, (3, 3), (2, 2), (1, 1)) == (1, 8, 16, 16)
    with pytest.raises(ValueError):
        sh.validate_allocation((1 << 40, 1 << 40))


def test_device_rules():
    with pytest.raises(PermissionError):
        Device(DeviceKind.CUDA(0))
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            Device.cuda(0)
    cpu = Device.CPU
    assert dv.same_result([cpu, cpu]) == cpu
    fake = Device.of_torch(torch.device("cpu"))
    assert dv.pointwise_result(cpu, 0, fake, 2) == cpu


def test_of_raw_rejects_mismatches():
    raw = torch.zeros(2, 3)
    Tensor.of_raw(raw, StaticSpec((2, 3), DType.Float32))
    with pytest.raises(SpecMismatch, match="shape"):
        Tensor.of_raw(raw, StaticSpec((3, 2), DType.Float32), "myOp")
    with pytest.raises(SpecMismatch, match="dtype"):
        Tensor.of_raw(raw, StaticSpec((2, 3), DType.Float64))


def test_typed_ops_check_before_and_after():
    a = O.randn((4, 3))
    b = O.ones((3, 5))
    assert O.matmul(a, b).shape == (4, 5)
    with pytest.raises(TypeError, match="matmul"):
        O.matmul(a, O.ones((4, 5)))
    with pytest.raises(TypeError, match="dtype"):
        O.matmul(a, O.ones((3, 5), DType.Float64))
    assert O.add(a, O.ones((3,), DType.Float64)).dtype is DType.Float64
    assert O.add(a, O.full((), 1.0, DType.Float64)).dtype is DType.Float32  # weak scalar
    assert O.div(O.ones((2,), DType.Int32), O.ones((2,), DType.Int32)).dtype is DType.Float32
    assert O.sum_(O.ones((2, 3), DType.Int32)).dtype is DType.Int64
    with pytest.raises(TypeError):
        O.mean(O.ones((2,), DType.Int32))
    with pytest.raises(TypeError, match="reshape"):
        O.reshape(a, (5, 5))
    assert O.cat([a, a], 0).shape == (8, 3)
    with pytest.raises(TypeError, match="cat"):
        O.cat([a, b], 0)
    assert O.permute(O.ones((2, 3, 4)), [2, 0, 1]).shape == (4, 2, 3)
    v, i = O.topk(a, 2)
    assert v.shape == (4, 2) and i.dtype is DType.Int64
    with pytest.raises(ValueError, match="out of range"):
        O.cross_entropy(O.randn((2, 5)), Tensor.of_tensor(torch.tensor([1, 7])))


def test_autograd_and_linalg():
    w = O.parameter(O.randn((3, 3)))
    x = O.randn((2, 3))
    loss = O.sum_(O.mul(O.linear(x, w), O.linear(x, w)))
    O.backward_loss(loss)
    g = O.grad_of(w)
    assert g is not None and g.shape == (3, 3)
    O.zero_grad(w)
    assert O.grad_of(w) is None
    q, r = O.qr_reduced(O.randn((5, 3)))
    assert q.shape == (5, 3) and r.shape == (3, 3)
    a = O.eye(3)
    assert O.allclose(O.matrix_exp(O.matrix_log(O.mul_scalar(a, 2.0))), O.mul_scalar(a, 2.0), atol=1e-5)
    with pytest.raises(O.LinAlgError):
        O.matrix_log(O.zeros((2, 2)))


def test_sampling_filters():
    logits = Tensor.of_tensor(torch.tensor([[1.0, 3.0, 2.0, 0.5]]))
    f = O.top_k_filter(logits, 2).raw
    assert torch.isinf(f[0, 0]) and torch.isinf(f[0, 3]) and f[0, 1] == 3.0
    p = O.top_p_filter(logits, 0.6).raw
    assert p[0, 1] == 3.0 and torch.isinf(p[0, 3])


def test_neural_ops():
    x = O.randn((2, 5, 2, 8))
    cos, sin = N.rotary_freqs(5, 8, 10000.0)
    y = N.apply_rotary(x, cos, sin)
    assert y.shape == x.shape
    assert torch.allclose(y.raw[:, 0], x.raw[:, 0], atol=1e-6)  # position 0 is the identity
    n = N.rms_norm(O.randn((3, 16), DType.BFloat16))
    assert n.dtype is DType.Float32
    q = O.randn((1, 4, 6, 8)); k = O.randn((1, 2, 6, 8)); v = O.randn((1, 2, 6, 8))
    assert N.attention_gqa(q, k, v, causal=True).shape == (1, 4, 6, 8)
    with pytest.raises(TypeError, match="multiple"):
        N.attention_gqa(O.randn((1, 3, 6, 8)), k, v)
    w = N.attention_window(q, k, v, True, False, 2)
    full = N.attention_gqa(q, k, v, causal=True)
    assert torch.allclose(w.raw[:, :, :2], full.raw[:, :, :2], atol=1e-5)
    te = N.timestep_embedding(Tensor.of_tensor(torch.tensor([0.0, 0.5])), 8)
    assert te.shape == (2, 8)
