"""Typed operations: each op computes its result ``StaticSpec`` from the operand specs BEFORE
calling torch (raising a ``TypeError``/``ValueError`` that names the op when the combination has
no result) and re-admits the native result through ``Tensor.of_raw`` afterwards.

Covers the surface of Tyr/Typed/Ops.lean (factories :46-88, arithmetic with promotion :301-427,
unary :439-531, matmul family :538-613, broadcasting variants :628-698, reductions :705-735,
shape ops :741-816, autograd :824-1018, ``rmsNormWeighted`` :1044-1056, ``TopK`` :1067, conv
:1099-1123) with the native semantics of cc/src/tyr.cpp.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from . import shape as sh
from .device import Device, pointwise_result, same_result, selection_result
from .dtype import DType, promote
from .spec import StaticSpec, TensorSpec, pointwise_dtype_opt
from .tensor import Tensor


def _fail(op: str, msg: str):
    raise TypeError(f"{op}: {msg}")


def _admit(op: str, raw: torch.Tensor, spec: StaticSpec) -> Tensor:
    return Tensor.of_raw(raw, spec, op)


# ------------------------------------------------------------------------------------------------
# factories
# ------------------------------------------------------------------------------------------------
def _factory_spec(shape, dtype: DType, device: Device) -> StaticSpec:
    s = sh.shape(shape)
    sh.validate_allocation(s)
    return StaticSpec(s, dtype, device)


def zeros(shape, dtype: DType = DType.Float32, device: Device = Device.CPU) -> Tensor:
    spec = _factory_spec(shape, dtype, device)
    return _admit("zeros", torch.zeros(spec.shape, dtype=dtype.torch, device=device.torch), spec)


def ones(shape, dtype: DType = DType.Float32, device: Device = Device.CPU) -> Tensor:
    spec = _factory_spec(shape, dtype, device)
    return _admit("ones", torch.ones(spec.shape, dtype=dtype.torch, device=device.torch), spec)


def full(shape, value, dtype: DType = DType.Float32, device: Device = Device.CPU) -> Tensor:
    spec = _factory_spec(shape, dtype, device)
    return _admit("full", torch.full(spec.shape, value, dtype=dtype.torch, device=device.torch), spec)


def randn(shape, dtype: DType = DType.Float32, device: Device = Device.CPU, requires_grad: bool = False,
          generator: Optional[torch.Generator] = None) -> Tensor:
    spec = _factory_spec(shape, dtype, device)
    raw = torch.randn(spec.shape, dtype=dtype.torch, device=device.torch, generator=generator)
    return _admit("randn", raw.requires_grad_(requires_grad), spec)


def rand(shape, dtype: DType = DType.Float32, device: Device = Device.CPU) -> Tensor:
    spec = _factory_spec(shape, dtype, device)
    return _admit("rand", torch.rand(spec.shape, dtype=dtype.torch, device=device.torch), spec)


def randint(low: int, high: int, shape, device: Device = Device.CPU) -> Tensor:
    spec = _factory_spec(shape, DType.Int64, device)
    return _admit("randint", torch.randint(low, high, spec.shape, device=device.torch), spec)


def arange(n: int, dtype: DType = DType.Int64, device: Device = Device.CPU) -> Tensor:
    spec = _factory_spec((n,), dtype, device)
    return _admit("arange", torch.arange(n, dtype=dtype.torch, device=device.torch), spec)


def eye(n: int, dtype: DType = DType.Float32, device: Device = Device.CPU) -> Tensor:
    spec = _factory_spec((n, n), dtype, device)
    return _admit("eye", torch.eye(n, dtype=dtype.torch, device=device.torch), spec)


def linspace(start: float, end: float, steps: int, device: Device = Device.CPU) -> Tensor:
    spec = _factory_spec((steps,), DType.Float32, device)
    return _admit("linspace", torch.linspace(start, end, steps, device=device.torch), spec)


def logspace(start: float, end: float, steps: int, base: float = 10.0, device: Device = Device.CPU) -> Tensor:
    spec = _factory_spec((steps,), DType.Float32, device)
    return _admit("logspace", torch.logspace(start, end, steps, base=base, device=device.torch), spec)


def zeros_like(t: Tensor) -> Tensor:
    return _admit("zerosLike", torch.zeros_like(t.raw), t.spec)


def ones_like(t: Tensor) -> Tensor:
    return _admit("onesLike", torch.ones_like(t.raw), t.spec)


def from_list(values, shape=None, dtype: DType = DType.Float32, device: Device = Device.CPU) -> Tensor:
    raw = torch.tensor(values, dtype=dtype.torch, device=device.torch)
    if shape is not None:
        raw = raw.reshape(tuple(shape))
    return Tensor.of_tensor(raw)


# ------------------------------------------------------------------------------------------------
# arithmetic
# ------------------------------------------------------------------------------------------------
def _pointwise_spec(op: str, a: Tensor, b: Tensor, division: bool = False) -> StaticSpec:
    s = sh.broadcast_shapes_opt(a.shape, b.shape)
    if s is None:
        _fail(op, f"shapes {list(a.shape)} and {list(b.shape)} do not broadcast")
    d = pointwise_dtype_opt(a.spec.tensor_spec, b.spec.tensor_spec)
    if d is None:
        _fail(op, f"no promotion between {a.dtype} and {b.dtype}")
    dev = pointwise_result(a.device, a.spec.rank, b.device, b.spec.rank)
    if dev is None:
        _fail(op, f"operands live on {a.device} and {b.device}")
    return StaticSpec(s, d.divide_result if division else d, dev)


def _binary(op: str, fn, a: Tensor, b: Tensor, division: bool = False, out_dtype: Optional[DType] = None) -> Tensor:
    spec = _pointwise_spec(op, a, b, division)
    if out_dtype is not None:
        spec = spec.with_dtype(out_dtype)
    return _admit(op, fn(a.raw, b.raw), spec)


def add(a, b): return _binary("add", torch.add, a, b)
def sub(a, b): return _binary("sub", torch.sub, a, b)
def mul(a, b): return _binary("mul", torch.mul, a, b)
def div(a, b): return _binary("div", torch.div, a, b, division=True)
def maximum(a, b): return _binary("maximum", torch.maximum, a, b)
def minimum(a, b): return _binary("minimum", torch.minimum, a, b)
def atan2(a, b): return _binary("atan2", torch.atan2, a, b)
def pow_tensor(a, b): return _binary("pow", torch.pow, a, b)

# explicit broadcasting spellings of the reference (addB, mulB, ...)
add_b, sub_b, mul_b, div_b = add, sub, mul, div


def _scalar_spec(op: str, a: Tensor, value, division: bool = False) -> StaticSpec:
    if isinstance(value, bool):
        sd = DType.Bool
    elif isinstance(value, int):
        sd = DType.Int64
    elif isinstance(value, float):
        sd = DType.Float32
    elif isinstance(value, complex):
        sd = DType.Complex64
    else:
        _fail(op, f"unsupported scalar {value!r}")
    from .dtype import promote_scalar
    d = promote_scalar(a.dtype, sd)
    if d is None:
        _fail(op, f"no promotion between {a.dtype} and a {sd} scalar")
    return a.spec.with_dtype(d.divide_result if division else d)


def add_scalar(a: Tensor, v): return _admit("addScalar", a.raw + v, _scalar_spec("addScalar", a, v))
def sub_scalar(a: Tensor, v): return _admit("subScalar", a.raw - v, _scalar_spec("subScalar", a, v))
def mul_scalar(a: Tensor, v): return _admit("mulScalar", a.raw * v, _scalar_spec("mulScalar", a, v))
def div_scalar(a: Tensor, v): return _admit("divScalar", a.raw / v, _scalar_spec("divScalar", a, v, True))
def pow_scalar(a: Tensor, v): return _admit("pow", torch.pow(a.raw, v), _scalar_spec("pow", a, v))


def clamp(a: Tensor, lo: Optional[float] = None, hi: Optional[float] = None) -> Tensor:
    return _admit("clamp", torch.clamp(a.raw, lo, hi), a.spec)


# ------------------------------------------------------------------------------------------------
# unary
# ------------------------------------------------------------------------------------------------
def _unary(op: str, fn, a: Tensor, floating_only: bool = True, out_dtype: Optional[DType] = None) -> Tensor:
    if floating_only and not a.dtype.is_inexact:
        _fail(op, f"expects a floating or complex dtype, got {a.dtype}")
    spec = a.spec if out_dtype is None else a.spec.with_dtype(out_dtype)
    return _admit(op, fn(a.raw), spec)


def neg(a): return _unary("neg", torch.neg, a, floating_only=False)
def abs_(a): return _unary("abs", torch.abs, a, floating_only=False, out_dtype=a.dtype.abs_result)
def exp(a): return _unary("exp", torch.exp, a)
def log(a): return _unary("log", torch.log, a)
def log10(a): return _unary("log10", torch.log10, a)
def sqrt(a): return _unary("sqrt", torch.sqrt, a)
def rsqrt(a): return _unary("rsqrt", torch.rsqrt, a)
def sin(a): return _unary("sin", torch.sin, a)
def cos(a): return _unary("cos", torch.cos, a)
def atan(a): return _unary("atan", torch.atan, a)
def tanh(a): return _unary("tanh", torch.tanh, a)
def floor(a): return _unary("floor", torch.floor, a)
def sigmoid(a): return _unary("sigmoid", torch.sigmoid, a)
def relu(a): return _unary("relu", torch.relu, a, floating_only=False)
def gelu(a): return _unary("gelu", F.gelu, a)
def silu(a): return _unary("silu", F.silu, a)
def elu(a): return _unary("elu", F.elu, a)
def softplus(a): return _unary("softplus", F.softplus, a)
def leaky_relu(a, slope: float = 0.01): return _unary("leakyRelu", lambda x: F.leaky_relu(x, slope), a)
def logical_not(a): return _unary("logicalNot", torch.logical_not, a, False, DType.Bool)


def softcap(a: Tensor, cap: float) -> Tensor:
    return _unary("softcap", lambda x: cap * torch.tanh(x / cap), a)


def softmax(a: Tensor, dim: int = -1) -> Tensor:
    return _unary("softmax", lambda x: torch.softmax(x, dim), a)


def log_softmax(a: Tensor, dim: int = -1) -> Tensor:
    return _unary("logSoftmax", lambda x: torch.log_softmax(x, dim), a)


def dropout(a: Tensor, p: float, training: bool = True) -> Tensor:
    return _unary("dropout", lambda x: F.dropout(x, p, training), a)


def to_float(a: Tensor) -> Tensor:
    return a.cast(DType.Float32)


def to_bfloat16(a: Tensor) -> Tensor:
    return a.cast(DType.BFloat16)


def to_long(a: Tensor) -> Tensor:
    return a.cast(DType.Int64)


# ------------------------------------------------------------------------------------------------
# comparison / logical / where
# ------------------------------------------------------------------------------------------------
def lt(a, b): return _binary("lt", torch.lt, a, b, out_dtype=DType.Bool)
def gt(a, b): return _binary("gt", torch.gt, a, b, out_dtype=DType.Bool)
def ge(a, b): return _binary("ge", torch.ge, a, b, out_dtype=DType.Bool)
def le(a, b): return _binary("le", torch.le, a, b, out_dtype=DType.Bool)
def eq(a, b): return _binary("eq", torch.eq, a, b, out_dtype=DType.Bool)
def logical_and(a, b): return _binary("logicalAnd", torch.logical_and, a, b, out_dtype=DType.Bool)
def logical_or(a, b): return _binary("logicalOr", torch.logical_or, a, b, out_dtype=DType.Bool)


def lt_scalar(a: Tensor, v): return _admit("ltScalar", a.raw < v, a.spec.with_dtype(DType.Bool))
def gt_scalar(a: Tensor, v): return _admit("gtScalar", a.raw > v, a.spec.with_dtype(DType.Bool))
def eq_scalar(a: Tensor, v): return _admit("eqScalar", a.raw == v, a.spec.with_dtype(DType.Bool))


def where(cond: Tensor, a: Tensor, b: Tensor) -> Tensor:
    if cond.dtype is not DType.Bool:
        _fail("where", f"condition must be Bool, got {cond.dtype}")
    val = _pointwise_spec("where", a, b)
    s = sh.broadcast_shapes_opt(cond.shape, val.shape)
    if s is None:
        _fail("where", f"condition shape {list(cond.shape)} does not broadcast with {list(val.shape)}")
    dev = selection_result(cond.device, a.device, a.spec.rank, b.device, b.spec.rank)
    if dev is None:
        _fail("where", "condition and operands live on different devices")
    return _admit("where", torch.where(cond.raw, a.raw, b.raw), StaticSpec(s, val.dtype, dev))


def masked_fill(a: Tensor, mask: Tensor, value) -> Tensor:
    if mask.dtype is not DType.Bool:
        _fail("maskedFill", f"mask must be Bool, got {mask.dtype}")
    if sh.broadcast_shapes_opt(a.shape, mask.shape) != a.shape:
        _fail("maskedFill", f"mask {list(mask.shape)} does not broadcast to {list(a.shape)}")
    return _admit("maskedFill", a.raw.masked_fill(mask.raw, value), a.spec)


def any_(a: Tensor) -> Tensor:
    return _admit("any", a.raw.any(), StaticSpec((), DType.Bool, a.device))


def all_(a: Tensor) -> Tensor:
    return _admit("all", a.raw.all(), StaticSpec((), DType.Bool, a.device))


def allclose(a: Tensor, b: Tensor, rtol: float = 1e-5, atol: float = 1e-8) -> bool:
    return bool(torch.allclose(a.raw, b.raw, rtol=rtol, atol=atol))


# ------------------------------------------------------------------------------------------------
# matmul family
# ------------------------------------------------------------------------------------------------
def _same_device(op: str, *ts: Tensor) -> Device:
    dev = same_result([t.device for t in ts])
    if dev is None:
        _fail(op, "operands live on different devices")
    return dev


def matmul(a: Tensor, b: Tensor) -> Tensor:
    s = sh.matmul_shape_opt(a.shape, b.shape)
    if s is None:
        _fail("matmul", f"incompatible shapes {list(a.shape)} and {list(b.shape)}")
    if a.dtype is not b.dtype:
        _fail("matmul", f"operands must share a dtype, got {a.dtype} and {b.dtype}")
    dev = _same_device("matmul", a, b)
    return _admit("matmul", torch.matmul(a.raw, b.raw), StaticSpec(s, a.dtype, dev))


def mm(a: Tensor, b: Tensor) -> Tensor:
    if a.spec.rank != 2 or b.spec.rank != 2:
        _fail("mm", "expects two matrices")
    return matmul(a, b)


def bmm(a: Tensor, b: Tensor) -> Tensor:
    if a.spec.rank != 3 or b.spec.rank != 3 or a.shape[0] != b.shape[0]:
        _fail("bmm", f"expects [b,m,k] and [b,k,n], got {list(a.shape)} and {list(b.shape)}")
    return matmul(a, b)


def bmm4d(a: Tensor, b: Tensor) -> Tensor:
    if a.spec.rank != 4 or b.spec.rank != 4 or a.shape[:2] != b.shape[:2]:
        _fail("bmm4d", f"expects [b,h,m,k] and [b,h,k,n], got {list(a.shape)} and {list(b.shape)}")
    return matmul(a, b)


def linear(x: Tensor, w: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    """x [..., in] @ w[out, in]^T (+ bias[out])."""
    if w.spec.rank != 2 or x.spec.rank < 1 or x.shape[-1] != w.shape[1]:
        _fail("linear", f"input {list(x.shape)} does not match weight {list(w.shape)}")
    if x.dtype is not w.dtype:
        _fail("linear", f"input dtype {x.dtype} differs from weight dtype {w.dtype}")
    dev = _same_device("linear", x, w, *([bias] if bias is not None else []))
    if bias is not None and bias.shape != (w.shape[0],):
        _fail("linear", f"bias {list(bias.shape)} does not match out features {w.shape[0]}")
    raw = F.linear(x.raw, w.raw, bias.raw if bias is not None else None)
    return _admit("linear", raw, StaticSpec(x.shape[:-1] + (w.shape[0],), x.dtype, dev))


def linear3d(x: Tensor, w: Tensor) -> Tensor:
    if x.spec.rank != 3:
        _fail("linear3d", f"expects [batch, seq, in], got {list(x.shape)}")
    return linear(x, w)


def affine3d(x: Tensor, w: Tensor, b: Tensor) -> Tensor:
    if x.spec.rank != 3:
        _fail("affine3d", f"expects [batch, seq, in], got {list(x.shape)}")
    return linear(x, w, b)


def matmul3d_2d(x: Tensor, w: Tensor) -> Tensor:
    """[b, s, k] @ [k, n]."""
    if x.spec.rank != 3 or w.spec.rank != 2:
        _fail("matmul3d", "expects a 3-D and a 2-D operand")
    return matmul(x, w)


# ------------------------------------------------------------------------------------------------
# reductions
# ------------------------------------------------------------------------------------------------
def sum_(a: Tensor, dim: Optional[int] = None, keepdim: bool = False) -> Tensor:
    if dim is None:
        return _admit("sum", a.raw.sum(), StaticSpec((), a.dtype.sum_result, a.device))
    if not 0 <= dim < a.spec.rank:
        _fail("sum", f"dim {dim} out of range for rank {a.spec.rank}")
    return _admit("sum", a.raw.sum(dim, keepdim), StaticSpec(sh.reduce_shape(a.shape, dim, keepdim), a.dtype.sum_result, a.device))


def mean(a: Tensor, dim: Optional[int] = None, keepdim: bool = False) -> Tensor:
    if not a.dtype.is_inexact:
        _fail("mean", f"expects a floating dtype, got {a.dtype} (convert explicitly)")
    if dim is None:
        return _admit("mean", a.raw.mean(), StaticSpec((), a.dtype, a.device))
    if not 0 <= dim < a.spec.rank:
        _fail("mean", f"dim {dim} out of range for rank {a.spec.rank}")
    return _admit("mean", a.raw.mean(dim, keepdim), StaticSpec(sh.reduce_shape(a.shape, dim, keepdim), a.dtype, a.device))


def max_all(a: Tensor) -> Tensor:
    if a.spec.numel == 0:
        _fail("maxAll", "tensor has no elements")
    return _admit("maxAll", a.raw.max(), StaticSpec((), a.dtype, a.device))


def max_dim(a: Tensor, dim: int, keepdim: bool = False) -> Tuple[Tensor, Tensor]:
    v, i = a.raw.max(dim, keepdim)
    s = sh.reduce_shape(a.shape, dim, keepdim)
    return (_admit("maxDim", v, StaticSpec(s, a.dtype, a.device)),
            _admit("maxDim", i, StaticSpec(s, DType.Int64, a.device)))


def argmax(a: Tensor, dim: int = -1) -> Tensor:
    d = dim % max(a.spec.rank, 1)
    return _admit("argmax", a.raw.argmax(d), StaticSpec(sh.reduce_shape(a.shape, d, False), DType.Int64, a.device))


def cumsum(a: Tensor, dim: int) -> Tensor:
    return _admit("cumsum", a.raw.cumsum(dim), a.spec.with_dtype(a.dtype.sum_result))


def topk(a: Tensor, k: int, dim: int = -1) -> Tuple[Tensor, Tensor]:
    d = dim % a.spec.rank
    if k > a.shape[d]:
        _fail("topk", f"k={k} exceeds extent {a.shape[d]}")
    v, i = torch.topk(a.raw, k, d)
    s = sh.replace_at_dim(a.shape, d, k)
    return _admit("topk", v, a.spec.with_shape(s)), _admit("topk", i, StaticSpec(s, DType.Int64, a.device))


# ------------------------------------------------------------------------------------------------
# shape ops
# ------------------------------------------------------------------------------------------------
def reshape(a: Tensor, shape) -> Tensor:
    s = sh.shape(shape)
    if sh.numel(s) != a.spec.numel:
        _fail("reshape", f"cannot view {list(a.shape)} ({a.spec.numel} elements) as {list(s)}")
    return _admit("reshape", a.raw.reshape(s), a.spec.with_shape(s))


def permute(a: Tensor, perm: Sequence[int]) -> Tensor:
    if not sh.is_permutation(perm, a.spec.rank):
        _fail("permute", f"{list(perm)} is not a permutation of {a.spec.rank} axes")
    return _admit("permute", a.raw.permute(*perm), a.spec.with_shape(sh.permute_shape(a.shape, perm)))


def transpose(a: Tensor, d0: int, d1: int) -> Tensor:
    s = sh.transpose_shape(a.shape, d0, d1)
    raw = a.raw if a.spec.rank == 0 else a.raw.transpose(d0, d1)
    return _admit("transpose", raw, a.spec.with_shape(s))


def transpose2d(a: Tensor) -> Tensor:
    if a.spec.rank != 2:
        _fail("transpose2d", "expects a matrix")
    return transpose(a, 0, 1)


def squeeze(a: Tensor, dim: int) -> Tensor:
    s = sh.squeeze_shape(a.shape, dim)
    return _admit("squeeze", a.raw.reshape(s), a.spec.with_shape(s))


def unsqueeze(a: Tensor, dim: int) -> Tensor:
    s = sh.unsqueeze_shape(a.shape, dim)
    return _admit("unsqueeze", a.raw.unsqueeze(dim), a.spec.with_shape(s))


def expand(a: Tensor, shape) -> Tensor:
    s = sh.shape(shape)
    if sh.broadcast_shapes_opt(a.shape, s) != s:
        _fail("expand", f"{list(a.shape)} does not broadcast to {list(s)}")
    return _admit("expand", a.raw.expand(s), a.spec.with_shape(s))


broadcast_to = expand


def slice_(a: Tensor, dim: int, start: int, length: int) -> Tensor:
    if not 0 <= dim < a.spec.rank or start + length > a.shape[dim]:
        _fail("slice", f"[{start}, {start + length}) along dim {dim} is outside {list(a.shape)}")
    return _admit("slice", a.raw.narrow(dim, start, length), a.spec.with_shape(sh.replace_at_dim(a.shape, dim, length)))


def slice_scatter(a: Tensor, src: Tensor, dim: int, start: int) -> Tensor:
    if not sh.slice_scatter_compatible(a.shape, src.shape, dim) or start + src.shape[dim] > a.shape[dim]:
        _fail("sliceScatter", f"source {list(src.shape)} does not fit {list(a.shape)} at {start} along {dim}")
    raw = torch.slice_scatter(a.raw, src.raw, dim, start, start + src.shape[dim])
    return _admit("sliceScatter", raw, a.spec)


def cat(ts: Sequence[Tensor], dim: int) -> Tensor:
    if not ts:
        _fail("cat", "empty tensor list")
    s = ts[0].shape
    for t in ts[1:]:
        if not sh.cat_compatible(s, t.shape, dim):
            _fail("cat", f"shapes {list(s)} and {list(t.shape)} do not concatenate along {dim}")
        if t.dtype is not ts[0].dtype:
            _fail("cat", f"dtypes differ: {ts[0].dtype} and {t.dtype}")
        s = sh.cat_shape(s, t.shape, dim)
    dev = _same_device("cat", *ts)
    return _admit("cat", torch.cat([t.raw for t in ts], dim), StaticSpec(s, ts[0].dtype, dev))


def stack(ts: Sequence[Tensor], dim: int = 0) -> Tensor:
    if not ts or any(t.spec != ts[0].spec for t in ts):
        _fail("stack", "expects a non-empty list of tensors with one spec")
    s = ts[0].shape[:dim] + (len(ts),) + ts[0].shape[dim:]
    return _admit("stack", torch.stack([t.raw for t in ts], dim), ts[0].spec.with_shape(s))


def unbind(a: Tensor, dim: int = 0) -> List[Tensor]:
    s = sh.unbind_shape(a.shape, dim)
    return [_admit("unbind", r, a.spec.with_shape(s)) for r in a.raw.unbind(dim)]


def gather(a: Tensor, dim: int, index: Tensor) -> Tensor:
    if not sh.gather_compatible(a.shape, index.shape, dim) or index.dtype is not DType.Int64:
        _fail("gather", f"index {list(index.shape)} ({index.dtype}) is not compatible with {list(a.shape)} along {dim}")
    return _admit("gather", torch.gather(a.raw, dim, index.raw), a.spec.with_shape(index.shape))


def index_select(a: Tensor, dim: int, index: Tensor) -> Tensor:
    if index.spec.rank != 1 or not index.dtype.is_index:
        _fail("indexSelect", "index must be a 1-D integer tensor")
    n = a.shape[dim]
    if index.spec.numel and (int(index.raw.min()) < 0 or int(index.raw.max()) >= n):
        raise IndexError(f"indexSelect: index out of range for extent {n}")
    return _admit("indexSelect", a.raw.index_select(dim, index.raw.long()),
                  a.spec.with_shape(sh.replace_at_dim(a.shape, dim, index.shape[0])))


def embedding(index: Tensor, table: Tensor) -> Tensor:
    if table.spec.rank != 2 or not index.dtype.is_index:
        _fail("embedding", "expects an integer index and a [vocab, dim] table")
    return _admit("embedding", F.embedding(index.raw.long(), table.raw),
                  StaticSpec(index.shape + (table.shape[1],), table.dtype, table.device))


def scatter_add(a: Tensor, dim: int, index: Tensor, src: Tensor) -> Tensor:
    return _admit("scatterAdd", a.raw.scatter_add(dim, index.raw, src.raw), a.spec)


# ------------------------------------------------------------------------------------------------
# losses, norms
# ------------------------------------------------------------------------------------------------
def _validate_targets(op: str, targets: Tensor, classes: int):
    """Label-range validation before the device kernel (cc/src/tyr.cpp:971-984)."""
    if targets.spec.numel:
        lo, hi = int(targets.raw.min()), int(targets.raw.max())
        if lo < 0 or hi >= classes:
            raise ValueError(f"{op}: target label out of range [0, {classes}): min {lo}, max {hi}")


def cross_entropy(logits: Tensor, targets: Tensor) -> Tensor:
    if logits.spec.rank != 2 or targets.shape != (logits.shape[0],) or targets.dtype is not DType.Int64:
        _fail("crossEntropy", f"expects [n, classes] logits and Int64 [n] targets, got {list(logits.shape)} / {list(targets.shape)}")
    _validate_targets("crossEntropy", targets, logits.shape[1])
    return _admit("crossEntropy", F.cross_entropy(logits.raw, targets.raw), StaticSpec((), logits.dtype, logits.device))


def cross_entropy_none(logits: Tensor, targets: Tensor) -> Tensor:
    _validate_targets("crossEntropyNone", targets, logits.shape[1])
    return _admit("crossEntropyNone", F.cross_entropy(logits.raw, targets.raw, reduction="none"),
                  StaticSpec((logits.shape[0],), logits.dtype, logits.device))


def layer_norm(x: Tensor, weight: Optional[Tensor], bias: Optional[Tensor], eps: float = 1e-5) -> Tensor:
    d = x.shape[-1]
    raw = F.layer_norm(x.raw, (d,), weight.raw if weight is not None else None,
                       bias.raw if bias is not None else None, eps)
    return _admit("layerNorm", raw, x.spec)


def group_norm(x: Tensor, groups: int, weight: Optional[Tensor], bias: Optional[Tensor], eps: float = 1e-5) -> Tensor:
    raw = F.group_norm(x.raw, groups, weight.raw if weight is not None else None,
                       bias.raw if bias is not None else None, eps)
    return _admit("groupNorm", raw, x.spec)


# ------------------------------------------------------------------------------------------------
# autograd
# ------------------------------------------------------------------------------------------------
def parameter(t: Tensor) -> Tensor:
    """A fresh leaf that requires grad."""
    return _admit("parameter", t.raw.detach().clone().requires_grad_(True), t.spec)


def set_requires_grad(t: Tensor, flag: bool) -> Tensor:
    return _admit("setRequiresGrad", t.raw.detach().requires_grad_(flag), t.spec)


def detach(t: Tensor) -> Tensor:
    return _admit("detach", t.raw.detach(), t.spec)


def requires_grad(t: Tensor) -> bool:
    return t.raw.requires_grad


def is_leaf(t: Tensor) -> bool:
    return t.raw.is_leaf


def has_grad_fn(t: Tensor) -> bool:
    return t.raw.grad_fn is not None


def backward_loss(loss: Tensor) -> None:
    if loss.spec.numel != 1:
        _fail("backwardLoss", f"loss must be a single element, got {list(loss.shape)}")
    loss.raw.backward()


def backward(t: Tensor, grad: Tensor) -> None:
    if grad.shape != t.shape:
        _fail("backward", f"gradient {list(grad.shape)} does not match {list(t.shape)}")
    t.raw.backward(grad.raw)


def grad_of(t: Tensor) -> Optional[Tensor]:
    g = t.raw.grad
    return None if g is None else _admit("gradOf", g, t.spec)


def zero_grad(t: Tensor) -> None:
    t.raw.grad = None


def grad(output: Tensor, inputs: Sequence[Tensor], grad_output: Optional[Tensor] = None) -> List[Tensor]:
    """One engine call for many inputs (``tensor_grad_many``, cc/src/tyr.cpp:789)."""
    go = grad_output.raw if grad_output is not None else None
    gs = torch.autograd.grad(output.raw, [i.raw for i in inputs], go, allow_unused=True)
    return [_admit("grad", g if g is not None else torch.zeros_like(i.raw), i.spec) for g, i in zip(gs, inputs)]


def clip_grad_norm_(t: Tensor, max_norm: float) -> float:
    if t.raw.grad is None:
        return 0.0
    return float(torch.nn.utils.clip_grad_norm_([t.raw], max_norm))


# ------------------------------------------------------------------------------------------------
# conv / pooling
# ------------------------------------------------------------------------------------------------
def conv2d(x: Tensor, w: Tensor, bias: Optional[Tensor] = None, stride=(1, 1), padding=(0, 0), dilation=(1, 1),
           groups: int = 1) -> Tensor:
    if x.spec.rank != 4 or w.spec.rank != 4 or x.shape[1] != w.shape[1] * groups:
        _fail("conv2d", f"input {list(x.shape)} does not match weight {list(w.shape)} (groups {groups})")
    s = sh.conv2d_shape(x.shape, w.shape[0], (w.shape[2], w.shape[3]), stride, padding, dilation)
    raw = F.conv2d(x.raw, w.raw, bias.raw if bias is not None else None, stride, padding, dilation, groups)
    return _admit("conv2d", raw, x.spec.with_shape(s))


def conv1d(x: Tensor, w: Tensor, bias: Optional[Tensor] = None, stride: int = 1, padding: int = 0,
           dilation: int = 1, groups: int = 1) -> Tensor:
    if x.spec.rank != 3 or w.spec.rank != 3 or x.shape[1] != w.shape[1] * groups:
        _fail("conv1d", f"input {list(x.shape)} does not match weight {list(w.shape)} (groups {groups})")
    s = sh.conv1d_shape(x.shape, w.shape[0], w.shape[2], stride, padding, dilation)
    raw = F.conv1d(x.raw, w.raw, bias.raw if bias is not None else None, stride, padding, dilation, groups)
    return _admit("conv1d", raw, x.spec.with_shape(s))


def conv_transpose1d(x: Tensor, w: Tensor, bias: Optional[Tensor] = None, stride: int = 1, padding: int = 0,
                     output_padding: int = 0, dilation: int = 1) -> Tensor:
    l = sh.conv_transpose1d_out_size(x.shape[2], w.shape[2], stride, padding, output_padding, dilation)
    raw = F.conv_transpose1d(x.raw, w.raw, bias.raw if bias is not None else None, stride, padding,
                             output_padding, 1, dilation)
    return _admit("convTranspose1d", raw, x.spec.with_shape((x.shape[0], w.shape[1], l)))


def avg_pool2d(x: Tensor, kernel, stride=None, padding=(0, 0)) -> Tensor:
    s = sh.pool2d_shape(x.shape, kernel, stride, padding)
    return _admit("avgPool2d", F.avg_pool2d(x.raw, kernel, stride, padding), x.spec.with_shape(s))


def interpolate_nearest(x: Tensor, scale: int) -> Tensor:
    s = x.shape[:2] + tuple(d * scale for d in x.shape[2:])
    return _admit("interpolate", F.interpolate(x.raw, scale_factor=scale, mode="nearest"), x.spec.with_shape(s))


# ------------------------------------------------------------------------------------------------
# linear algebra
# ------------------------------------------------------------------------------------------------
class LinAlgError(ValueError):
    pass


def qr_reduced(a: Tensor) -> Tuple[Tensor, Tensor]:
    m, n = a.shape[-2:]
    k = min(m, n)
    q, r = torch.linalg.qr(a.raw, mode="reduced")
    return (_admit("qrReduced", q, a.spec.with_shape(a.shape[:-2] + (m, k))),
            _admit("qrReduced", r, a.spec.with_shape(a.shape[:-2] + (k, n))))


def qr_complete(a: Tensor) -> Tuple[Tensor, Tensor]:
    m, n = a.shape[-2:]
    q, r = torch.linalg.qr(a.raw, mode="complete")
    return (_admit("qr", q, a.spec.with_shape(a.shape[:-2] + (m, m))),
            _admit("qr", r, a.spec.with_shape(a.shape[:-2] + (m, n))))


def svd_reduced(a: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
    m, n = a.shape[-2:]
    k = min(m, n)
    try:
        u, s, vh = torch.linalg.svd(a.raw, full_matrices=False)
    except RuntimeError as e:
        raise LinAlgError(f"svd: {e}") from None
    b = a.shape[:-2]
    return (_admit("svd", u, a.spec.with_shape(b + (m, k))),
            _admit("svd", s, a.spec.with_shape(b + (k,)).with_dtype(a.dtype.real_result)),
            _admit("svd", vh, a.spec.with_shape(b + (k, n))))


def svdvals(a: Tensor) -> Tensor:
    k = min(a.shape[-2:])
    return _admit("svdvals", torch.linalg.svdvals(a.raw), a.spec.with_shape(a.shape[:-2] + (k,)).with_dtype(a.dtype.real_result))


def matrix_exp(a: Tensor) -> Tensor:
    return _admit("matrixExp", torch.linalg.matrix_exp(a.raw), a.spec)


def matrix_log(a: Tensor) -> Tensor:
    """Principal logarithm through an eigen-decomposition, checked: raises ``LinAlgError`` when the
    matrix is singular / defective or the result is not real (cc/src/tyr.cpp:3600-3639)."""
    w, v = torch.linalg.eig(a.raw.to(torch.float64))
    if (w.abs() < 1e-12).any():
        raise LinAlgError("matrixLog: singular matrix has no logarithm")
    try:
        vinv = torch.linalg.inv(v)
    except RuntimeError:
        raise LinAlgError("matrixLog: defective matrix (eigenvectors not invertible)") from None
    res = v @ torch.diag_embed(torch.log(w)) @ vinv
    if res.imag.abs().max() > 1e-8 * max(1.0, float(res.real.abs().max())):
        raise LinAlgError("matrixLog: logarithm is not real")
    return _admit("matrixLog", res.real.to(a.raw.dtype), a.spec)


def inv(a: Tensor) -> Tensor:
    try:
        return _admit("inv", torch.linalg.inv(a.raw), a.spec)
    except RuntimeError as e:
        raise LinAlgError(f"inv: {e}") from None


def diag(a: Tensor) -> Tensor:
    if a.spec.rank == 1:
        n = a.shape[0]
        return _admit("diag", torch.diag(a.raw), a.spec.with_shape((n, n)))
    return _admit("diag", torch.diag(a.raw), a.spec.with_shape((min(a.shape),)))


def diagflat(a: Tensor) -> Tensor:
    n = a.spec.numel
    return _admit("diagflat", torch.diagflat(a.raw), a.spec.with_shape((n, n)))


def _scalar_real(op: str, raw: torch.Tensor, a: Tensor) -> Tensor:
    return _admit(op, raw, StaticSpec((), a.dtype.real_result, a.device))


def spectral_norm(a: Tensor) -> Tensor: return _scalar_real("spectralNorm", torch.linalg.matrix_norm(a.raw, 2), a)
def nuclear_norm(a: Tensor) -> Tensor: return _scalar_real("nuclearNorm", torch.linalg.matrix_norm(a.raw, "nuc"), a)
def frobenius_norm(a: Tensor) -> Tensor: return _scalar_real("frobeniusNorm", torch.linalg.matrix_norm(a.raw, "fro"), a)
def l2_norm(a: Tensor) -> Tensor: return _scalar_real("l2Norm", torch.linalg.vector_norm(a.raw), a)


def row_norms(a: Tensor) -> Tensor:
    return _admit("rowNorms", torch.linalg.vector_norm(a.raw, dim=-1), a.spec.with_shape(a.shape[:-1]).with_dtype(a.dtype.real_result))


def max_row_norm(a: Tensor) -> Tensor:
    return _scalar_real("maxRowNorm", torch.linalg.vector_norm(a.raw, dim=-1).max(), a)


# ------------------------------------------------------------------------------------------------
# sampling
# ------------------------------------------------------------------------------------------------
def top_k_filter(logits: Tensor, k: int) -> Tensor:
    """Keep the k largest logits per row, others -> -inf (cc/src/tyr.cpp:3469)."""
    if k <= 0 or k >= logits.shape[-1]:
        return logits
    v, _ = torch.topk(logits.raw, k, dim=-1)
    thr = v[..., -1:]
    return _admit("topkFilter", logits.raw.masked_fill(logits.raw < thr, float("-inf")), logits.spec)


def top_p_filter(logits: Tensor, p: float) -> Tensor:
    """Nucleus filter: smallest prefix of the sorted distribution whose mass reaches p (:3505)."""
    if p >= 1.0:
        return logits
    sorted_logits, idx = torch.sort(logits.raw, dim=-1, descending=True)
    cum = torch.softmax(sorted_logits.float(), -1).cumsum(-1)
    remove = cum > p
    remove[..., 1:] = remove[..., :-1].clone()
    remove[..., 0] = False
    mask = torch.zeros_like(remove).scatter(-1, idx, remove)
    return _admit("toppFilter", logits.raw.masked_fill(mask, float("-inf")), logits.spec)


def multinomial(probs: Tensor, n: int = 1, generator: Optional[torch.Generator] = None) -> Tensor:
    raw = torch.multinomial(probs.raw.float(), n, generator=generator)
    return _admit("multinomial", raw, StaticSpec(probs.shape[:-1] + (n,), DType.Int64, probs.device))


# ------------------------------------------------------------------------------------------------
# runtime
# ------------------------------------------------------------------------------------------------
def manual_seed(seed: int) -> None:
    torch.manual_seed(seed)


def cuda_is_available() -> bool:
    return torch.cuda.is_available()


def cuda_synchronize() -> None:
    if torch.cuda.is_available():
        torch.cuda.synchronize()
