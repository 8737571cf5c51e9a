"""DType algebra: the 46 scalar types, name parsing, safetensors tags and PyTorch's promotion
rules as total functions (``None`` = PyTorch has no result).

Mirrors Tyr/Basic/Types.lean:16-199 (constructor order, ``ofString?``, ``canonicalName``,
``safeTensorFormat?``) and Tyr/Typed/DType.lean:14-279 (predicates, ``bitWidth?``, ``promote?``,
``promoteScalar?`` and the result-dtype rules).  Recognising a dtype does not imply that a
backend implements arithmetic for it.
"""
from __future__ import annotations

import enum
from typing import Optional, Tuple

import torch


class DType(enum.Enum):
    UInt8 = 0
    Int8 = 1
    Int16 = 2
    Int32 = 3
    Int64 = 4
    Float16 = 5
    BFloat16 = 6
    Float32 = 7
    Float64 = 8
    Bool = 9
    Float8E4M3FN = 10
    Float8E5M2 = 11
    Complex32 = 12
    Complex64 = 13
    Complex128 = 14
    QInt8 = 15
    QUInt8 = 16
    QInt32 = 17
    QUInt4x2 = 18
    QUInt2x4 = 19
    Bits1x8 = 20
    Bits2x4 = 21
    Bits4x2 = 22
    Bits8 = 23
    Bits16 = 24
    Float8E5M2FNUZ = 25
    Float8E4M3FNUZ = 26
    UInt16 = 27
    UInt32 = 28
    UInt64 = 29
    UInt1 = 30
    UInt2 = 31
    UInt3 = 32
    UInt4 = 33
    UInt5 = 34
    UInt6 = 35
    UInt7 = 36
    Int1 = 37
    Int2 = 38
    Int3 = 39
    Int4 = 40
    Int5 = 41
    Int6 = 42
    Int7 = 43
    Float8E8M0FNU = 44
    Float4E2M1FNX2 = 45

    def __str__(self) -> str:
        return self.name

    def __repr__(self) -> str:
        return f"DType.{self.name}"

    # ---- classification -------------------------------------------------------------------
    @property
    def is_bool(self) -> bool:
        return self is DType.Bool

    @property
    def is_unsigned_integral(self) -> bool:
        return self in (DType.UInt8, DType.UInt16, DType.UInt32, DType.UInt64)

    @property
    def is_signed_integral(self) -> bool:
        return self in (DType.Int8, DType.Int16, DType.Int32, DType.Int64)

    @property
    def is_integral(self) -> bool:
        return self.is_unsigned_integral or self.is_signed_integral

    @property
    def is_float8(self) -> bool:
        return self in (DType.Float8E4M3FN, DType.Float8E5M2, DType.Float8E4M3FNUZ,
                        DType.Float8E5M2FNUZ, DType.Float8E8M0FNU)

    @property
    def is_floating(self) -> bool:
        return self in (DType.Float16, DType.BFloat16, DType.Float32, DType.Float64,
                        DType.Float4E2M1FNX2) or self.is_float8

    @property
    def is_real_floating(self) -> bool:
        return self in (DType.Float16, DType.BFloat16, DType.Float32, DType.Float64)

    @property
    def is_complex(self) -> bool:
        return self in (DType.Complex32, DType.Complex64, DType.Complex128)

    @property
    def is_quantized(self) -> bool:
        return self in (DType.QInt8, DType.QUInt8, DType.QInt32, DType.QUInt4x2, DType.QUInt2x4)

    @property
    def is_bits(self) -> bool:
        return self in (DType.Bits1x8, DType.Bits2x4, DType.Bits4x2, DType.Bits8, DType.Bits16)

    @property
    def is_barebones_unsigned(self) -> bool:
        return self in (DType.UInt1, DType.UInt2, DType.UInt3, DType.UInt4, DType.UInt5, DType.UInt6,
                        DType.UInt7, DType.UInt16, DType.UInt32, DType.UInt64)

    @property
    def is_standard(self) -> bool:
        return self in _STANDARD

    @property
    def is_inexact(self) -> bool:
        return self.is_floating or self.is_complex

    @property
    def is_differentiable(self) -> bool:
        return self.is_inexact

    @property
    def is_index(self) -> bool:
        return self in (DType.UInt8, DType.Int32, DType.Int64)

    # ---- names ----------------------------------------------------------------------------
    @property
    def canonical_name(self) -> str:
        return self.name

    @staticmethod
    def of_string(raw: str) -> Optional["DType"]:
        tok = raw.lower()
        if tok.startswith("torch."):
            tok = tok[6:]
        return _NAME_TABLE.get(tok)

    @property
    def safetensor_format(self) -> Optional[Tuple[str, int]]:
        return _SAFETENSOR.get(self)

    @property
    def safetensor_tag(self) -> Optional[str]:
        f = _SAFETENSOR.get(self)
        return f[0] if f else None

    @staticmethod
    def of_safetensor_tag(tag: str) -> Optional["DType"]:
        for k, (t, _) in _SAFETENSOR.items():
            if t == tag:
                return k
        return None

    def can_represent_safetensors(self) -> bool:
        return self in _SAFETENSOR

    @property
    def bit_width(self) -> Optional[int]:
        return _BIT_WIDTH.get(self)

    # ---- result dtypes ----------------------------------------------------------------------
    @property
    def at_least_float(self) -> "DType":
        if self.is_bool or self.is_integral:
            return DType.Float32
        return self

    @property
    def to_complex(self) -> Optional["DType"]:
        return {DType.Float16: DType.Complex32, DType.Complex32: DType.Complex32,
                DType.BFloat16: DType.Complex64, DType.Float32: DType.Complex64,
                DType.Complex64: DType.Complex64, DType.Float64: DType.Complex128,
                DType.Complex128: DType.Complex128}.get(self)

    @property
    def real_result(self) -> "DType":
        return {DType.Complex32: DType.Float16, DType.Complex64: DType.Float32,
                DType.Complex128: DType.Float64}.get(self, self)

    @property
    def abs_result(self) -> "DType":
        return self.real_result

    @property
    def sum_result(self) -> "DType":
        if self.is_bool or self.is_integral:
            return DType.Int64
        return self

    @property
    def prod_result(self) -> "DType":
        return self.sum_result

    @property
    def mean_result(self) -> "DType":
        return self

    @property
    def divide_result(self) -> "DType":
        return self.at_least_float

    # ---- torch bridge ---------------------------------------------------------------------
    @property
    def torch(self) -> torch.dtype:
        t = _TO_TORCH.get(self)
        if t is None:
            raise TypeError(f"dtype {self} has no tensor representation in this PyTorch build")
        return t

    @staticmethod
    def of_torch(t: torch.dtype) -> "DType":
        try:
            return _FROM_TORCH[t]
        except KeyError:
            raise TypeError(f"unknown torch dtype {t}") from None


ALL = tuple(DType)

_STANDARD = frozenset({DType.Bool, DType.UInt8, DType.Int8, DType.Int16, DType.Int32, DType.Int64,
                       DType.Float16, DType.BFloat16, DType.Float32, DType.Float64,
                       DType.Complex32, DType.Complex64, DType.Complex128})

_SAFETENSOR = {
    DType.UInt8: ("U8", 1), DType.Int8: ("I8", 1), DType.Int16: ("I16", 2), DType.Int32: ("I32", 4),
    DType.Int64: ("I64", 8), DType.Float16: ("F16", 2), DType.BFloat16: ("BF16", 2),
    DType.Float32: ("F32", 4), DType.Float64: ("F64", 8), DType.Bool: ("BOOL", 1),
    DType.Float8E4M3FN: ("F8_E4M3", 1), DType.Float8E5M2: ("F8_E5M2", 1),
}

_ALIASES = {
    DType.UInt8: ("uint8", "byte", "u8"), DType.Int8: ("int8", "char", "i8"),
    DType.Int16: ("int16", "short", "i16"), DType.Int32: ("int32", "int", "i32"),
    DType.Int64: ("int64", "long", "i64"), DType.Float16: ("float16", "half", "f16"),
    DType.BFloat16: ("bfloat16", "bf16"), DType.Float32: ("float32", "float", "f32"),
    DType.Float64: ("float64", "double", "f64"), DType.Bool: ("bool",),
    DType.Float8E4M3FN: ("float8e4m3fn", "float8_e4m3fn", "f8_e4m3"),
    DType.Float8E5M2: ("float8e5m2", "float8_e5m2", "f8_e5m2"),
    DType.Complex32: ("complex32", "complexhalf", "chalf"),
    DType.Complex64: ("complex64", "complexfloat", "cfloat"),
    DType.Complex128: ("complex128", "complexdouble", "cdouble"),
    DType.QInt8: ("qint8",), DType.QUInt8: ("quint8",), DType.QInt32: ("qint32",),
    DType.QUInt4x2: ("quint4x2",), DType.QUInt2x4: ("quint2x4",),
    DType.Bits1x8: ("bits1x8",), DType.Bits2x4: ("bits2x4",), DType.Bits4x2: ("bits4x2",),
    DType.Bits8: ("bits8",), DType.Bits16: ("bits16",),
    DType.Float8E5M2FNUZ: ("float8e5m2fnuz", "float8_e5m2fnuz"),
    DType.Float8E4M3FNUZ: ("float8e4m3fnuz", "float8_e4m3fnuz"),
    DType.UInt16: ("uint16", "u16"), DType.UInt32: ("uint32", "u32"), DType.UInt64: ("uint64", "u64"),
    DType.UInt1: ("uint1", "bit"), DType.UInt2: ("uint2",), DType.UInt3: ("uint3",),
    DType.UInt4: ("uint4",), DType.UInt5: ("uint5",), DType.UInt6: ("uint6",), DType.UInt7: ("uint7",),
    DType.Int1: ("int1",), DType.Int2: ("int2",), DType.Int3: ("int3",), DType.Int4: ("int4",),
    DType.Int5: ("int5",), DType.Int6: ("int6",), DType.Int7: ("int7",),
    DType.Float8E8M0FNU: ("float8e8m0fnu", "float8_e8m0fnu"),
    DType.Float4E2M1FNX2: ("float4e2m1fnx2", "float4_e2m1fn_x2"),
}
_NAME_TABLE = {alias: dt for dt, aliases in _ALIASES.items() for alias in aliases}

_BIT_WIDTH = {}
for _dt, _w in (
    ((DType.Bool, DType.UInt1, DType.Int1), 1), ((DType.UInt2, DType.Int2, DType.QUInt2x4), 2),
    ((DType.UInt3, DType.Int3), 3), ((DType.UInt4, DType.Int4, DType.QUInt4x2, DType.Float4E2M1FNX2), 4),
    ((DType.UInt5, DType.Int5), 5), ((DType.UInt6, DType.Int6), 6), ((DType.UInt7, DType.Int7), 7),
    ((DType.UInt8, DType.Int8, DType.QInt8, DType.QUInt8, DType.Float8E4M3FN, DType.Float8E5M2,
      DType.Float8E4M3FNUZ, DType.Float8E5M2FNUZ, DType.Float8E8M0FNU, DType.Bits1x8, DType.Bits2x4,
      DType.Bits4x2, DType.Bits8), 8),
    ((DType.Int16, DType.UInt16, DType.Float16, DType.BFloat16, DType.Bits16), 16),
    ((DType.Int32, DType.UInt32, DType.Float32, DType.Complex32, DType.QInt32), 32),
    ((DType.Int64, DType.UInt64, DType.Float64, DType.Complex64), 64),
    ((DType.Complex128,), 128),
):
    for _d in _dt:
        _BIT_WIDTH[_d] = _w

_TO_TORCH = {}
for _name, _tname in (
    ("UInt8", "uint8"), ("Int8", "int8"), ("Int16", "int16"), ("Int32", "int32"), ("Int64", "int64"),
    ("Float16", "float16"), ("BFloat16", "bfloat16"), ("Float32", "float32"), ("Float64", "float64"),
    ("Bool", "bool"), ("Float8E4M3FN", "float8_e4m3fn"), ("Float8E5M2", "float8_e5m2"),
    ("Complex32", "complex32"), ("Complex64", "complex64"), ("Complex128", "complex128"),
    ("QInt8", "qint8"), ("QUInt8", "quint8"), ("QInt32", "qint32"), ("QUInt4x2", "quint4x2"),
    ("QUInt2x4", "quint2x4"), ("Bits1x8", "bits1x8"), ("Bits2x4", "bits2x4"), ("Bits4x2", "bits4x2"),
    ("Bits8", "bits8"), ("Bits16", "bits16"), ("Float8E5M2FNUZ", "float8_e5m2fnuz"),
    ("Float8E4M3FNUZ", "float8_e4m3fnuz"), ("UInt16", "uint16"), ("UInt32", "uint32"),
    ("UInt64", "uint64"), ("UInt1", "uint1"), ("UInt2", "uint2"), ("UInt3", "uint3"),
    ("UInt4", "uint4"), ("UInt5", "uint5"), ("UInt6", "uint6"), ("UInt7", "uint7"),
    ("Int1", "int1"), ("Int2", "int2"), ("Int3", "int3"), ("Int4", "int4"), ("Int5", "int5"),
    ("Int6", "int6"), ("Int7", "int7"), ("Float8E8M0FNU", "float8_e8m0fnu"),
    ("Float4E2M1FNX2", "float4_e2m1fn_x2"),
):
    _t = getattr(torch, _tname, None)
    if isinstance(_t, torch.dtype):
        _TO_TORCH[DType[_name]] = _t
_FROM_TORCH = {v: k for k, v in _TO_TORCH.items()}


def _promote_integral(a: DType, b: DType) -> DType:
    for t in (DType.Int64, DType.Int32, DType.Int16):
        if a is t or b is t:
            return t
    if {a, b} == {DType.UInt8, DType.Int8}:
        return DType.Int16
    if a is DType.Int8 or b is DType.Int8:
        return DType.Int8
    if a is DType.UInt8 or b is DType.UInt8:
        return DType.UInt8
    return DType.Bool


def _promote_standard(a: DType, b: DType) -> DType:
    s = {a, b}
    if DType.Complex128 in s:
        return DType.Complex128
    if DType.Float64 in s and (DType.Complex64 in s or DType.Complex32 in s):
        return DType.Complex128
    if DType.Complex64 in s:
        return DType.Complex64
    if DType.Complex32 in s and (DType.Float32 in s or DType.BFloat16 in s):
        return DType.Complex64
    if DType.Complex32 in s:
        return DType.Complex32
    if DType.Float64 in s:
        return DType.Float64
    if DType.Float32 in s:
        return DType.Float32
    if s == {DType.Float16, DType.BFloat16}:
        return DType.Float32
    if DType.Float16 in s:
        return DType.Float16
    if DType.BFloat16 in s:
        return DType.BFloat16
    return _promote_integral(a, b)


def promote(lhs: DType, rhs: DType) -> Optional[DType]:
    """Exact ``torch.promote_types`` for every known dtype; ``None`` where PyTorch rejects."""
    if lhs is rhs:
        return lhs
    if (lhs.is_quantized or rhs.is_quantized or lhs.is_bits or rhs.is_bits
            or lhs.is_float8 or rhs.is_float8):
        return None
    if not lhs.is_barebones_unsigned and not rhs.is_barebones_unsigned:
        if lhs.is_standard and rhs.is_standard:
            return _promote_standard(lhs, rhs)
        return None
    if lhs.is_floating:
        return lhs
    if rhs.is_floating:
        return rhs
    return None


def promote_scalar(tensor: DType, scalar: DType) -> Optional[DType]:
    """Result dtype for a dimensioned tensor combined with a zero-dimensional tensor: the
    dimensioned operand fixes the precision inside its category."""
    if tensor.is_complex:
        return tensor
    if scalar.is_complex:
        return tensor.to_complex if tensor.is_floating else scalar
    if tensor.is_floating:
        return tensor
    if tensor.is_bool or scalar.is_floating:
        return promote(tensor, scalar)
    return tensor


def real_floating(dtype: DType) -> DType:
    """Validate a runtime-selected dtype before using real floating algorithms."""
    if not dtype.is_real_floating:
        raise TypeError(f"Expected a standard real floating dtype, got {dtype}")
    return dtype


def expected_eq(expected: DType, actual: DType) -> None:
    if expected is not actual:
        raise TypeError(f"Expected dtype {expected}, got {actual}")
