"""Shape algebra (pure functions over tuples of ints).

Counterparts: Tyr/Basic/Types.lean:278-362 (unsqueeze/squeeze/transpose/reduce/matmul shapes),
Tyr/Typed/Spec.lean:21-147 (compatibility predicates, broadcasting, ``matmulShape?``),
Tyr/Torch.lean:35-96 (conv/pool output sizes) and Tyr/Shape/Allocation.lean:8-19.
Functions ending in ``_opt`` return ``None`` where the reference returns ``none``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

Shape = Tuple[int, ...]
INT64_MAX = (1 << 63) - 1


def shape(*dims) -> Shape:
    if len(dims) == 1 and isinstance(dims[0], (tuple, list)):
        dims = tuple(dims[0])
    out = tuple(int(d) for d in dims)
    if any(d < 0 for d in out):
        raise ValueError(f"negative extent in shape {out}")
    return out


def numel(s: Sequence[int]) -> int:
    n = 1
    for d in s:
        n *= d
    return n


def validate_allocation(s: Sequence[int]) -> None:
    """Reject extents, contiguous strides or element counts beyond int64 before any native
    constructor runs (zero-element shapes are still stride-checked)."""
    stride = 1
    for d in reversed(tuple(s)):
        if d < 0 or d > INT64_MAX:
            raise ValueError(f"shape {tuple(s)}: extent {d} is outside int64")
        if stride > INT64_MAX:
            raise ValueError(f"shape {tuple(s)}: contiguous stride exceeds int64")
        stride *= max(d, 1)
    if numel(s) > INT64_MAX:
        raise ValueError(f"shape {tuple(s)}: element count exceeds int64")


def unsqueeze_shape(s: Shape, dim: int) -> Shape:
    if not 0 <= dim <= len(s):
        raise IndexError(f"unsqueeze dim {dim} out of range for rank {len(s)}")
    return s[:dim] + (1,) + s[dim:]


def squeeze_shape(s: Shape, dim: int) -> Shape:
    if not 0 <= dim < max(1, len(s)):
        raise IndexError(f"squeeze dim {dim} out of range for rank {len(s)}")
    if len(s) == 0:
        return s
    return s[:dim] + s[dim + 1:] if s[dim] == 1 else s


def transpose_shape(s: Shape, dim0: int, dim1: int) -> Shape:
    r = max(1, len(s))
    if not (0 <= dim0 < r and 0 <= dim1 < r):
        raise IndexError(f"transpose dims ({dim0}, {dim1}) out of range for rank {len(s)}")
    if len(s) == 0:
        return s
    l = list(s)
    l[dim0], l[dim1] = l[dim1], l[dim0]
    return tuple(l)


def reduce_shape(s: Shape, dim: int, keepdim: bool) -> Shape:
    if 0 <= dim < len(s):
        return s[:dim] + ((1,) if keepdim else ()) + s[dim + 1:]
    return s


def replace_at_dim(s: Shape, dim: int, new_size: int) -> Shape:
    if 0 <= dim < len(s):
        return s[:dim] + (new_size,) + s[dim + 1:]
    return s


def unbind_shape(s: Shape, dim: int) -> Shape:
    if not 0 <= dim < len(s):
        raise IndexError(f"unbind dim {dim} out of range for rank {len(s)}")
    return s[:dim] + s[dim + 1:]


def broadcast_shapes_opt(lhs: Shape, rhs: Shape) -> Optional[Shape]:
    if len(lhs) == 0:
        return rhs
    if len(rhs) == 0:
        return lhs
    out: List[int] = []
    for off in range(max(len(lhs), len(rhs))):
        l = lhs[len(lhs) - 1 - off] if off < len(lhs) else 1
        r = rhs[len(rhs) - 1 - off] if off < len(rhs) else 1
        if l == r:
            out.append(l)
        elif l == 1:
            out.append(r)
        elif r == 1:
            out.append(l)
        else:
            return None
    return tuple(reversed(out))


def broadcast_list_opt(shapes: Sequence[Shape]) -> Optional[Shape]:
    if not shapes:
        return None
    acc = shapes[0]
    for s in shapes[1:]:
        acc = broadcast_shapes_opt(acc, s)
        if acc is None:
            return None
    return acc


def broadcasts_to(src: Shape, dst: Shape) -> bool:
    return broadcast_shapes_opt(src, dst) == dst


def matmul_shape_opt(lhs: Shape, rhs: Shape) -> Optional[Shape]:
    n1, n2 = len(lhs), len(rhs)
    if n1 == 0 or n2 == 0:
        return None
    if n1 == 1 and n2 == 1:
        return () if lhs[0] == rhs[0] else None
    if n1 == 1:
        return rhs[:-2] + (rhs[-1],) if lhs[0] == rhs[-2] else None
    if n2 == 1:
        return lhs[:-2] + (lhs[-2],) if lhs[-1] == rhs[0] else None
    if lhs[-1] != rhs[-2]:
        return None
    batch = broadcast_shapes_opt(lhs[:-2], rhs[:-2])
    if batch is None:
        return None
    return batch + (lhs[-2], rhs[-1])


def matmul_shape(lhs: Shape, rhs: Shape) -> Shape:
    out = matmul_shape_opt(lhs, rhs)
    if out is None:
        raise ValueError(f"matmul: incompatible shapes {lhs} and {rhs}")
    return out


def cat_compatible(s1: Shape, s2: Shape, dim: int) -> bool:
    return (0 <= dim < len(s1) and len(s1) == len(s2)
            and all(i == dim or a == b for i, (a, b) in enumerate(zip(s1, s2))))


def cat_shape(s1: Shape, s2: Shape, dim: int) -> Shape:
    return replace_at_dim(s1, dim, (s1[dim] if dim < len(s1) else 0) + (s2[dim] if dim < len(s2) else 0))


def gather_compatible(inp: Shape, indices: Shape, dim: int) -> bool:
    return (0 <= dim < len(inp) and len(inp) == len(indices)
            and all(i == dim or b <= a for i, (a, b) in enumerate(zip(inp, indices))))


def slice_scatter_compatible(inp: Shape, source: Shape, dim: int) -> bool:
    return (0 <= dim < len(inp) and len(inp) == len(source)
            and all(i == dim or a == b for i, (a, b) in enumerate(zip(inp, source))))


def is_permutation(perm: Sequence[int], rank: int) -> bool:
    return len(perm) == rank and all(i in perm for i in range(rank))


def permute_shape(s: Shape, perm: Sequence[int]) -> Shape:
    return tuple(s[p] if 0 <= p < len(s) else 0 for p in perm)


def conv_out_size(size: int, kernel: int, stride: int = 1, padding: int = 0, dilation: int = 1) -> int:
    return (size + 2 * padding - dilation * (kernel - 1) - 1) // stride + 1


def conv2d_shape(inp: Shape, out_channels: int, kernel: Tuple[int, int], stride=(1, 1), padding=(0, 0),
                 dilation=(1, 1)) -> Shape:
    n, _, h, w = inp
    return (n, out_channels, conv_out_size(h, kernel[0], stride[0], padding[0], dilation[0]),
            conv_out_size(w, kernel[1], stride[1], padding[1], dilation[1]))


def conv1d_shape(inp: Shape, out_channels: int, kernel: int, stride=1, padding=0, dilation=1) -> Shape:
    n, _, l = inp
    return (n, out_channels, conv_out_size(l, kernel, stride, padding, dilation))


def conv_transpose1d_out_size(size: int, kernel: int, stride: int = 1, padding: int = 0,
                              output_padding: int = 0, dilation: int = 1) -> int:
    return (size - 1) * stride - 2 * padding + dilation * (kernel - 1) + output_padding + 1


def pool2d_shape(inp: Shape, kernel: Tuple[int, int], stride=None, padding=(0, 0)) -> Shape:
    stride = stride or kernel
    n, c, h, w = inp
    return (n, c, conv_out_size(h, kernel[0], stride[0], padding[0]),
            conv_out_size(w, kernel[1], stride[1], padding[1]))
