"""TensorTreeCast: convert every leaf of a tree to the dtype / device of a destination tree type
(Tyr/TensorStruct/Cast.lean:19,169 and ``derive_tensor_tree_cast``).  Shape changes are rejected."""
from __future__ import annotations

from typing import Optional

import torch

from ..typed.device import Device
from ..typed.dtype import DType
from ..typed.tensor import Tensor
from .tree import tree_map, zip_with


def cast_to(tree, *, dtype: Optional[DType] = None, device: Optional[Device] = None,
            floating_only: bool = True):
    """Move a whole tree.  ``dtype`` applies to floating leaves only unless ``floating_only=False``
    (integer index tensors keep their dtype)."""
    def conv(t):
        if isinstance(t, Tensor):
            out = t
            if device is not None and out.device != device:
                out = out.to(device)
            if dtype is not None and out.dtype is not dtype and (out.dtype.is_floating or not floating_only):
                out = out.cast(dtype)
            return out
        r = t
        if device is not None:
            r = r.to(device.torch)
        if dtype is not None and (r.dtype.is_floating_point or not floating_only):
            r = r.to(dtype.torch)
        return r
    return tree_map(conv, tree)


def cast_like(tree, template):
    """Cast each leaf to the dtype and device of the corresponding leaf of ``template``; a shape
    difference is an error (the destination type fixes dtype/device only)."""
    def conv(src, dst):
        s_shape = tuple(src.shape)
        d_shape = tuple(dst.shape)
        if s_shape != d_shape:
            raise TypeError(f"castTo: shape change {list(s_shape)} -> {list(d_shape)} is not a cast")
        if isinstance(src, Tensor):
            tgt = dst if isinstance(dst, Tensor) else Tensor.of_tensor(dst)
            return src.to(tgt.device).cast(tgt.dtype)
        d = dst.raw if isinstance(dst, Tensor) else dst
        return src.to(device=d.device, dtype=d.dtype)
    return zip_with(conv, tree, template)
