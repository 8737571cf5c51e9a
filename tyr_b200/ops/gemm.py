"""bf16 GEMM on the hand-written tcgen05 kernel (csrc/gemm_tcgen05.cu) with fused epilogues,
plus the autograd `linear` built from it.

Operand layouts (no transposes are ever materialised):

* ``a_layout='K'``  : ``a`` has shape ``[..., M, K]``   (reduction dim contiguous)
* ``a_layout='MN'`` : ``a`` has shape ``[..., K, M]``   (row dim contiguous)
* ``b_layout='K'``  : ``b`` has shape ``[..., N, K]``
* ``b_layout='MN'`` : ``b`` has shape ``[..., K, N]``

``out = alpha * act(A @ B) + beta * aux`` (``act='relu2_grad'``: ``alpha * (A @ B) * 2*sqrt(aux)``); ``out_dtype`` bf16 or fp32; ``accumulate=True`` adds
into an existing fp32 ``out`` with an even stream-K split (used for weight gradients).

The reference reaches cuBLAS for these products (cc/src/tyr.cpp:1003-1036, 1267-1300) and runs
the epilogue math as separate kernels.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .._native import GemmArgs
from ._common import check, cur_stream, err_word, lib

_ACT = {None: 0, "none": 0, "relu2": 1, "relu": 2, "relu2_grad": 3, "swiglu": 4, "geglu": 5}


def _dims(t, layout, is_a):
    # returns (rows_mn, k, ld, batch, batch_stride)
    if t.dim() == 2:
        r0, r1 = t.shape
        batch, bs = 1, 0
        ld = t.stride(0)
    elif t.dim() == 3:
        batch, r0, r1 = t.shape
        bs = t.stride(0)
        ld = t.stride(1)
    else:
        raise ValueError("gemm operands must be 2-D or 3-D")
    if t.stride(-1) != 1:
        raise ValueError("gemm operands need a contiguous last dimension")
    if layout == "K":
        return r0, r1, ld, batch, bs
    return r1, r0, ld, batch, bs


def _reference(a, b, a_layout, b_layout, aux, alpha, beta, act, out_dtype):
    A = a.float() if a_layout == "K" else a.float().transpose(-1, -2)
    B = b.float().transpose(-1, -2) if b_layout == "K" else b.float()
    acc = A @ B
    if act in ("swiglu", "geglu"):
        # column blocks of 256: 128 gate columns followed by the matching 128 up columns
        N = acc.shape[-1]
        blk = acc.reshape(*acc.shape[:-1], N // 256, 2, 128)
        gate, up = alpha * blk[..., 0, :], beta * blk[..., 1, :]
        fn = torch.nn.functional.silu if act == "swiglu" else (lambda t: torch.nn.functional.gelu(t, approximate="tanh"))
        return (fn(gate) * up).reshape(*acc.shape[:-1], N // 2).to(out_dtype)
    if act == "relu2":
        acc = torch.relu(acc) ** 2
    elif act == "relu":
        acc = torch.relu(acc)
    elif act == "relu2_grad":
        # aux holds y = relu(z)^2 of the forward pass: d/dz = 2*relu(z) = 2*sqrt(y)
        return (alpha * acc * 2.0 * torch.sqrt(aux.float().clamp_min(0))).to(out_dtype)
    acc = alpha * acc
    if aux is not None and beta != 0.0:
        acc = acc + beta * aux.float()
    return acc.to(out_dtype)


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_layout: str = "K", b_layout: str = "K",
         out: Optional[torch.Tensor] = None, aux: Optional[torch.Tensor] = None,
         alpha: float = 1.0, beta: float = 0.0, act: Optional[str] = None,
         out_dtype: Optional[torch.dtype] = None, accumulate: bool = False,
         bn: int = 0, sm_count: int = 0) -> torch.Tensor:
    M, K, lda, batch_a, sA = _dims(a, a_layout, True)
    N, K2, ldb, batch_b, sB = _dims(b, b_layout, False)
    if K != K2:
        raise ValueError(f"gemm reduction mismatch: {tuple(a.shape)} ({a_layout}) vs {tuple(b.shape)} ({b_layout})")
    batch = max(batch_a, batch_b)
    if batch_a not in (1, batch) or batch_b not in (1, batch):
        raise ValueError("gemm batch mismatch")
    gated = act in ("swiglu", "geglu")
    if gated:
        # b holds, per block of 256 rows, 128 gate rows then the matching 128 up rows (`interleave_gate_up`); the result
        # is silu(alpha * gate) * (beta * up) (tanh-GELU for "geglu"), N / 2 columns wide
        if N % 256 != 0 or b_layout != "K" or aux is not None or accumulate or batch != 1:
            raise ValueError("gated gemm needs K-major b with N % 256 == 0, no aux, no accumulation, no batch")
        if beta == 0.0:
            beta = 1.0
        bn = 256
    n_out = N // 2 if gated else N
    shape = (M, n_out) if (a.dim() == 2 and b.dim() == 2) else (batch, M, n_out)
    if out_dtype is None:
        out_dtype = torch.bfloat16 if a.is_cuda else a.dtype
    if accumulate:
        if out is None or out.dtype != torch.float32:
            raise ValueError("accumulate=True needs an fp32 `out`")
        out_dtype = torch.float32
    if not a.is_cuda:
        res = _reference(a, b, a_layout, b_layout, aux, alpha, beta, act, out_dtype)
        if out is not None:
            if accumulate:
                out.add_(res.reshape(out.shape))
            else:
                out.copy_(res.reshape(out.shape))
            return out
        return res.reshape(shape)
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("tcgen05 gemm takes bf16 operands")
    if out is None:
        out = torch.empty(shape, dtype=out_dtype, device=a.device)
    elif out.dtype != out_dtype or out.stride(-1) != 1:
        raise ValueError("gemm `out` has the wrong dtype or a strided last dimension")
    args = GemmArgs()
    args.A, args.B, args.C = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.aux = aux.data_ptr() if aux is not None else None
    args.M, args.N, args.K, args.batch = M, N, K, batch
    args.lda, args.ldb = lda, ldb
    args.ldc = out.stride(-2)
    args.sA = sA if batch_a > 1 else 0
    args.sB = sB if batch_b > 1 else 0
    args.sC = out.stride(0) if out.dim() == 3 else 0
    if aux is not None:
        if aux.dtype != torch.bfloat16 or aux.stride(-1) != 1:
            raise ValueError("gemm `aux` must be bf16 with a contiguous last dimension")
        args.ldaux = aux.stride(-2)
        args.sAux = aux.stride(0) if aux.dim() == 3 else 0
    args.a_mn = 1 if a_layout == "MN" else 0
    args.b_mn = 1 if b_layout == "MN" else 0
    args.out_mode = 2 if accumulate else (0 if out_dtype == torch.bfloat16 else 1)
    args.act = _ACT[act]
    args.alpha, args.beta = alpha, beta
    args.bn, args.sm_count = bn, sm_count
    args.err = err_word(a.device).data_ptr()
    args.stream = cur_stream(a.device).value
    # batch==1 operands broadcast over the batch: the tensor map gets batch stride 0 only when
    # its batch extent is 1, so replicate through an expanded view is not needed here.
    if batch > 1 and (batch_a == 1 or batch_b == 1):
        raise ValueError("broadcast batched gemm is not supported; expand the operand")
    check(lib().tyr_gemm_bf16(ctypes.byref(args)), "tyr_gemm_bf16")
    return out


class _LinearFn(torch.autograd.Function):
    """y = act(x @ w^T); bf16 in/out; weight gradient accumulated in fp32 into ``w.main_grad``
    when the parameter carries such a buffer (the fused optimizer reads it), otherwise returned."""

    @staticmethod
    def forward(ctx, x, w, act):
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm(x2, w, a_layout="K", b_layout="K", act=act)
        ctx.save_for_backward(x2, w, y if act == "relu2" else None)
        ctx.act = act
        ctx.xshape = x.shape
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, y = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if ctx.act == "relu2":
            # y = relu(z)^2  =>  dz = dy * 2*relu(z) = dy * 2*sqrt(y)
            dy2 = relu2_bwd(dy2, y)
        elif ctx.act is not None:
            raise NotImplementedError(ctx.act)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, a_layout="K", b_layout="MN").reshape(ctx.xshape)
        dw = None
        if ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                gemm(dy2, x2, a_layout="MN", b_layout="MN", out=mg, accumulate=True)
                dw = None
                w.grad_ready = True
            else:
                dw32 = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
                gemm(dy2, x2, a_layout="MN", b_layout="MN", out=dw32, accumulate=True)
                dw = dw32.to(w.dtype)
        return dx, dw, None


def interleave_gate_up(w: torch.Tensor) -> torch.Tensor:
    """[2*M, K] weights with the M gate rows first and the M up rows second -> the row order the gated epilogue reads:
    per block of 256 rows, 128 gate rows followed by the matching 128 up rows (M % 128 == 0)."""
    M2, K = w.shape
    M = M2 // 2
    if M % 128:
        raise ValueError("interleave_gate_up needs a multiple of 128 rows per half")
    return torch.stack([w[:M].reshape(M // 128, 128, K), w[M:].reshape(M // 128, 128, K)], dim=1).reshape(M2, K).contiguous()


def relu2_bwd(dy, y):
    """dz = dy * 2*sqrt(y) for y = relu(z)^2 (elementwise, bf16)."""
    return (dy.float() * 2.0 * torch.sqrt(y.float())).to(dy.dtype)


def linear(x: torch.Tensor, w: torch.Tensor, act: Optional[str] = None) -> torch.Tensor:
    """Autograd linear ``act(x @ w^T)`` on the tcgen05 GEMM (weights ``[out, in]``)."""
    return _LinearFn.apply(x, w, act)


def grouped_gemm(a: torch.Tensor, b: torch.Tensor, group_offsets: torch.Tensor,
                 group_tiles: Optional[torch.Tensor] = None, *,
                 act: Optional[str] = None, alpha: float = 1.0, beta: float = 1.0,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Grouped (MoE) product on the tcgen05 kernel.

    ``a``: packed rows ``[total_rows, K]``; group g owns rows ``[offsets[g], offsets[g+1])`` and is
    multiplied by ``b[g]`` (``[G, N, K]``, K-major).  ``group_tiles`` (int32 ``[G+1]``, the prefix sum of
    ``ceil(rows_g / 128)``) lets the kernel walk the non-empty row tiles without a device->host read
    of the counts; it is derived on the device when not given.  ``act='swiglu'`` expects each 256-row
    block of ``b[g]`` to hold 128 gate rows followed by the matching 128 up rows and returns
    ``[total_rows, N/2]`` with ``silu(alpha*gate) * (beta*up)``; ``act='geglu'`` is the same with tanh-GELU on the gate."""
    total, K = a.shape
    G, N, K2 = b.shape
    assert K == K2 and group_offsets.numel() == G + 1
    swiglu = act in ("swiglu", "geglu")          # gated pairs: SiLU or tanh-GELU on the gate half
    n_out = N // 2 if swiglu else N
    if not a.is_cuda:
        offs = group_offsets.tolist()
        res = torch.zeros(total, n_out, dtype=a.dtype)
        for g in range(G):
            lo, hi = offs[g], offs[g + 1]
            if hi <= lo:
                continue
            acc = a[lo:hi].float() @ b[g].float().T
            if swiglu:
                blk = acc.reshape(hi - lo, N // 256, 2, 128)
                gate, up = alpha * blk[:, :, 0], beta * blk[:, :, 1]
                fn = torch.nn.functional.silu if act == "swiglu" else (lambda t: torch.nn.functional.gelu(t, approximate="tanh"))
                acc = (fn(gate) * up).reshape(hi - lo, n_out)
            else:
                acc = alpha * acc
            res[lo:hi] = acc.to(a.dtype)
        return res
    if swiglu and N % 256 != 0:
        raise ValueError("swiglu grouped gemm needs N to be a multiple of 256")
    if out is None:
        out = torch.empty((total, n_out), dtype=torch.bfloat16, device=a.device)
    args = GemmArgs()
    args.A, args.B, args.C = a.data_ptr(), b.data_ptr(), out.data_ptr()
    if group_tiles is None:
        cnt = group_offsets[1:] - group_offsets[:-1]
        group_tiles = torch.cat([torch.zeros(1, dtype=torch.int32, device=a.device),
                                 torch.cumsum((cnt + 127) // 128, 0).to(torch.int32)])
    args.M, args.N, args.K, args.batch = max(1, total), N, K, G
    args.lda, args.ldb, args.ldc = a.stride(0), b.stride(1), out.stride(0)
    args.sA, args.sB = total, b.stride(0)
    args.out_mode = 0
    args.act = (4 if act == "swiglu" else 5) if swiglu else _ACT[act]
    args.alpha = alpha
    args.beta = beta if swiglu else 0.0
    args.bn = 256
    args.err = err_word(a.device).data_ptr()
    args.stream = cur_stream(a.device).value
    args.group_offsets = group_offsets.data_ptr()
    args.group_tiles = group_tiles.data_ptr()
    check(lib().tyr_gemm_bf16(ctypes.byref(args)), "tyr_gemm_bf16(grouped)")
    return out
