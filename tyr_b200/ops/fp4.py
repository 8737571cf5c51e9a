"""Block-scaled NVFP4 tensor-core path for the MoE experts (csrc/fp4_gemm.cu).

``Fp4Experts.prepare`` re-lays a checkpoint's NVFP4 banks once (values stay 4-bit; nothing is dequantised):
gate and up rows are interleaved in groups of 64 so that one 128-column tile of the first product holds matching gate /
up columns, and the UE4M3 block scales are permuted into the tensor core's 128 x 4 order.  ``moe_fp4_tc_forward`` then
runs   gather + quantise  ->  grouped FP4 GEMM with SwiGLU and re-quantisation in its epilogue  ->  grouped FP4 GEMM
-> weighted combine,  all without a host read.

The same arithmetic in plain PyTorch (``quantize_rows_ref``, ``moe_fp4_tc_reference``) is the oracle of the tests.
What the reference does on the hardware it supports: cc/src/tyr_laguna_moe.cu:612-641 (scale order), :678-728
(activation quantisation), :730-766 (SwiGLU + re-quantise), :839-982 (batched block-scaled matmul).
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .._native import register_signatures
from ._common import check, cur_stream, err_word, lib, ptr

E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


class _GemmArgs(ctypes.Structure):
    _fields_ = [("a_packed", ctypes.c_void_p), ("a_sf", ctypes.c_void_p), ("a_row_scale", ctypes.c_void_p),
                ("w_packed", ctypes.c_void_p), ("w_sf", ctypes.c_void_p), ("w_global", ctypes.c_void_p),
                ("w_global2", ctypes.c_void_p), ("group_tiles", ctypes.c_void_p), ("group_rows", ctypes.c_void_p),
                ("out", ctypes.c_void_p), ("out_sf", ctypes.c_void_p),
                ("padded_rows", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int), ("groups", ctypes.c_int),
                ("mode", ctypes.c_int), ("sm_count", ctypes.c_int), ("all_active", ctypes.c_int),
                ("err", ctypes.c_void_p), ("stream", ctypes.c_void_p)]


@register_signatures
def _sigs(lib_):
    P, I = ctypes.c_void_p, ctypes.c_int
    fn = getattr(lib_, "tyr_fp4_gather_quantize", None)
    if fn is not None:
        fn.argtypes = [P, P, P, P, P, P, P, P, P, I, I, I, I, P]
        fn.restype = I
    fn = getattr(lib_, "tyr_fp4_grouped_gemm", None)
    if fn is not None:
        fn.argtypes = [ctypes.POINTER(_GemmArgs)]
        fn.restype = I
    fn = getattr(lib_, "tyr_fp4_scatter_quantize_fixed", None)
    if fn is not None:
        fn.argtypes = [P, P, P, P, P, P, P, I, I, I, I, P, P]
        fn.restype = I


def available() -> bool:
    return hasattr(lib(), "tyr_fp4_grouped_gemm")


# ---- scale order -------------------------------------------------------------------------------------------
def swizzle_scales(sf: torch.Tensor) -> torch.Tensor:
    """[..., rows, K/16] scale bytes (rows % 128 == 0, K % 64 == 0) -> the tensor core's order, flat per leading index:
    chunk (row tile, K/64) of 512 bytes, byte (row % 32) * 16 + (row // 32 % 4) * 4 + (k // 16) % 4."""
    u = sf.view(torch.uint8) if sf.dtype != torch.uint8 else sf
    *lead, R, KB = u.shape
    if R % 128 or KB % 4:
        raise ValueError(f"scale matrix [{R}, {KB}] does not tile into 128 x 4 chunks")
    v = u.reshape(*lead, R // 128, 4, 32, KB // 4, 4)            # [tile, r // 32, r % 32, k tile, k % 4]
    n = len(lead)
    v = v.permute(*range(n), n, n + 3, n + 2, n + 1, n + 4)      # [tile, k tile, r % 32, r // 32, k % 4]
    return v.contiguous().reshape(*lead, R * KB)


def unswizzle_scales(flat: torch.Tensor, rows: int, kblocks: int) -> torch.Tensor:
    *lead, _ = flat.shape
    v = flat.reshape(*lead, rows // 128, kblocks // 4, 32, 4, 4)
    n = len(lead)
    v = v.permute(*range(n), n, n + 3, n + 2, n + 1, n + 4)
    return v.contiguous().reshape(*lead, rows, kblocks)


# ---- reference arithmetic (any device) ------------------------------------------------------------------------
def _e2m1_codes(q: torch.Tensor) -> torch.Tensor:
    a = q.abs()
    mag = torch.zeros_like(a, dtype=torch.uint8)
    for thr, strict, code in ((0.25, False, 1), (0.75, True, 2), (1.25, False, 3), (1.75, True, 4), (2.5, False, 5),
                              (3.5, True, 6), (5.0, False, 7)):
        mag = torch.where((a >= thr) if strict else (a > thr), torch.full_like(mag, code), mag)
    return mag | ((q < 0).to(torch.uint8) << 3)


def quantize_rows_ref(x: torch.Tensor, per_row_scale: bool = True):
    """bf16 / fp32 [R, K] -> (codes uint8 [R, K], block scales fp32 [R, K/16] (already UE4M3-rounded), row scale [R])
    with the arithmetic of the device kernels: row scale amax / (6 * 448) (or 1), block scale e4m3(block amax / 6 / row
    scale), codes round-to-nearest-even on the e2m1 grid."""
    xf = x.float()
    R, K = xf.shape
    g = xf.abs().amax(1) * (1.0 / (6.0 * 448.0)) if per_row_scale else torch.ones(R, device=x.device)
    g = torch.where(g > 0, g, torch.ones_like(g))
    blocks = xf.reshape(R, K // 16, 16)
    bm = blocks.abs().amax(-1)
    sb = ((bm * (1.0 / g)[:, None]) * (1.0 / 6.0)).clamp(max=448.0).to(torch.float8_e4m3fn)
    s = sb.float() * g[:, None]
    inv = torch.where(s > 0, 1.0 / s, torch.zeros_like(s))
    codes = _e2m1_codes(blocks * inv[..., None]).reshape(R, K)
    return codes, sb.float(), g


def dequant_rows_ref(codes: torch.Tensor, sb: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    vals = E2M1_VALUES.to(codes.device)[codes.long()]
    return vals * (sb * g[:, None]).repeat_interleave(16, dim=1)


def tile_weights(w: torch.Tensor) -> torch.Tensor:
    """[E, N, K/2] packed bytes (N % 128 == 0, K % 256 == 0) -> [E, N/128, K/256, 16384]: for every (128-row tile, 256-element
    stage) the 16 KB image the kernel's shared memory holds for it, i.e. rows of 128 bytes whose 16-byte chunks are XOR-ed with
    (row & 7) (the 128-byte swizzle the tensor-core descriptors expect).  The kernel then fetches a stage's weights with ONE
    contiguous bulk copy instead of a 128-row tiled copy, and DRAM sees 16 KB bursts."""
    E, N, Kb = w.shape
    if N % 128 or Kb % 128:
        raise ValueError("tile_weights: rows must be a multiple of 128 and the reduction a multiple of 256 elements")
    r = torch.arange(128, device=w.device)
    src_chunk = (torch.arange(8, device=w.device)[None, :] ^ (r[:, None] & 7))               # [128, 8]: chunk stored at (r, c')
    idx = src_chunk[None, None, None, :, :, None].expand(1, N // 128, Kb // 128, 128, 8, 16)
    out = torch.empty((E, N // 128, Kb // 128, 128 * 128), dtype=torch.uint8, device=w.device)
    for e in range(E):                                                                    # one expert at a time: bounded scratch
        t = w[e].reshape(N // 128, 128, Kb // 128, 8, 16).permute(0, 2, 1, 3, 4).unsqueeze(0)   # [1, nt, ks, r, c, 16]
        out[e] = torch.gather(t, 4, idx).reshape(N // 128, Kb // 128, 128 * 128)
    return out


# ---- prepared weights ----------------------------------------------------------------------------------------
@dataclass
class Fp4Experts:
    """NVFP4 banks in the layout of the tensor-core kernels.  ``gu_*``: gate and up rows interleaved in groups of 64
    ([E, 2 * mi, h / 2] bytes) and then cut into per-stage shared-memory images (``tile_weights``); ``dn_*``: the down bank
    ([E, h, mi / 2]) likewise.  Scales are flat per expert, tensor-core order."""
    gu_packed: torch.Tensor
    gu_sf: torch.Tensor
    gate_global: torch.Tensor
    up_global: torch.Tensor
    dn_packed: torch.Tensor
    dn_sf: torch.Tensor
    dn_global: torch.Tensor
    hidden: int
    moe_int: int

    @staticmethod
    def supported(hidden: int, moe_int: int) -> bool:
        return hidden % 256 == 0 and moe_int % 256 == 0

    @staticmethod
    def prepare(ex) -> "Fp4Experts":
        """``ex``: ops.moe.PackedExperts.  One-time permutation of bytes; the 4-bit values are not touched."""
        E, mi, h = ex.num_experts, ex.moe_int, ex.hidden
        if not Fp4Experts.supported(h, mi):
            raise ValueError(f"fp4 tensor-core path needs hidden and expert width in multiples of 256, got {h}, {mi}")

        def inter(g, u):     # [E, mi, c] x 2 -> [E, 2 mi, c], 64 gate rows then the 64 matching up rows
            c = g.shape[-1]
            return torch.stack([g.reshape(E, mi // 64, 64, c), u.reshape(E, mi // 64, 64, c)], dim=2).reshape(E, 2 * mi, c)

        u8 = lambda t: t.view(torch.uint8) if t.dtype != torch.uint8 else t
        gu_packed = tile_weights(inter(ex.gate_packed, ex.up_packed).contiguous())
        gu_sf = swizzle_scales(inter(u8(ex.gate_scale), u8(ex.up_scale)))
        return Fp4Experts(gu_packed, gu_sf.contiguous(), ex.gate_global.float().contiguous(), ex.up_global.float().contiguous(),
                          tile_weights(ex.down_packed.contiguous()), swizzle_scales(u8(ex.down_scale)).contiguous(),
                          ex.down_global.float().contiguous(), h, mi)


_prepared = {}


def prepared(ex) -> Fp4Experts:
    """Cached per bank (keyed by the storage addresses of its packed tensors)."""
    key = (ex.gate_packed.data_ptr(), ex.up_packed.data_ptr(), ex.down_packed.data_ptr(), ex.gate_packed.numel())
    hit = _prepared.get(key)
    if hit is None:
        hit = Fp4Experts.prepare(ex)
        if len(_prepared) > 512:
            _prepared.clear()
        _prepared[key] = hit
    return hit


# ---- device ops --------------------------------------------------------------------------------------------------
def gather_quantize(x: torch.Tensor, order: Optional[torch.Tensor], ids: Optional[torch.Tensor], offsets: Optional[torch.Tensor],
                    tiles: Optional[torch.Tensor], k: int, padded_rows: int, pairs: Optional[int] = None):
    """-> (packed [padded_rows, h/2] u8, scales flat u8, row_scale fp32 [padded_rows], pair_ppos int32 [pairs] | None)."""
    T, h = x.shape
    n = pairs if pairs is not None else (order.numel() if order is not None else T)
    dev = x.device
    packed = torch.empty((padded_rows, h // 2), dtype=torch.uint8, device=dev)
    sf = torch.empty(padded_rows * (h // 16), dtype=torch.uint8, device=dev)
    rs = torch.empty(padded_rows, dtype=torch.float32, device=dev)
    ppos = torch.zeros(n, dtype=torch.int32, device=dev) if order is not None else None
    E = (offsets.numel() - 1) if offsets is not None else 1
    check(lib().tyr_fp4_gather_quantize(ptr(x.contiguous()), ptr(order), ptr(ids), ptr(offsets), ptr(tiles), ptr(packed), ptr(sf),
                                        ptr(rs), ptr(ppos), n, k, h, E, cur_stream(dev)), "fp4_gather_quantize")
    return packed, sf, rs, ppos


def grouped_gemm_fp4(a_packed, a_sf, a_row_scale, w_packed, w_sf, w_global, tiles, rows, N: int, K: int, *, mode: int = 0,
                     w_global2=None, sm_count: int = 0, all_active: bool = False):
    """``w_packed``: the weights as ``tile_weights`` images.  mode 0 -> bf16 [padded_rows, N]; mode 1 -> (packed
    [padded_rows, N/4] u8, scales flat u8) of silu(gate) * up."""
    padded = a_packed.shape[0]
    dev = a_packed.device
    groups = tiles.numel() - 1 if tiles is not None else rows.numel()     # no tile table: ``rows`` are per-expert counts
    if mode == 0:
        out = torch.empty((padded, N), dtype=torch.bfloat16, device=dev)
        out_sf = None
    else:
        out = torch.empty((padded, N // 4), dtype=torch.uint8, device=dev)
        out_sf = torch.empty(padded * (N // 2 // 16), dtype=torch.uint8, device=dev)
    a = _GemmArgs()
    a.a_packed, a.a_sf, a.a_row_scale = a_packed.data_ptr(), a_sf.data_ptr(), (a_row_scale.data_ptr() if a_row_scale is not None else None)
    a.w_packed, a.w_sf, a.w_global = w_packed.data_ptr(), w_sf.data_ptr(), w_global.data_ptr()
    a.w_global2 = w_global2.data_ptr() if w_global2 is not None else None
    a.group_tiles, a.group_rows = (tiles.data_ptr() if tiles is not None else None), rows.data_ptr()
    a.out, a.out_sf = out.data_ptr(), (out_sf.data_ptr() if out_sf is not None else None)
    a.padded_rows, a.N, a.K, a.groups, a.mode, a.sm_count = padded, N, K, groups, mode, sm_count
    a.all_active = 1 if (all_active and tiles is None) else 0
    a.err = err_word(dev).data_ptr()
    a.stream = cur_stream(dev)
    check(lib().tyr_fp4_grouped_gemm(ctypes.byref(a)), "fp4_grouped_gemm")
    return out if mode == 0 else (out, out_sf)


def moe_fp4_tc_forward(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, ex, offsets, order, tiles,
                       add: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, h] bf16, ids int32 [T, k], weights fp32 [T, k]; ``offsets`` / ``order`` / ``tiles`` from ``ops.moe.layout``.
    Everything stays on the device: the row count of the padded layout is bounded on the host by T * k + 127 * E."""
    from . import moe as M
    T, h = x.shape
    k = ids.shape[1]
    w4 = prepared(ex)
    E, mi = ex.num_experts, w4.moe_int
    pairs = T * k
    padded = ((pairs + 127 * min(E, pairs) + 127) // 128) * 128
    st = cur_stream(x.device)
    ids32 = ids.to(torch.int32).contiguous()
    xq, xsf, xrs, ppos = gather_quantize(x, order, ids32.reshape(-1), offsets, tiles, k, padded, pairs)
    hq, hsf = grouped_gemm_fp4(xq, xsf, xrs, w4.gu_packed, w4.gu_sf, w4.gate_global, tiles, offsets,
                               2 * mi, h, mode=1, w_global2=w4.up_global)
    y = grouped_gemm_fp4(hq, hsf, None, w4.dn_packed, w4.dn_sf, w4.dn_global, tiles, offsets, h, mi, mode=0)
    out = torch.empty_like(x)
    check(lib().tyr_moe_combine(ptr(y), ptr(ppos), ptr(weights.float().contiguous()), ptr(add.contiguous() if add is not None else None),
                                ptr(out), T, k, h, st), "moe_combine")
    return out


FIXED_SLOT_MAX_TOKENS = 128


_FIXED_SLOTS = os.environ.get("TYR_MOE_FIXED_SLOTS", "1") != "0"     # 0: always build the sorted layout (for comparisons)


def fixed_slots_supported(T: int, h: int) -> bool:
    return (_FIXED_SLOTS and T <= FIXED_SLOT_MAX_TOKENS and h % 256 == 0
            and hasattr(lib(), "tyr_fp4_scatter_quantize_fixed"))


def moe_fp4_tc_forward_fixed(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, ex,
                             add: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The same product for at most 128 tokens without a sorted layout: an expert can receive a token once, so every expert
    owns 128 fixed rows of the padded activation matrix, a row takes its slot with one atomic, and the grouped GEMM reads the
    slot cursors as its row counts.  Four launches (scatter + quantise, gate / up, down, combine) and one memset instead of the
    count / offsets / scatter / tile table / quantise launches of the sorted layout.  Slots are handed out in arrival order,
    which changes nothing: a row's result does not depend on where it sits."""
    T, h = x.shape
    k = ids.shape[1]
    w4 = prepared(ex)
    E, mi = ex.num_experts, w4.moe_int
    dev = x.device
    st = cur_stream(dev)
    ids32 = ids.to(torch.int32).contiguous()
    padded = E * 128
    cursors = torch.zeros(E, dtype=torch.int32, device=dev)
    xq = torch.empty((padded, h // 2), dtype=torch.uint8, device=dev)
    xsf = torch.empty(padded * (h // 16), dtype=torch.uint8, device=dev)
    xrs = torch.empty(padded, dtype=torch.float32, device=dev)
    ppos = torch.empty(T * k, dtype=torch.int32, device=dev)
    check(lib().tyr_fp4_scatter_quantize_fixed(ptr(x.contiguous()), ptr(ids32), ptr(cursors), ptr(xq), ptr(xsf), ptr(xrs), ptr(ppos),
                                               T, k, h, E, ptr(err_word(dev)), st), "fp4_scatter_quantize_fixed")
    # with six or more pairs per expert on average an expert without rows is rare (e^-6 under uniform routing): the GEMMs
    # may then fetch the weights of their first tiles before the row counts exist
    dense = T * k >= 6 * E
    hq, hsf = grouped_gemm_fp4(xq, xsf, xrs, w4.gu_packed, w4.gu_sf, w4.gate_global, None, cursors,
                               2 * mi, h, mode=1, w_global2=w4.up_global, all_active=dense)
    y = grouped_gemm_fp4(hq, hsf, None, w4.dn_packed, w4.dn_sf, w4.dn_global, None, cursors, h, mi, mode=0, all_active=dense)
    out = torch.empty_like(x)
    check(lib().tyr_moe_combine(ptr(y), ptr(ppos), ptr(weights.float().contiguous()), ptr(add.contiguous() if add is not None else None),
                                ptr(out), T, k, h, st), "moe_combine")
    return out


def moe_fp4_tc_reference(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, ex, add: Optional[torch.Tensor] = None):
    """The same computation in fp32 PyTorch: activations and SwiGLU outputs quantised to NVFP4 exactly like the kernels,
    weights decoded exactly, fp32 accumulation."""
    from . import moe as M
    T, h = x.shape
    k = ids.shape[1]
    dev = x.device
    lut = E2M1_VALUES.to(dev)

    def decode_bank(packed, scale, glob):
        lo, hi = lut[(packed & 15).long()], lut[(packed >> 4).long()]
        vals = torch.stack([lo, hi], -1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
        sf = scale.view(torch.float8_e4m3fn).float() if scale.dtype == torch.uint8 else scale.float()
        return vals * sf.repeat_interleave(16, dim=-1) / glob.float().reshape(-1, 1, 1)

    g_w, u_w, d_w = (decode_bank(ex.gate_packed, ex.gate_scale, ex.gate_global), decode_bank(ex.up_packed, ex.up_scale, ex.up_global),
                     decode_bank(ex.down_packed, ex.down_scale, ex.down_global))
    xq = dequant_rows_ref(*quantize_rows_ref(x))
    out = torch.zeros(T, h, dtype=torch.float32, device=dev)
    for e in torch.unique(ids).tolist():
        if e < 0 or e >= g_w.shape[0]:
            continue
        tok, slot = torch.nonzero(ids == e, as_tuple=True)
        xe = xq[tok]
        hid = torch.nn.functional.silu(xe @ g_w[e].T) * (xe @ u_w[e].T)
        hq = dequant_rows_ref(*quantize_rows_ref(hid, per_row_scale=False))
        y = (hq @ d_w[e].T).to(torch.bfloat16).float()
        out.index_add_(0, tok, y * weights[tok, slot].float()[:, None])
    if add is not None:
        out += add.float()
    return out.to(x.dtype)
