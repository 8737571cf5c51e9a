"""NVFP4 mixture-of-experts ops (csrc/moe_nvfp4.cu + the grouped tcgen05 GEMM).

``moe_fp4_forward`` is the counterpart of the reference's fused op
``lagunaMoeFp4Forward`` (Tyr/Model/Laguna/Fused.lean:61-113, cc/src/tyr_laguna_moe.cu:1233):
``out[t] = sum_s w[t,s] * down_e(silu(gate_e x_t) * up_e x_t)`` with ``e = ids[t,s]`` and NVFP4
banks.  Small batches take the weight-streaming grouped GEMV; larger ones the block-scaled FP4
tensor-core path of :mod:`tyr_b200.ops.fp4` (activations quantised on the fly, SwiGLU and
re-quantisation in the first product's epilogue); the banks are never dequantised.
The eager path ``moe_eager`` (per-expert loop) is the CPU oracle.
"""
from __future__ import annotations

import collections
import os
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from .._native import register_signatures
from ._common import check, cur_stream, lib, ptr
from .gemm import grouped_gemm

E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


@register_signatures
def _sigs(lib_):
    import ctypes
    P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    table = {
        "tyr_nvfp4_quantize": [P, P, P, P, L, L, P], "tyr_nvfp4_dequant": [P, P, P, P, L, L, P],
        "tyr_moe_route": [P, P, P, P, P, I, I, I, I, I, F, F, P],
        "tyr_moe_route_fused": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, F, P],
        "tyr_moe_layout": [P, P, P, P, P, P, P, P, I, I, P], "tyr_moe_count": [P, P, I, I, P],
        "tyr_moe_gather_rows": [P, P, P, I, I, I, P], "tyr_moe_combine": [P, P, P, P, P, I, I, I, P],
        "tyr_moe_fp4_gemv": [P] * 17 + [I, I, I, I, I, P], "tyr_moe_finalize": [P, P, P, L, P],
    }
    for name, args in table.items():
        fn = getattr(lib_, name, None)
        if fn is not None:
            fn.argtypes = args
            fn.restype = ctypes.c_int


# ---- quantise / dequantise ---------------------------------------------------------------------------
def nvfp4_global_scale(w: torch.Tensor) -> torch.Tensor:
    """One fp32 scale per leading matrix: (448 * 6) / amax, so that block scales fill e4m3's range."""
    lead = w.reshape(w.shape[0], -1) if w.dim() == 3 else w.reshape(1, -1)
    amax = lead.float().abs().amax(dim=1).clamp_min(1e-12)
    return (448.0 * 6.0) / amax


def _e4m3(x: torch.Tensor) -> torch.Tensor:
    return x.clamp(-448.0, 448.0).to(torch.float8_e4m3fn)


def nvfp4_quantize(w: torch.Tensor, global_scale: Optional[torch.Tensor] = None):
    """w: [.., out, in] (in % 16 == 0) -> (packed u8 [.., out, in/2], scales e4m3 [.., out, in/16],
    global fp32 [lead])."""
    if w.shape[-1] % 16 != 0:
        raise ValueError(f"nvfp4: inFeatures={w.shape[-1]} not divisible by 16")
    g = global_scale if global_scale is not None else nvfp4_global_scale(w)
    mats = w.shape[0] if w.dim() == 3 else 1
    if w.is_cuda:
        wb = w.to(torch.bfloat16).contiguous()
        packed = torch.empty(w.shape[:-1] + (w.shape[-1] // 2,), dtype=torch.uint8, device=w.device)
        scales = torch.empty(w.shape[:-1] + (w.shape[-1] // 16,), dtype=torch.uint8, device=w.device)
        gc = g.float().contiguous()
        check(lib().tyr_nvfp4_quantize(ptr(wb), ptr(packed), ptr(scales), ptr(gc), mats, wb.numel() // mats,
                                       cur_stream(w.device)), "nvfp4_quantize")
        return packed, scales.view(torch.float8_e4m3fn), gc
    wf = w.to(torch.bfloat16).float()
    blocks = wf.reshape(*w.shape[:-1], w.shape[-1] // 16, 16)
    gb = g.float().reshape(-1, *([1] * (blocks.dim() - 1))) if w.dim() == 3 else g.float().reshape(())
    amax = blocks.abs().amax(-1, keepdim=True)
    s8 = _e4m3(amax / 6.0 * gb)
    s = s8.float()
    q = torch.where(s > 0, blocks * (gb / s.clamp_min(1e-30)), torch.zeros_like(blocks))
    a = q.abs()
    mag = torch.zeros_like(a, dtype=torch.uint8)
    for thr_lo, strict, code in ((0.25, False, 1), (0.75, True, 2), (1.25, False, 3), (1.75, True, 4),
                                 (2.5, False, 5), (3.5, True, 6), (5.0, False, 7)):
        mag = torch.where((a >= thr_lo) if strict else (a > thr_lo), torch.full_like(mag, code), mag)
    nib = mag | ((q < 0).to(torch.uint8) << 3)
    nib = nib.reshape(*w.shape[:-1], w.shape[-1] // 2, 2)
    packed = nib[..., 0] | (nib[..., 1] << 4)
    return packed, s8.reshape(*w.shape[:-1], w.shape[-1] // 16), g.float()


def nvfp4_dequant(packed: torch.Tensor, scales: torch.Tensor, global_scale: torch.Tensor) -> torch.Tensor:
    """Exact inverse map to bf16: e2m1(nibble) * (e4m3(scale) / global), fp32 product rounded once."""
    shape = packed.shape[:-1] + (packed.shape[-1] * 2,)
    mats = packed.shape[0] if packed.dim() == 3 else 1
    if packed.is_cuda:
        out = torch.empty(shape, dtype=torch.bfloat16, device=packed.device)
        sc = scales.view(torch.uint8).contiguous()
        gc = global_scale.float().reshape(-1).contiguous()
        check(lib().tyr_nvfp4_dequant(ptr(packed.contiguous()), ptr(sc), ptr(gc), ptr(out), mats, out.numel() // mats,
                                      cur_stream(packed.device)), "nvfp4_dequant")
        return out
    lut = E2M1.to(packed.device)
    lo = lut[(packed & 15).long()]
    hi = lut[(packed >> 4).long()]
    vals = torch.stack([lo, hi], dim=-1).reshape(shape)
    sf = scales.view(torch.float8_e4m3fn).float() if scales.dtype == torch.uint8 else scales.float()
    g = global_scale.float().reshape(-1, 1, 1) if packed.dim() == 3 else global_scale.float().reshape(())
    sd = (sf / g).repeat_interleave(16, dim=-1)
    return (sd * vals).to(torch.bfloat16)


# ---- routing -------------------------------------------------------------------------------------------
def route(logits: torch.Tensor, k: int, *, softmax: bool = False, bias: Optional[torch.Tensor] = None,
          renorm: bool = True, softcap: float = 0.0, scale: float = 1.0, want_counts: bool = True):
    """logits fp32 [T, E] -> (ids int32 [T, k], weights fp32 [T, k], counts int32 [E]).
    Sigmoid (Laguna, Tyr/Model/Laguna/MoE.lean:71-90) or softmax (Qwen3.5) scores; the selection
    bias only influences WHICH experts are picked; ties go to the lower expert index."""
    T, E = logits.shape
    if logits.is_cuda:
        lg = logits.float().contiguous()
        ids = torch.empty((T, k), dtype=torch.int32, device=logits.device)
        w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
        counts = torch.zeros(E, dtype=torch.int32, device=logits.device)
        b = bias.float().contiguous() if bias is not None else None
        check(lib().tyr_moe_route(ptr(lg), ptr(b), ptr(ids), ptr(w), ptr(counts), T, E, k, 1 if softmax else 0,
                                  1 if renorm else 0, softcap, scale, cur_stream(logits.device)), "moe_route")
        return ids, w, counts
    l = logits.float()
    if softcap > 0:
        l = softcap * torch.tanh(l / softcap)
    scores = torch.softmax(l, -1) if softmax else torch.sigmoid(l)
    sel = scores + bias.float() if bias is not None else scores
    order = torch.argsort(sel, dim=-1, descending=True, stable=True)[:, :k]
    w = torch.gather(scores, 1, order)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    ids = order.to(torch.int32)
    counts = torch.bincount(ids.reshape(-1).long(), minlength=E).to(torch.int32)
    return ids, w * scale, counts


def count_experts(ids: torch.Tensor, E: int) -> torch.Tensor:
    """int32 [E] histogram of the expert ids; ids outside [0, E) (padding rows) are not counted.  No host synchronisation on CUDA."""
    flat = ids.reshape(-1)
    if not ids.is_cuda:
        flat = flat.long()
        return torch.bincount(flat[(flat >= 0) & (flat < E)], minlength=E).to(torch.int32)
    counts = torch.zeros(E, dtype=torch.int32, device=ids.device)
    flat = flat.to(torch.int32).contiguous()
    check(lib().tyr_moe_count(ptr(flat), ptr(counts), flat.numel(), E, cur_stream(ids.device)), "moe_count")
    return counts


ROUTE_FUSED_MAX_TOKENS = 256
_ROUTE_FUSED = os.environ.get("TYR_ROUTE_FUSED", "1") != "0"


def route_fused_supported(x: torch.Tensor, router_w: torch.Tensor) -> bool:
    """Decode-sized bf16 batches with an fp32 router: logits and routing in one launch."""
    return (_ROUTE_FUSED and x.is_cuda and x.dtype == torch.bfloat16 and router_w.dtype == torch.float32 and x.dim() == 2
            and x.shape[0] <= ROUTE_FUSED_MAX_TOKENS and x.shape[1] % 8 == 0 and router_w.shape[0] <= 512 and 16 * x.shape[1] <= 160 * 1024
            and x.is_contiguous() and router_w.is_contiguous() and hasattr(lib(), "tyr_moe_route_fused"))


def route_fused(x: torch.Tensor, router_w: torch.Tensor, k: int, *, softmax: bool = False, bias: Optional[torch.Tensor] = None,
                renorm: bool = True, softcap: float = 0.0, scale: float = 1.0):
    """x bf16 [T, h], router_w fp32 [E, h] -> (ids, weights, counts) as :func:`route` of ``x.float() @ router_w.T`` (fp32
    accumulation inside the kernel; the logits are never written out)."""
    T, E = x.shape[0], router_w.shape[0]
    ids = torch.empty((T, k), dtype=torch.int32, device=x.device)
    w = torch.empty((T, k), dtype=torch.float32, device=x.device)
    zeros = torch.zeros(E + (T + 3) // 4, dtype=torch.int32, device=x.device)       # expert counts, then one ticket per group of 4 tokens
    counts, tickets = zeros[:E], zeros[E:]
    logits = torch.empty((T, E), dtype=torch.float32, device=x.device)
    b = bias.float().contiguous() if bias is not None else None
    check(lib().tyr_moe_route_fused(ptr(x), ptr(router_w), ptr(b), ptr(logits), ptr(tickets), ptr(ids), ptr(w), ptr(counts), T, E, k, x.shape[1], 1 if softmax else 0,
                                    1 if renorm else 0, softcap, scale, cur_stream(x.device)), "moe_route_fused")
    return ids, w, counts


def layout(ids: torch.Tensor, counts: torch.Tensor, want_tiles: bool = False, want_active: bool = False):
    """(offsets int32 [E+1], pair_order int32 [pairs], pair_pos int32 [pairs]) - expert-major.
    With ``want_tiles`` a fourth result: the 128-row tile prefix table the grouped GEMM walks."""
    pairs, E = ids.numel(), counts.numel()
    if ids.is_cuda:
        meta = torch.empty(4 * E + 3, dtype=torch.int32, device=ids.device)
        offsets, tiles, cursors, active = meta[:E + 1], meta[E + 1:2 * E + 2], meta[2 * E + 2:3 * E + 2], meta[3 * E + 2:]
        op = torch.zeros(2 * pairs, dtype=torch.int32, device=ids.device)     # positions no routed pair fills (padding ids) must stay valid indices
        order, pos = op[:pairs], op[pairs:]
        check(lib().tyr_moe_layout(ptr(ids.contiguous()), ptr(counts), ptr(offsets), ptr(cursors), ptr(tiles), ptr(active),
                                   ptr(order), ptr(pos), pairs, E, cur_stream(ids.device)), "moe_layout")
        if want_active:
            return offsets, order, pos, tiles, active       # active[:E] compact expert list, active[E] their number
        return (offsets, order, pos, tiles) if want_tiles else (offsets, order, pos)
    flat = ids.reshape(-1).long()
    order = torch.argsort(flat, stable=True).to(torch.int32)
    pos = torch.empty(pairs, dtype=torch.int32)
    pos[order.long()] = torch.arange(pairs, dtype=torch.int32)
    offsets = torch.cat([torch.zeros(1, dtype=torch.int32), torch.cumsum(counts, 0).to(torch.int32)])
    if want_tiles:
        return offsets, order, pos, group_tile_prefix(offsets)
    return offsets, order, pos


def group_tile_prefix(offsets: torch.Tensor) -> torch.Tensor:
    """int32 [G+1]: exclusive prefix sum of ceil(rows_g / 128)."""
    cnt = (offsets[1:] - offsets[:-1]).to(torch.int64)
    t = torch.cumsum((cnt + 127) // 128, 0).to(torch.int32)
    return torch.cat([torch.zeros(1, dtype=torch.int32, device=offsets.device), t])


# ---- expert banks ------------------------------------------------------------------------------------------
@dataclass
class PackedExperts:
    """NVFP4 banks: gate/up packed [E, mi, h/2] + scales [E, mi, h/16] + global [E]; down [E, h, mi/2]..."""
    gate_packed: torch.Tensor
    gate_scale: torch.Tensor
    gate_global: torch.Tensor
    up_packed: torch.Tensor
    up_scale: torch.Tensor
    up_global: torch.Tensor
    down_packed: torch.Tensor
    down_scale: torch.Tensor
    down_global: torch.Tensor

    @property
    def num_experts(self): return self.gate_packed.shape[0]
    @property
    def hidden(self): return self.gate_packed.shape[2] * 2
    @property
    def moe_int(self): return self.gate_packed.shape[1]

    @staticmethod
    def quantize(gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> "PackedExperts":
        gp, gs, gg = nvfp4_quantize(gate)
        up_, us, ug = nvfp4_quantize(up)
        dp, ds, dg = nvfp4_quantize(down)
        return PackedExperts(gp, gs, gg, up_, us, ug, dp, ds, dg)

    def validate(self):
        E, mi, h = self.num_experts, self.moe_int, self.hidden
        exp = {"gate_packed": (E, mi, h // 2), "gate_scale": (E, mi, h // 16), "gate_global": (E,),
               "up_packed": (E, mi, h // 2), "up_scale": (E, mi, h // 16), "up_global": (E,),
               "down_packed": (E, h, mi // 2), "down_scale": (E, h, mi // 16), "down_global": (E,)}
        for k, shp in exp.items():
            if tuple(getattr(self, k).shape) != shp:
                raise ValueError(f"nvfp4: {k} must have shape {list(shp)}, got {list(getattr(self, k).shape)}")
        if h % 32 or mi % 32:
            raise ValueError("laguna moe: hidden and moe_intermediate must be multiples of 32")

    def dense(self):
        """(gate, up, down) dequantised to bf16."""
        return (nvfp4_dequant(self.gate_packed, self.gate_scale, self.gate_global),
                nvfp4_dequant(self.up_packed, self.up_scale, self.up_global),
                nvfp4_dequant(self.down_packed, self.down_scale, self.down_global))

    def weight_bytes_per_pair(self) -> int:
        """FP4 bytes the fused op reads per (token, slot) pair (Tests/RunLagunaFused.lean:373-375)."""
        h, mi = self.hidden, self.moe_int
        return 2 * (mi * h // 2 + mi * h // 16) + (h * mi // 2 + h * mi // 16)


def moe_eager(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, gate: torch.Tensor, up: torch.Tensor,
              down: torch.Tensor, act: str = "swiglu") -> torch.Tensor:
    """Per-unique-expert loop on dense banks (the reference's eager path, MoE.lean:313-356); fp32 math.  ``act``: "swiglu"
    or "geglu" (tanh-GELU gate, Gemma 4); ids outside the bank are skipped."""
    T, h = x.shape
    out = torch.zeros(T, h, dtype=torch.float32, device=x.device)
    xf = x.float()
    fn = torch.nn.functional.silu if act == "swiglu" else (lambda t: torch.nn.functional.gelu(t, approximate="tanh"))
    for e in torch.unique(ids).tolist():
        if e < 0 or e >= gate.shape[0]:
            continue
        tok, slot = torch.nonzero(ids == e, as_tuple=True)
        xe = xf[tok]
        hdn = fn(xe @ gate[e].float().T) * (xe @ up[e].float().T)
        out.index_add_(0, tok, (hdn @ down[e].float().T) * weights[tok, slot].float().unsqueeze(-1))
    return out.to(x.dtype)


def moe_eager_model_dtype(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, gate: torch.Tensor, up: torch.Tensor,
                          down: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """The same per-unique-expert loop with every operation in the model dtype and in the order of the reference's eager
    path (MoE.lean:313-356): experts in ascending order, ``linear`` / SiLU / product / ``linear`` each rounded to ``x.dtype``,
    routing weights (without the routed scale, rounded to ``x.dtype``) applied to the expert output, accumulator in
    ``x.dtype``, the routed scale applied once after accumulation.  In bf16 this reproduces the rounding points of the
    Hugging Face implementation that generated the reference's fixtures; in fp32 it equals :func:`moe_eager`."""
    T, h = x.shape
    dt = x.dtype
    acc = torch.zeros(T, h, dtype=dt, device=x.device)
    w = weights.to(dt)
    lin = torch.nn.functional.linear
    for e in torch.unique(ids).tolist():
        if e < 0 or e >= gate.shape[0]:
            continue
        tok, slot = torch.nonzero(ids == e, as_tuple=True)
        xe = x[tok]
        hdn = torch.nn.functional.silu(lin(xe, gate[e].to(dt))) * lin(xe, up[e].to(dt))
        oe = lin(hdn, down[e].to(dt)) * w[tok, slot].unsqueeze(-1)
        acc.index_add_(0, tok, oe)
    return acc * scale


GEMV_MAX_PAIRS_PER_EXPERT = 8


def moe_fp4_forward(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, ex: PackedExperts,
                    counts: Optional[torch.Tensor] = None, add: Optional[torch.Tensor] = None,
                    force_path: Optional[str] = None) -> torch.Tensor:
    """x: [T, h] bf16; ids int32 [T, k]; weights fp32 [T, k] -> [T, h] bf16 (+ ``add`` if given)."""
    T, h = x.shape
    k = ids.shape[1]
    E, mi = ex.num_experts, ex.moe_int
    if T * k < 1 or T * k > (1 << 24):
        raise ValueError("laguna moe: tokens*k out of range")
    if not x.is_cuda:
        g, u, d = ex.dense()
        y = moe_eager(x, ids, weights, g, u, d)
        return y + add if add is not None else y
    wf = weights.float().contiguous()
    from . import fp4
    tc_ok = fp4.available() and fp4.Fp4Experts.supported(h, mi) and x.dtype == torch.bfloat16
    gemv_ok = h % 128 == 0 and mi % 128 == 0
    # measured at hidden 3072 / 256 experts / top-10: the tensor-core path overtakes the weight-streaming GEMV once an
    # expert sees more than about two rows (64 tokens: 0.27 ms against 0.39 ms)
    gemv_limit = (2 if tc_ok else GEMV_MAX_PAIRS_PER_EXPERT) * E
    path = force_path or ("gemv" if (T * k <= gemv_limit and gemv_ok) else "gemm")
    if path in ("gemm", "gemm_sorted") and not tc_ok:
        path = "gemv" if gemv_ok else "eager"
    if path == "gemv" and not gemv_ok:
        path = "gemm" if tc_ok else "eager"
    if path == "gemm" and fp4.fixed_slots_supported(T, h):
        # decode-sized batch: fixed 128-row slots per expert, no sorted layout ("gemm_sorted" forces the layout below)
        return fp4.moe_fp4_tc_forward_fixed(x, ids, wf, ex, add=add)
    if counts is None:
        counts = count_experts(ids, E)
    offsets, order, pos, tiles, active = layout(ids.to(torch.int32), counts, want_active=True)
    st = cur_stream(x.device)
    if path == "eager":      # shapes neither kernel tiles (tiny test models): per-expert loop on banks decoded on the fly
        g, u, d = ex.dense()
        y = moe_eager(x, ids, weights, g, u, d)
        return (y.float() + add.float()).to(x.dtype) if add is not None else y
    if path == "gemv":
        hid = torch.zeros((2, T * k, mi), dtype=torch.float32, device=x.device)
        routed = torch.zeros((T, h), dtype=torch.float32, device=x.device)
        sc = lambda t: t.view(torch.uint8)
        check(lib().tyr_moe_fp4_gemv(ptr(x.contiguous()), ptr(ex.gate_packed), ptr(sc(ex.gate_scale)), ptr(ex.gate_global),
                                     ptr(ex.up_packed), ptr(sc(ex.up_scale)), ptr(ex.up_global),
                                     ptr(ex.down_packed), ptr(sc(ex.down_scale)), ptr(ex.down_global),
                                     ptr(offsets), ptr(active), ptr(active[E:]), ptr(order), ptr(wf), ptr(hid), ptr(routed),
                                     T * k, E, k, h, mi, st),
              "moe_fp4_gemv")
        out = torch.empty_like(x)
        check(lib().tyr_moe_finalize(ptr(routed), ptr(add.contiguous() if add is not None else None), ptr(out),
                                     routed.numel(), st), "moe_finalize")
        return out
    # block-scaled FP4 tensor-core path: activations quantised on the fly, banks stay 4-bit end to end
    return fp4.moe_fp4_tc_forward(x, ids, wf, ex, offsets, order, tiles, add=add)


_gu_cache: Dict[int, torch.Tensor] = {}


def interleave_gate_up(gate_up: torch.Tensor) -> torch.Tensor:
    """[E, 2*mi, h] (gate rows then up rows) -> 128-row gate/up interleave expected by the grouped GEMM's
    SwiGLU epilogue; mi is padded to a multiple of 128 with zero rows.  Cached per source tensor."""
    key = gate_up.data_ptr()
    hit = _gu_cache.get(key)
    if hit is not None and hit.shape[0] == gate_up.shape[0]:
        return hit
    E, two_mi, h = gate_up.shape
    mi = two_mi // 2
    g, u = gate_up[:, :mi], gate_up[:, mi:]
    pad = (-mi) % 128
    if pad:
        g, u = torch.nn.functional.pad(g, (0, 0, 0, pad)), torch.nn.functional.pad(u, (0, 0, 0, pad))
    mp = mi + pad
    out = torch.stack([g.reshape(E, mp // 128, 128, h), u.reshape(E, mp // 128, 128, h)], dim=2).reshape(E, 2 * mp, h).contiguous()
    if len(_gu_cache) > 256:
        _gu_cache.clear()
    _gu_cache[key] = out
    return out


def moe_dense_forward(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor,
                      counts: Optional[torch.Tensor] = None, add: Optional[torch.Tensor] = None, act: str = "swiglu") -> torch.Tensor:
    """bf16 expert banks: ``gate_up`` [E, 2*mi, h], ``down`` [E, h, mi].  Grouped tensor-core path on the
    GPU for bf16; per-expert loop otherwise (Tyr/Model/Qwen35/Model.lean:200-248 computes the same sum
    by gathering one expert matrix per (token, slot))."""
    T, h = x.shape
    E, two_mi, _ = gate_up.shape
    mi = two_mi // 2
    k = ids.shape[1]
    if not (x.is_cuda and x.dtype == torch.bfloat16 and gate_up.dtype == torch.bfloat16 and h % 8 == 0 and mi % 8 == 0):
        y = moe_eager(x, ids, weights, gate_up[:, :mi], gate_up[:, mi:], down, act=act)
        return y if add is None else (y.float() + add.float()).to(x.dtype)
    if counts is None:
        counts = count_experts(ids, E)
    offsets, order, pos, tiles = layout(ids.to(torch.int32), counts, want_tiles=True)
    st = cur_stream(x.device)
    gu = interleave_gate_up(gate_up)
    dn = down if mi % 128 == 0 else torch.nn.functional.pad(down, (0, (-mi) % 128)).contiguous()
    xs = torch.empty((T * k, h), dtype=x.dtype, device=x.device)
    check(lib().tyr_moe_gather_rows(ptr(x.contiguous()), ptr(order), ptr(xs), T * k, k, h, st), "moe_gather_rows")
    hid = grouped_gemm(xs, gu, offsets, tiles, act=act)
    y = grouped_gemm(hid, dn.contiguous(), offsets, tiles)
    out = torch.empty_like(x)
    check(lib().tyr_moe_combine(ptr(y), ptr(pos), ptr(weights.float().contiguous()), ptr(add.contiguous() if add is not None else None),
                                ptr(out), T, k, h, st), "moe_combine")
    return out
