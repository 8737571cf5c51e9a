"""Gated delta rule (Qwen3.5 GatedDeltaNet core): chunked prefill, recurrent oracle, fused decode step.

q, k: [B, S, H, dk]; v: [B, S, H, dv]; g (log decay, <= 0) and beta: [B, S, H]; state [B, H, dk, dv] fp32.
Semantics: cc/src/tyr_qwen35.cpp:12-170 of the reference (L2-normalised q/k, q scaled by dk^-1/2).
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from .._native import register_signatures
from ._common import check, cur_stream, err_word, lib, ptr


@register_signatures
def _sigs(lib_):
    import ctypes
    P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    fn = getattr(lib_, "tyr_gdr_decode", None)
    if fn is not None:
        fn.argtypes = [P, P, P, P, P, P, P, I, I, I, I, I, L, L, P]
        fn.restype = ctypes.c_int
    fn = getattr(lib_, "tyr_gdr_decode_norm", None)
    if fn is not None:
        fn.argtypes = [P, P, P, P, P, P, P, I, I, I, I, I, L, L, P, L, P, ctypes.c_float, P]
        fn.restype = ctypes.c_int
    fn = getattr(lib_, "tyr_gdr_decode_tile", None)
    if fn is not None:
        fn.argtypes = [P, P, P, P, P, P, P, I, I, I, I, L, L, P, L, P, ctypes.c_float, P, P]
        fn.restype = ctypes.c_int
    fn = getattr(lib_, "tyr_gdn_conv_gates", None)
    if fn is not None:
        fn.argtypes = [P] * 3 + [L, L, L] + [P] * 8 + [I, I, I, I, P]
        fn.restype = ctypes.c_int
    fn = getattr(lib_, "tyr_gdr_chunk_scan", None)
    if fn is not None:
        fn.argtypes = [P] * 9 + [I, I, I, I, I, I, I, P]
        fn.restype = ctypes.c_int
    fn = getattr(lib_, "tyr_gdr_chunk_prepare", None)
    if fn is not None:
        fn.argtypes = [P] * 11 + [ctypes.POINTER(L), I, I, I, I, I, I, P]
        fn.restype = ctypes.c_int
    fn = getattr(lib_, "tyr_causal_conv1d_silu", None)
    if fn is not None:
        fn.argtypes = [P, P, P, P, I, I, I, I, L, L, P]
        fn.restype = ctypes.c_int


_CHUNK_KERNEL = os.environ.get("TYR_GDR_CHUNK_KERNEL", "1") != "0"


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def recurrent_gated_delta_rule(q, k, v, g, beta, state: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Token-by-token recurrence in fp32 (oracle and the multi-token fallback with an initial state)."""
    dt = q.dtype
    qf = l2norm(q.float()).transpose(1, 2) * (q.shape[-1] ** -0.5)
    kf = l2norm(k.float()).transpose(1, 2)
    vf, bf, gf = v.float().transpose(1, 2), beta.float().transpose(1, 2), g.float().transpose(1, 2)
    B, H, S, dk = kf.shape
    dv = vf.shape[-1]
    st = torch.zeros(B, H, dk, dv, device=q.device) if state is None else state.float().clone()
    out = torch.empty(B, H, S, dv, device=q.device)
    for i in range(S):
        st = st * gf[:, :, i].exp()[..., None, None]
        kv = (st * kf[:, :, i].unsqueeze(-1)).sum(-2)
        delta = (vf[:, :, i] - kv) * bf[:, :, i].unsqueeze(-1)
        st = st + kf[:, :, i].unsqueeze(-1) * delta.unsqueeze(-2)
        out[:, :, i] = (st * qf[:, :, i].unsqueeze(-1)).sum(-2)
    return out.transpose(1, 2).contiguous().to(dt), st


def chunk_kernels_supported(q, k, v, chunk_size: int = 64) -> bool:
    """Both chunk kernels (csrc/delta_rule.cu) apply: bf16 on CUDA, dk 128, dv 64 or 128, chunk 64, 16-byte aligned q / k rows;
    q and k may carry fewer heads than v (grouped keys)."""
    ok_view = lambda t: t.stride(3) == 1 and all(x % 8 == 0 for x in t.stride()[:3]) and t.data_ptr() % 16 == 0
    return (_CHUNK_KERNEL and q.is_cuda and q.dtype == k.dtype == v.dtype == torch.bfloat16 and q.shape[-1] == 128 and v.shape[-1] in (64, 128)
            and chunk_size == 64 and v.shape[2] % q.shape[2] == 0 and q.shape[2] == k.shape[2] and ok_view(q) and ok_view(k) and ok_view(v)
            and hasattr(lib(), "tyr_gdr_chunk_prepare") and hasattr(lib(), "tyr_gdr_chunk_scan"))


def chunk_gated_delta_rule_fused(q, k, v, g, beta, state: Optional[torch.Tensor] = None):
    """Two launches: the chunk-local quantities (normalisation, decay, the two 64 x 64 products, the triangular solve) and the
    recurrence over the chunks.  q, k: [B, S, Hk, 128] with Hk dividing Hv (keys are not repeated); see :func:`chunk_kernels_supported`."""
    import ctypes
    B, S, Hk, dk = q.shape
    Hv, dv = v.shape[2], v.shape[3]
    n, BH, dev = (S + 63) // 64, B * Hv, q.device
    f32 = lambda *shape: torch.empty(shape, dtype=torch.float32, device=dev)
    u, w, qg, kd, intra, glast = f32(BH, n, 64, dv), f32(BH, n, 64, dk), f32(BH, n, 64, dk), f32(BH, n, 64, dk), f32(BH, n, 64, 64), f32(BH, n)
    strides = (ctypes.c_longlong * 9)(*[t.stride(i) for t in (q, k, v) for i in range(3)])
    gc, bc = g.float().contiguous(), beta.float().contiguous()
    st = cur_stream(dev)
    check(lib().tyr_gdr_chunk_prepare(ptr(q), ptr(k), ptr(v), ptr(gc), ptr(bc), ptr(u), ptr(w), ptr(qg), ptr(kd), ptr(intra), ptr(glast), strides,
                                      B, S, Hk, Hv, dk, dv, st), "gdr_chunk_prepare")
    st_in = None if state is None else state.float().contiguous()
    st_out = f32(B, Hv, dk, dv)
    out = torch.empty((B, S, Hv, dv), dtype=torch.bfloat16, device=dev)          # written in the layer's layout by the scan kernel
    check(lib().tyr_gdr_chunk_scan(ptr(u), ptr(w), ptr(qg), ptr(kd), ptr(intra), ptr(glast), ptr(st_in), ptr(st_out), ptr(out), BH, n, dk, dv, 64, S, Hv, st),
          "gdr_chunk_scan")
    return out, st_out


def causal_conv1d_silu(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x: [B, S, C] (channels last), weight: [C, K] -> silu(causal depthwise conv + bias) as [B, S, C], zero history."""
    B, S, C = x.shape
    K = weight.shape[-1]
    if (x.is_cuda and x.dtype == torch.bfloat16 and C % 8 == 0 and K <= 4 and x.stride(2) == 1 and x.stride(0) % 8 == 0 and x.stride(1) % 8 == 0
            and x.data_ptr() % 16 == 0 and hasattr(lib(), "tyr_causal_conv1d_silu")):
        y = torch.empty((B, S, C), dtype=x.dtype, device=x.device)
        wf = weight.reshape(C, K).float().contiguous()
        bf = None if bias is None else bias.float().contiguous()
        check(lib().tyr_causal_conv1d_silu(ptr(x), ptr(wf), ptr(bf), ptr(y), B, S, C, K, x.stride(0), x.stride(1), cur_stream(x.device)), "causal_conv1d_silu")
        return y
    xc = x.transpose(1, 2)
    y = torch.nn.functional.conv1d(torch.nn.functional.pad(xc, (K - 1, 0)), weight.reshape(C, 1, K).to(xc.dtype), None if bias is None else bias.to(xc.dtype), groups=C)
    return torch.nn.functional.silu(y).transpose(1, 2)


def chunk_gated_delta_rule(q, k, v, g, beta, chunk_size: int = 64, state: Optional[torch.Tensor] = None):
    """Chunk-parallel form: the intra-chunk triangular system is solved with one batched
    unit-lower-triangular solve; chunks are chained through the [dk, dv] state."""
    if chunk_kernels_supported(q, k, v, chunk_size):
        return chunk_gated_delta_rule_fused(q, k, v, g, beta, state)
    if q.shape[2] != v.shape[2]:
        rep = v.shape[2] // q.shape[2]
        q, k = q.repeat_interleave(rep, dim=2), k.repeat_interleave(rep, dim=2)
    dt = q.dtype
    qf = l2norm(q.float()).transpose(1, 2) * (q.shape[-1] ** -0.5)
    kf = l2norm(k.float()).transpose(1, 2)
    vf, bf, gf = v.float().transpose(1, 2), beta.float().transpose(1, 2), g.float().transpose(1, 2)
    B, H, S, dk = kf.shape
    dv = vf.shape[-1]
    pad = (-S) % chunk_size
    if pad:
        P = lambda t, d: torch.nn.functional.pad(t, (0, 0, 0, pad) if d else (0, pad))
        qf, kf, vf, bf, gf = P(qf, 1), P(kf, 1), P(vf, 1), P(bf, 0), P(gf, 0)
    n, C = (S + pad) // chunk_size, chunk_size
    rs = lambda t: t.reshape(B, H, n, C, *t.shape[3:])
    qf, kf, vf, bf, gf = rs(qf), rs(kf), rs(vf), rs(bf), rs(gf)
    gc = gf.cumsum(-1)
    decay = torch.tril((gc.unsqueeze(-1) - gc.unsqueeze(-2))).exp().tril()
    kb, vb = kf * bf.unsqueeze(-1), vf * bf.unsqueeze(-1)
    L = (kb @ kf.transpose(-1, -2) * decay).tril(-1)                           # strictly lower
    eye = torch.eye(C, device=q.device)
    rhs = torch.cat([vb, kb * gc.exp().unsqueeze(-1)], dim=-1)
    sol = torch.linalg.solve_triangular(eye + L, rhs, upper=False, unitriangular=True)
    u, w = sol[..., :dv], sol[..., dv:]                                          # "value" and "k_cumdecay"
    intra = (qf @ kf.transpose(-1, -2) * decay).tril()
    st = torch.zeros(B, H, dk, dv, device=q.device) if state is None else state.float().clone()
    out = torch.empty(B, H, n, C, dv, device=q.device)
    for i in range(n):
        v_new = u[:, :, i] - w[:, :, i] @ st
        out[:, :, i] = (qf[:, :, i] * gc[:, :, i].exp().unsqueeze(-1)) @ st + intra[:, :, i] @ v_new
        g_last = gc[:, :, i, -1]
        st = st * g_last.exp()[..., None, None] + (kf[:, :, i] * (g_last.unsqueeze(-1) - gc[:, :, i]).exp().unsqueeze(-1)).transpose(-1, -2) @ v_new
    out = out.reshape(B, H, n * C, dv)[:, :, :S].transpose(1, 2).contiguous().to(dt)
    return out, st


def gdr_decode_step(q, k, v, g, beta, state: torch.Tensor) -> torch.Tensor:
    """One token: q, k [B, 1, Hk, dk] (un-repeated key heads), v [B, 1, Hv, dv], g/beta [B, 1, Hv];
    ``state`` fp32 [B, Hv, dk, dv] is updated IN PLACE.  Returns [B, 1, Hv, dv]."""
    B, _, Hk, dk = q.shape
    Hv, dv = v.shape[2], v.shape[3]
    if (q.is_cuda and q.dtype == torch.bfloat16 and dk in (64, 128) and state.dtype == torch.float32
            and state.is_contiguous() and q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
            and q.stride(2) == dk and k.stride(2) == dk and v.stride(2) == dv and q.stride(0) == k.stride(0)):
        out = torch.empty((B, 1, Hv, dv), dtype=q.dtype, device=q.device)
        gc, bc = g.float().contiguous(), beta.float().contiguous()
        if _tile_ok(dv, v, None, B * Hv):
            check(lib().tyr_gdr_decode_tile(ptr(q), ptr(k), ptr(v), ptr(gc), ptr(bc), ptr(state), ptr(out), B, Hk, Hv, dk,
                                            q.stride(0), v.stride(0), None, 0, None, 0.0, ptr(err_word(q.device)),
                                            cur_stream(q.device)), "gdr_decode_tile")
            return out
        check(lib().tyr_gdr_decode(ptr(q), ptr(k), ptr(v), ptr(gc), ptr(bc), ptr(state), ptr(out), B, Hk, Hv, dk, dv,
                                   q.stride(0), v.stride(0), cur_stream(q.device)), "gdr_decode")
        return out
    rep = Hv // Hk
    qr, kr = q.repeat_interleave(rep, dim=2), k.repeat_interleave(rep, dim=2)
    out, st = recurrent_gated_delta_rule(qr, kr, v, g, beta, state)
    state.copy_(st)
    return out


_GDN_FUSED = os.environ.get("TYR_GDN_DECODE_FUSED", "1") != "0"
_GDR_TILE = os.environ.get("TYR_GDR_DECODE_TILE", "1") != "0"      # 0: the register-resident form of the decode step
# Fewer (batch, head) tiles than this: the register-resident form.  The tile form was faster at every size measured (8 to 64
# rows x 48 heads) once the weight-streaming GEMMs state their own shared-memory / L1 split (csrc/skinny_gemm.cu): its
# 64 KB tiles leave the SMs configured for shared memory.
_GDR_TILE_MIN_TILES = int(os.environ.get("TYR_GDR_TILE_MIN_TILES", "0"))


def _tile_ok(dv: int, v: torch.Tensor, z: Optional[torch.Tensor], tiles: int) -> bool:
    """The shared-memory tile form of the decode step: dv == 128, 8-byte aligned v / z rows, enough tiles."""
    if not (_GDR_TILE and dv == 128 and tiles >= _GDR_TILE_MIN_TILES and hasattr(lib(), "tyr_gdr_decode_tile")):
        return False
    for t in (v, z):
        if t is not None and (t.data_ptr() % 8 or t.stride(0) % 4):
            return False
    return True


def gdn_decode_fused_supported(mixed, conv_state, rec_state, dk: int, dv: int) -> bool:
    return (_GDN_FUSED and mixed.is_cuda and mixed.dtype == torch.bfloat16 and mixed.shape[1] == 1 and mixed.stride(-1) == 1
            and conv_state is not None and conv_state.dtype == torch.bfloat16 and conv_state.is_contiguous()
            and rec_state is not None and rec_state.dtype == torch.float32 and rec_state.is_contiguous()
            and dk in (64, 128) and dv == 128 and hasattr(lib(), "tyr_gdn_conv_gates") and hasattr(lib(), "tyr_gdr_decode_norm"))


def gdn_decode_fused(mixed, z, b, a, conv_state, conv_w, conv_b, dt_bias, a_log, norm_w, eps: float, rec_state,
                     Hk: int, Hv: int, dk: int, dv: int) -> torch.Tensor:
    """One GatedDeltaNet decode token between the input and output projections in two launches.

    ``mixed`` [B, 1, cd] (q | k | v channels), ``z`` [B, 1, Hv*dv], ``b`` / ``a`` [B, 1, Hv]: column windows of one projection
    output or separate tensors (rows may be strided).  Kernel 1: causal conv + bias + SiLU with ``conv_state`` ([B, cd, K] bf16) shifted in place,
    beta = sigmoid(b), g = -softplus(a + dt_bias) * exp(a_log).  Kernel 2: the recurrent step on ``rec_state`` (fp32
    [B, Hv, dk, dv], in place; L2-normalised q / k inside) with the gated RMSNorm ``norm(o) * norm_w * silu(z)`` in its
    epilogue.  Returns [B, 1, Hv*dv].  Model.lean:642-779 of the reference, which issues library ops."""
    B, _, cd = mixed.shape
    K = conv_state.shape[-1]
    assert b.stride(-1) == 1 and a.stride(-1) == 1 and z.stride(-1) == 1 and b.dtype == a.dtype == z.dtype == torch.bfloat16
    dev = mixed.device
    conv_out = torch.empty((B, cd), dtype=torch.bfloat16, device=dev)
    g = torch.empty((B, Hv), dtype=torch.float32, device=dev)
    beta = torch.empty((B, Hv), dtype=torch.float32, device=dev)
    w = conv_w.reshape(cd, K)
    if w.dtype != torch.bfloat16 or not w.is_contiguous():
        w = w.to(torch.bfloat16).contiguous()
    cb = None if conv_b is None else conv_b.to(torch.bfloat16).contiguous()
    check(lib().tyr_gdn_conv_gates(ptr(mixed), ptr(b), ptr(a), mixed.stride(0), b.stride(0), a.stride(0), ptr(conv_state), ptr(w), ptr(cb), ptr(dt_bias.float().contiguous()),
                                   ptr(a_log.float().contiguous()), ptr(conv_out), ptr(g), ptr(beta), B, cd, K, Hv, cur_stream(dev)),
          "gdn_conv_gates")
    kd = Hk * dk
    q, k, v = conv_out[:, :kd], conv_out[:, kd:2 * kd], conv_out[:, 2 * kd:]
    out = torch.empty((B, 1, Hv * dv), dtype=torch.bfloat16, device=dev)
    nw = norm_w if (norm_w.dtype == torch.bfloat16 and norm_w.is_contiguous()) else norm_w.to(torch.bfloat16).contiguous()
    if _tile_ok(dv, v, z, B * Hv):
        check(lib().tyr_gdr_decode_tile(ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta), ptr(rec_state), ptr(out), B, Hk, Hv, dk, cd, cd,
                                        ptr(z), z.stride(0), ptr(nw), eps, ptr(err_word(dev)), cur_stream(dev)), "gdr_decode_tile")
        return out
    check(lib().tyr_gdr_decode_norm(ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta), ptr(rec_state), ptr(out), B, Hk, Hv, dk, dv, cd, cd,
                                    ptr(z), z.stride(0), ptr(nw), eps, cur_stream(dev)), "gdr_decode_norm")
    return out
