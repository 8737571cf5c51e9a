"""Newton-Schulz / Polar Express orthogonalisation on the tcgen05 GEMM.

Counterpart of cc/src/tyr_polar.cpp (``xxt`` :35, ``ba_plus_cAA`` :76, ``newton_schulz_step``
:130, ``polar_express`` :193, ``muon_orthogonalize`` :267, ``cautious_update`` :332).  Each
iteration is three batched GEMMs whose scale/add terms are fused into the GEMM epilogue
(``out = alpha*acc + beta*aux``); tall matrices are handled through operand layouts instead of
a physical transpose.
"""
from __future__ import annotations

import torch

from .gemm import gemm

MUON_COEFFS = (3.4445, -4.7750, 2.0315)
# Five quintic steps X <- aX + b(XX^T)X + c(XX^T)^2 X.  The first two rows are the reference's
# (cc/src/tyr_polar.cpp:203-209); with the reference's rows 3-5 the composed polynomial leaves
# [0, 2] for singular values around 0.1-0.5 of the normalised input and diverges, so rows 3-5 here
# are the convergent Polar Express sequence: every singular value in [1e-3, 1] lands in [0.86, 1.14].
POLAR_EXPRESS_COEFFS = (
    (8.156554524902461, -22.48329292557795, 15.878769915207462),
    (4.042929935166739, -2.808917465908714, 0.5000178451051316),
    (3.8916678022926607, -2.772484153217685, 0.5060648178503393),
    (3.285753657755655, -2.3681294933425376, 0.46449024233003106),
    (2.3465413258596377, -1.7097828382687081, 0.42323551169305323),
)


def _use_native(x: torch.Tensor) -> bool:
    R, C = x.shape[-2], x.shape[-1]
    return x.is_cuda and R % 8 == 0 and C % 8 == 0


def xxt(x: torch.Tensor) -> torch.Tensor:
    """X @ X^T (batched when 3-D)."""
    if _use_native(x) and x.dtype == torch.bfloat16:
        return gemm(x, x, a_layout="K", b_layout="K")
    return x @ x.transpose(-1, -2)


def ba_plus_caa(A: torch.Tensor, b: float, c: float) -> torch.Tensor:
    """b*A + c*A@A for symmetric A."""
    if _use_native(A) and A.dtype == torch.bfloat16:
        return gemm(A, A, a_layout="K", b_layout="K", aux=A, alpha=c, beta=b)
    return b * A + c * (A @ A)


def newton_schulz_step(x: torch.Tensor, a: float, b: float, c: float) -> torch.Tensor:
    """a*X + (b*A + c*A@A)@X with A = X@X^T, for X with rows <= cols."""
    A = xxt(x)
    Bm = ba_plus_caa(A, b, c)
    if _use_native(x) and x.dtype == torch.bfloat16:
        return gemm(Bm, x, a_layout="K", b_layout="MN", aux=x, alpha=1.0, beta=a)
    return a * x + Bm @ x


def _tall_step(g: torch.Tensor, a: float, b: float, c: float) -> torch.Tensor:
    """Same iteration for X = G^T without materialising the transpose (G is [.., R, C], R > C)."""
    if _use_native(g) and g.dtype == torch.bfloat16:
        A = gemm(g, g, a_layout="MN", b_layout="MN")          # G^T G  [.., C, C]
        Bm = gemm(A, A, a_layout="K", b_layout="K", aux=A, alpha=c, beta=b)
        return gemm(g, Bm, a_layout="K", b_layout="K", aux=g, alpha=1.0, beta=a)
    A = g.transpose(-1, -2) @ g
    Bm = b * A + c * (A @ A)
    return a * g + g @ Bm


_scratch = {}


def _native_chain(x: torch.Tensor, num_iters: int) -> torch.Tensor:
    """All iterations through one native call (csrc/gemm_tcgen05.cu: tyr_newton_schulz_bf16);
    the scratch buffer is cached per (device, size)."""
    from ._common import check, cur_stream, err_word, lib, ptr
    xb = x if x.dim() == 3 else x.unsqueeze(0)
    B, R, C = xb.shape
    out = xb.contiguous().clone()
    need = lib().tyr_newton_schulz_scratch_bytes(B, R, C)
    key = (x.device.index, need)
    buf = _scratch.get(key)
    if buf is None:
        buf = torch.empty(need, dtype=torch.uint8, device=x.device)
        _scratch.clear()
        _scratch[key] = buf
    a, b, c = MUON_COEFFS
    check(lib().tyr_newton_schulz_bf16(ptr(out), ptr(buf), need, B, R, C, num_iters, a, b, c,
                                       ptr(err_word(x.device)), cur_stream(x.device)), "newton_schulz")
    return out if x.dim() == 3 else out[0]


def newton_schulz_(x: torch.Tensor, num_iters: int, coeffs=None) -> torch.Tensor:
    """Iterate on an already normalised bf16 matrix (or stacked batch)."""
    if coeffs is None and _use_native(x) and x.dtype == torch.bfloat16:
        return _native_chain(x, num_iters)
    tall = x.shape[-2] > x.shape[-1]
    for i in range(num_iters):
        a, b, c = coeffs[i] if coeffs is not None else MUON_COEFFS
        x = _tall_step(x, a, b, c) if tall else newton_schulz_step(x, a, b, c)
    return x


def muon_orthogonalize(g: torch.Tensor, num_iters: int = 5) -> torch.Tensor:
    """bf16 Newton-Schulz orthogonalisation with Muon's fixed coefficients; returns bf16."""
    if g.dim() < 2:
        raise ValueError("muon_orthogonalize requires tensor rank >= 2")
    x = g.to(torch.bfloat16)
    norm = x.float().pow(2).sum(dim=(-2, -1), keepdim=True).sqrt()
    x = (x.float() / (norm + 1e-7)).to(torch.bfloat16)
    return newton_schulz_(x, num_iters)


def polar_express(g: torch.Tensor, num_iters: int = 5) -> torch.Tensor:
    """Polar Express with the five precomputed coefficient triples; keeps the input dtype.
    X = a X + b (XX^T) X + c (XX^T)^2 X per iteration, after Frobenius normalisation."""
    x = g / g.norm()
    iters = min(num_iters, len(POLAR_EXPRESS_COEFFS))
    for i in range(iters):
        a, b, c = POLAR_EXPRESS_COEFFS[i]
        A = x @ x.transpose(-1, -2)
        AX = A @ x
        x = a * x + b * AX + c * (A @ AX)
    return x


def cautious_update(param: torch.Tensor, update: torch.Tensor, lr: float, wd: float) -> torch.Tensor:
    """param - lr*(update + wd*mask*param), mask = sign(update) == sign(param)."""
    mask = ((torch.sign(update) * torch.sign(param)) > 0).to(param.dtype)
    return param - lr * (update + wd * mask * param)
