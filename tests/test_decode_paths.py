"""Host-side logic of the decode-sized kernels' wrappers: CPU fallbacks equal the plain formulas and the path predicates
refuse what the kernels do not take (the kernels themselves are tested on a GPU in test_gpu_kernels.py / test_moe.py /
test_qwen35.py)."""
import torch

from tyr_b200.ops import decode_gemm as DG
from tyr_b200.ops import delta_rule as DR
from tyr_b200.ops import fp4


def test_decode_gemm_cpu_fallback_and_predicate():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(20, 128, generator=g).bfloat16()
    wg = (torch.randn(256, 128, generator=g) * 0.1).bfloat16()
    wu = (torch.randn(256, 128, generator=g) * 0.1).bfloat16()
    assert not DG.supported(x, wg) and not DG.supported(x, wg, wu, min_tiles=1)       # CPU tensors never take the kernel
    ref = x.float() @ wg.float().T
    assert torch.equal(DG.decode_linear(x, wg), ref.to(torch.bfloat16))
    out = torch.zeros(20, 256 + 8, dtype=torch.bfloat16)
    DG.decode_linear(x, wg, out=out[:, 8:])
    assert torch.equal(out[:, 8:], ref.to(torch.bfloat16)) and torch.equal(out[:, :8], torch.zeros(20, 8, dtype=torch.bfloat16))
    gated = (torch.nn.functional.silu(ref) * (x.float() @ wu.float().T)).to(torch.bfloat16)
    assert torch.equal(DG.decode_swiglu(x, wg, wu), gated)


def test_decode_gemm_thresholds_are_ordered():
    # the gated form is taken from fewer tiles than the plain one, and the plain one has an upper bound
    assert DG.MIN_ROWS == 17 and DG.MAX_ROWS == 64
    assert 1 <= DG.MIN_ROW_TILES <= DG.MAX_ROW_TILES
    assert DG.GATED_MIN_ROW_TILES >= 1


def test_fixed_slot_predicate():
    assert not fp4.fixed_slots_supported(129, 2048)            # an expert could receive more rows than a slot tile holds
    assert not fp4.fixed_slots_supported(64, 2048 + 64)        # hidden size must be a multiple of 256
    assert fp4.FIXED_SLOT_MAX_TOKENS == 128


def test_gdr_tile_predicate_needs_aligned_rows(monkeypatch):
    monkeypatch.setattr(DR, "_GDR_TILE_MIN_TILES", 0)
    v = torch.zeros(4, 1, 8 * 128, dtype=torch.bfloat16)
    assert not DR._tile_ok(64, v, None, 32)                     # value head width other than 128
    z = torch.zeros(4, 1, 8 * 128 + 2, dtype=torch.bfloat16)[..., :8 * 128]
    if DR._tile_ok(128, v, None, 32):                            # only when the library carries the kernel
        assert not DR._tile_ok(128, v, z, 32)                    # row stride not a multiple of 4 elements
        monkeypatch.setattr(DR, "_GDR_TILE_MIN_TILES", 64)
        assert not DR._tile_ok(128, v, None, 32)                 # fewer tiles than the threshold
