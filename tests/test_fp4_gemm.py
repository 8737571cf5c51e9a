"""Block-scaled NVFP4 tensor-core path (csrc/fp4_gemm.cu) against fp32 PyTorch arithmetic on exactly decoded operands.

Accuracy bars of the reference for this path: W4A4 against W4A16 NRMSE <= 0.35, fused against eager rtol 2 % / atol 0.5,
including a 17-token case with skewed routing (Tests/RunLagunaFused.lean:307-341)."""
import pytest
import torch

from tyr_b200.ops import fp4
from tyr_b200.ops import moe as M


def test_scale_order_round_trip_and_formula():
    sf = torch.arange(256 * 8, dtype=torch.int32).reshape(256, 8).to(torch.uint8)
    sw = fp4.swizzle_scales(sf)
    assert torch.equal(fp4.unswizzle_scales(sw, 256, 8), sf)
    for r in (0, 31, 32, 77, 127, 128, 255):
        for kb in range(8):
            off = ((r >> 7) * 2 + (kb >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (kb & 3)
            assert int(sw[off]) == int(sf[r, kb])
    batched = torch.stack([sf, sf.flip(0)])
    assert torch.equal(fp4.swizzle_scales(batched)[1], fp4.swizzle_scales(sf.flip(0)))


def test_reference_quantiser_is_nvfp4():
    """Row quantiser of the oracle: values on the e2m1 grid, block scales UE4M3, error bounded by half a grid step."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(8, 256, generator=g) * torch.logspace(-2, 1, 8)[:, None]
    codes, sb, rs = fp4.quantize_rows_ref(x)
    assert codes.max() <= 15 and torch.equal(sb, sb.to(torch.float8_e4m3fn).float())
    back = fp4.dequant_rows_ref(codes, sb, rs)
    blk_max = x.reshape(8, 16, 16).abs().amax(-1).repeat_interleave(16, 1)
    # half of the largest e2m1 gap (4 -> 6, a third of the block maximum) plus the UE4M3 rounding of the block scale (2^-4)
    assert ((back - x).abs() <= blk_max * (0.5 / 3.0 + 1.0 / 16.0) + 1e-6).all()


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.gpu
@pytest.mark.parametrize("M_,N,K", [(256, 256, 512), (128, 384, 256), (640, 1536, 2048)])
def test_fp4_gemm_dense_matches_decoded_operands(M_, N, K):
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cuda").manual_seed(3)
    x = (torch.randn(M_, K, device=dev, generator=g) * 0.7).bfloat16()
    w = torch.randn(1, N, K, device=dev, generator=g) * 0.05
    # device quantiser against the oracle: identical codes, scales and row scales
    xq, xsf, xrs, _ = fp4.gather_quantize(x, None, None, None, None, 1, M_)
    codes, sb, rs = fp4.quantize_rows_ref(x)
    got_codes = torch.stack([xq & 15, xq >> 4], -1).reshape(M_, K)
    got_sb = fp4.unswizzle_scales(xsf, M_, K // 16).view(torch.float8_e4m3fn).float()
    # the device divides with fast reciprocals: a value that sits on a rounding boundary may land on the neighbouring code
    # or scale; everything else is identical
    assert (got_codes != codes).float().mean().item() < 5e-3
    assert (got_sb != sb).float().mean().item() < 5e-3
    assert torch.allclose(xrs, rs, rtol=1e-5)
    assert _rel(fp4.dequant_rows_ref(got_codes, got_sb, xrs), fp4.dequant_rows_ref(codes, sb, rs)) < 2e-2
    codes, sb, rs = got_codes, got_sb, xrs            # the product below is checked on the operands the kernel really read
    wp, ws, wg = M.nvfp4_quantize(w)
    tiles = torch.tensor([0, M_ // 128], dtype=torch.int32, device=dev)
    rows = torch.tensor([0, M_], dtype=torch.int32, device=dev)
    out = fp4.grouped_gemm_fp4(xq, xsf, xrs, fp4.tile_weights(wp.reshape(1, N, K // 2)), fp4.swizzle_scales(ws.view(torch.uint8))[0].contiguous(), wg,
                               tiles, rows, N, K, mode=0)
    torch.cuda.synchronize()
    a_hat = fp4.dequant_rows_ref(codes, sb, rs)
    w_hat = M.nvfp4_dequant(wp, ws, wg)[0].float()        # exact decode (bf16 holds e2m1 x e4m3 / global only approximately)
    lut = fp4.E2M1_VALUES.to(dev)
    vals = torch.stack([lut[(wp[0] & 15).long()], lut[(wp[0] >> 4).long()]], -1).reshape(N, K)
    w_exact = vals * ws[0].float().repeat_interleave(16, 1) / wg[0]
    ref = a_hat @ w_exact.T
    assert _rel(out, ref) < 6e-3, _rel(out, ref)
    assert (out.float() - ref).abs().max() < 2e-2 * ref.abs().max() + 1e-3
    assert _rel(w_hat, w_exact) < 1e-2


def _experts(E, mi, h, dev, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, device=dev, generator=g)
    return M.PackedExperts.quantize(mk(E, mi, h) * 0.05, mk(E, mi, h) * 0.05, mk(E, h, mi) * 0.05)


@pytest.mark.gpu
@pytest.mark.parametrize("T,E,k,h,mi,skew", [(64, 8, 2, 512, 256, False), (17, 8, 4, 512, 256, True), (300, 16, 4, 1024, 512, False)])
def test_fp4_moe_tensor_core_path(T, E, k, h, mi, skew):
    dev = torch.device("cuda:0")
    ex = _experts(E, mi, h, dev, 7)
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(T, h, device=dev, generator=g).bfloat16()
    if skew:     # every token picks expert 0 first: one large group, several empty ones
        ids = torch.stack([torch.zeros(T, dtype=torch.int64, device=dev)] +
                          [torch.randint(1, 3, (T,), device=dev, generator=g) + 2 * j for j in range(k - 1)], 1).to(torch.int32)
    else:
        ids = torch.stack([torch.randperm(E, device=dev, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    w = torch.rand(T, k, device=dev, generator=g) + 0.1
    add = torch.randn(T, h, device=dev, generator=g).bfloat16()
    counts = M.count_experts(ids, E)
    offsets, order, pos, tiles = M.layout(ids, counts, want_tiles=True)
    out = fp4.moe_fp4_tc_forward(x, ids, w, ex, offsets, order, tiles, add=add)
    torch.cuda.synchronize()
    ref = fp4.moe_fp4_tc_reference(x, ids.long(), w, ex, add=add)
    # against the same arithmetic in fp32.  The device quantisers divide with fast reciprocals, so a value on a rounding
    # boundary may take the neighbouring 4-bit code; such flips move single outputs by more than the reference's
    # rtol 2 % / atol 0.5 in rare cases, hence the bound on their share instead of zero
    d = (out.float() - ref.float()).abs()
    assert (d > 0.5 + 0.02 * ref.float().abs()).float().mean().item() < 2e-3
    assert _rel(out, ref) < 3e-2, _rel(out, ref)
    # stage by stage on the operands the kernels really produced: these comparisons are tight
    w4 = fp4.prepared(ex)
    padded = ((T * k + 127 * min(E, T * k) + 127) // 128) * 128
    xq, xsf, xrs, ppos = fp4.gather_quantize(x, order, ids.reshape(-1).contiguous(), offsets, tiles, k, padded, T * k)
    hq, hsf = fp4.grouped_gemm_fp4(xq, xsf, xrs, w4.gu_packed, w4.gu_sf, w4.gate_global, tiles, offsets,
                                   2 * mi, h, mode=1, w_global2=w4.up_global)
    y = fp4.grouped_gemm_fp4(hq, hsf, None, w4.dn_packed, w4.dn_sf, w4.dn_global, tiles, offsets, h, mi, mode=0)
    torch.cuda.synchronize()
    lut = fp4.E2M1_VALUES.to(dev)

    def dec_rows(packed, sf_flat, cols, rs=None):
        codes = torch.stack([packed & 15, packed >> 4], -1).reshape(packed.shape[0], cols)
        sb = fp4.unswizzle_scales(sf_flat, packed.shape[0], cols // 16).view(torch.float8_e4m3fn).float()
        return fp4.dequant_rows_ref(codes, sb, rs if rs is not None else torch.ones(packed.shape[0], device=dev))

    def dec_bank(packed, scale, glob):
        vals = torch.stack([lut[(packed & 15).long()], lut[(packed >> 4).long()]], -1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
        return vals * scale.view(torch.float8_e4m3fn).float().repeat_interleave(16, dim=-1) / glob.float().reshape(-1, 1, 1)

    gw, uw, dw = dec_bank(ex.gate_packed, ex.gate_scale, ex.gate_global), dec_bank(ex.up_packed, ex.up_scale, ex.up_global), \
        dec_bank(ex.down_packed, ex.down_scale, ex.down_global)
    pp = ppos.long()
    pair_e = ids.reshape(-1).long()
    x_hat = dec_rows(xq, xsf, h, xrs)[pp]                      # quantised activations of every (token, slot) pair
    hid_want = torch.nn.functional.silu(torch.einsum("pk,pnk->pn", x_hat, gw[pair_e])) * torch.einsum("pk,pnk->pn", x_hat, uw[pair_e])
    hid_got = dec_rows(hq, hsf, mi)[pp]
    hid_ref = fp4.dequant_rows_ref(*fp4.quantize_rows_ref(hid_want, per_row_scale=False))
    assert _rel(hid_got, hid_ref) < 2e-2, _rel(hid_got, hid_ref)
    assert (hid_got != hid_ref).float().mean().item() < 1e-2
    y_want = torch.einsum("pk,pnk->pn", hid_got, dw[pair_e])
    assert _rel(y[pp], y_want) < 6e-3, _rel(y[pp], y_want)
    assert (y[pp].float() - y_want).abs().max() < 2e-2 * y_want.abs().max() + 1e-3
    # against 16-bit activations on the same 4-bit weights (the reference's W4A4 vs W4A16 bar)
    gd, ud, dd = ex.dense()
    w4a16 = M.moe_eager(x, ids.long(), w, gd, ud, dd).float() + add.float()
    nrmse = ((out.float() - w4a16).pow(2).mean().sqrt() / (w4a16.pow(2).mean().sqrt() + 1e-12)).item()
    assert nrmse <= 0.35, nrmse
