"""NVFP4 banks, routing, layout and the MoE forward on CPU (oracle paths), plus their GPU kernels.

Mirrors the reference's Tests/RunLagunaFused.lean (fused vs eager within 2 % of the output scale,
validation errors) and the quantiser conventions of cc/src/tyr_laguna_moe.cu."""
import pytest
import torch

from tyr_b200.ops import moe
from tyr_b200.ops.gemm import grouped_gemm


def _banks(E, mi, h, device="cpu", seed=0):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: (torch.randn(*s, generator=g) * 0.05).to(device)
    return moe.PackedExperts.quantize(mk(E, mi, h), mk(E, mi, h), mk(E, h, mi))


def test_nvfp4_roundtrip_exact_on_grid():
    # values already on scale * e2m1 grid survive quantise -> dequantise bit-exactly
    lut = moe.E2M1
    codes = torch.randint(0, 16, (2, 8, 64))
    codes[..., ::16] = 7                              # every block holds a 6.0 so the block scale is exact
    scale = torch.tensor([0.5, 2.0]).reshape(2, 1, 1)
    w = lut[codes] * scale
    glob = torch.tensor([1.0, 1.0])
    p, s, g = moe.nvfp4_quantize(w, glob)
    assert torch.equal(moe.nvfp4_dequant(p, s, g).float(), w)
    assert p.dtype == torch.uint8 and p.shape == (2, 8, 32) and s.shape == (2, 8, 4)
    # low nibble first
    assert int(p[0, 0, 0]) & 15 == 7


def test_nvfp4_error_bound_and_validation():
    w = torch.randn(4, 32, 128) * 0.02
    p, s, g = moe.nvfp4_quantize(w)
    d = moe.nvfp4_dequant(p, s, g).float()
    assert ((d - w).norm() / w.norm()).item() < 0.13
    with pytest.raises(ValueError, match="not divisible by 16"):
        moe.nvfp4_quantize(torch.randn(2, 4, 24))


def test_route_sigmoid_bias_only_selects():
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0]])
    ids, w, counts = moe.route(logits, 2, bias=torch.tensor([0.0, 0.0, 0.0, 10.0]))
    assert sorted(ids[0].tolist()) == [0, 3]
    sig = torch.sigmoid(logits[0])
    exp = torch.stack([sig[3], sig[0]]) / (sig[3] + sig[0])
    assert torch.allclose(w[0], exp, atol=1e-6)
    assert counts.tolist() == [1, 0, 0, 1]
    # ties go to the lower index
    ids2, _, _ = moe.route(torch.zeros(1, 8), 3)
    assert ids2[0].tolist() == [0, 1, 2]
    ids3, w3, _ = moe.route(torch.randn(6, 16), 4, softmax=True, renorm=False, scale=2.5)
    assert w3.shape == (6, 4) and (w3.sum(-1) <= 2.5 + 1e-5).all()


def test_layout_is_expert_major_and_stable():
    ids = torch.tensor([[2, 0], [0, 1], [2, 1]], dtype=torch.int32)
    counts = torch.tensor([2, 2, 2], dtype=torch.int32)
    off, order, pos = moe.layout(ids, counts)
    assert off.tolist() == [0, 2, 4, 6]
    assert order.tolist() == [1, 2, 3, 5, 0, 4]
    assert pos[order.long()].tolist() == list(range(6))


def test_moe_forward_matches_dense_oracle_cpu():
    ex = _banks(8, 64, 32)
    ex.validate()
    x = torch.randn(5, 32).bfloat16()
    ids, w, _ = moe.route(torch.randn(5, 8), 2)
    y = moe.moe_fp4_forward(x, ids, w, ex)
    g, u, d = ex.dense()
    ref = torch.zeros(5, 32)
    for t in range(5):
        for s in range(2):
            e = int(ids[t, s])
            hdn = torch.nn.functional.silu(g[e].float() @ x[t].float()) * (u[e].float() @ x[t].float())
            ref[t] += w[t, s] * (d[e].float() @ hdn)
    assert torch.allclose(y.float(), ref, atol=2e-2 * ref.abs().max().item())
    bad = moe.PackedExperts(ex.gate_packed, ex.gate_scale[:, :, :1], ex.gate_global, ex.up_packed, ex.up_scale,
                            ex.up_global, ex.down_packed, ex.down_scale, ex.down_global)
    with pytest.raises(ValueError, match="gate_scale must have shape"):
        bad.validate()


def test_grouped_gemm_cpu_swiglu_layout():
    a = torch.randn(7, 16).bfloat16()
    b = torch.randn(2, 256, 16).bfloat16()
    off = torch.tensor([0, 3, 7], dtype=torch.int32)
    y = grouped_gemm(a, b, off, act="swiglu")
    gate, up = b[1, :128].float(), b[1, 128:].float()
    ref = torch.nn.functional.silu(a[4].float() @ gate.T) * (a[4].float() @ up.T)
    assert torch.allclose(y[4].float(), ref, atol=0.05, rtol=0.02)


# ---------------------------------------------------------------------------------------------------
@pytest.mark.gpu
def test_gpu_nvfp4_quant_dequant_match_cpu():
    w = (torch.randn(6, 96, 256) * 0.03).bfloat16()
    pc, sc, gc = moe.nvfp4_quantize(w.float())
    pg, sg, gg = moe.nvfp4_quantize(w.cuda())
    # the device divides with a 1-ulp-accurate reciprocal: a scale byte may differ by one step on a rounding tie
    ds = (sg.view(torch.uint8).cpu().int() - sc.view(torch.uint8).int()).abs()
    assert ds.max().item() <= 1 and (ds != 0).float().mean().item() < 2e-3
    same = (ds == 0).repeat_interleave(8, dim=-1)
    assert ((pg.cpu() != pc) & same).float().mean().item() < 2e-3
    dg = moe.nvfp4_dequant(pg, sg, gg)
    dc = moe.nvfp4_dequant(pg.cpu(), sg.cpu(), gg.cpu())
    assert torch.equal(dg.cpu(), dc)


@pytest.mark.gpu
@pytest.mark.parametrize("softmax", [False, True])
def test_gpu_route_and_layout(softmax):
    torch.manual_seed(1)
    T, E, k = 77, 256, 10
    logits = torch.randn(T, E)
    bias = torch.randn(E) * 0.05
    ids_c, w_c, cnt_c = moe.route(logits, k, softmax=softmax, bias=bias, softcap=30.0, scale=1.5)
    ids_g, w_g, cnt_g = moe.route(logits.cuda(), k, softmax=softmax, bias=bias.cuda(), softcap=30.0, scale=1.5)
    assert torch.equal(ids_g.cpu().sort(-1).values, ids_c.sort(-1).values)
    assert torch.allclose(w_g.cpu().sort(-1).values, w_c.sort(-1).values, atol=1e-5)
    assert torch.equal(cnt_g.cpu(), cnt_c)
    off, order, pos = moe.layout(ids_g, cnt_g)
    off_c = torch.cat([torch.zeros(1, dtype=torch.int32), cnt_c.cumsum(0).int()])
    assert torch.equal(off.cpu(), off_c)
    flat = ids_g.reshape(-1).cpu()
    o = order.cpu().long()
    assert sorted(o.tolist()) == list(range(T * k))
    assert torch.equal(flat[o], flat[o].sort().values)          # expert-major
    assert torch.equal(pos.cpu()[o], torch.arange(T * k, dtype=torch.int32))


@pytest.mark.gpu
@pytest.mark.parametrize("T,path", [(1, "gemv"), (5, "gemv"), (40, "gemv"), (40, "gemm"), (40, "gemm_sorted"), (128, "gemm"),
                                    (3, "gemm"), (300, "gemm")])
def test_gpu_moe_forward_vs_eager(T, path):
    torch.manual_seed(2)
    E, mi, h, k = 16, 256, 512, 4
    ex = _banks(E, mi, h, device="cuda")
    x = torch.randn(T, h, device="cuda").bfloat16()
    ids, w, cnt = moe.route(torch.randn(T, E, device="cuda"), k)
    add = torch.randn(T, h, device="cuda").bfloat16()
    y = moe.moe_fp4_forward(x, ids, w, ex, counts=cnt, add=add, force_path=path)
    g, u, d = ex.dense()
    ref = moe.moe_eager(x.float(), ids, w, g, u, d) + add.float()
    torch.cuda.synchronize()
    scale = ref.abs().max().item()
    if path == "gemv":       # 16-bit activations on the 4-bit banks: equals the eager loop on the decoded banks
        assert torch.allclose(y.float(), ref, rtol=2e-2, atol=2e-2 * scale), (y.float() - ref).abs().max().item()
    else:                    # block-scaled tensor-core path: activations are 4-bit too (W4A4)
        from tyr_b200.ops import fp4
        same = fp4.moe_fp4_tc_reference(x, ids.long(), w, ex, add=add).float()
        assert ((y.float() - same).norm() / same.norm()).item() < 3e-2
        nrmse = ((y.float() - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt()).item()
        assert nrmse <= 0.35, nrmse          # the reference's W4A4 against W4A16 bar (Tests/RunLagunaFused.lean:307-341)


@pytest.mark.gpu
def test_gpu_moe_fixed_slots_equal_sorted_layout():
    """At most 128 tokens: the fixed-slot path (no sorted layout) against the sorted path; the two run the same quantiser and
    the same tensor-core kernel on the same rows, so the outputs agree bit for bit.  One pair carries an id outside the bank
    (what a rank sees for a pair that belongs elsewhere) and must contribute nothing."""
    from tyr_b200.ops import fp4
    torch.manual_seed(5)
    E, mi, h, k = 16, 256, 512, 4
    ex = _banks(E, mi, h, device="cuda")
    for T in (1, 17, 128):
        x = torch.randn(T, h, device="cuda").bfloat16()
        ids, w, _ = moe.route(torch.randn(T, E, device="cuda"), k)
        add = torch.randn(T, h, device="cuda").bfloat16()
        assert fp4.fixed_slots_supported(T, h)
        y_fixed = moe.moe_fp4_forward(x, ids, w, ex, add=add, force_path="gemm")
        y_sorted = moe.moe_fp4_forward(x, ids, w, ex, add=add, force_path="gemm_sorted")
        assert torch.equal(y_fixed, y_sorted), (y_fixed.float() - y_sorted.float()).abs().max().item()
    ids2 = ids.clone()
    ids2[0, 0] = E + 3
    w2 = w.clone()
    y = fp4.moe_fp4_tc_forward_fixed(x, ids2, w2, ex, add=add)
    w2[0, 0] = 0.0
    ids2[0, 0] = ids[0, 0]
    y_ref = fp4.moe_fp4_tc_forward_fixed(x, ids2, w2, ex, add=add)
    assert torch.isfinite(y.float()).all()
    assert torch.equal(y, y_ref)


@pytest.mark.gpu
def test_gpu_grouped_gemm_empty_and_ragged_groups():
    torch.manual_seed(3)
    G, N, K = 6, 384, 256
    counts = [0, 130, 1, 0, 257, 5]
    off = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device="cuda")
    total = sum(counts)
    a = torch.randn(total, K, device="cuda").bfloat16()
    b = (torch.randn(G, N, K, device="cuda") * 0.1).bfloat16()
    y = grouped_gemm(a, b, off)
    ref = grouped_gemm(a.cpu(), b.cpu(), off.cpu())
    assert torch.allclose(y.float().cpu(), ref.float(), atol=0.05, rtol=0.02)


