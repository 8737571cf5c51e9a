"""Numerics of every hand-written kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda:0")


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.fixture(autouse=True)
def _check_error_word():
    yield
    from tyr_b200.ops._common import raise_on_device_error
    torch.cuda.synchronize()
    raise_on_device_error()


@pytest.mark.parametrize("a_layout,b_layout", [("K", "K"), ("K", "MN"), ("MN", "MN"), ("MN", "K")])
@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (384, 320, 192), (1000, 264, 520), (128, 128, 64)])
def test_gemm_layouts(a_layout, b_layout, M, N, K):
    from tyr_b200.ops.gemm import gemm
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn((M, K) if a_layout == "K" else (K, M), device=_dev(), generator=g).bfloat16()
    b = torch.randn((N, K) if b_layout == "K" else (K, N), device=_dev(), generator=g).bfloat16()
    out = gemm(a, b, a_layout=a_layout, b_layout=b_layout)
    A = a.float() if a_layout == "K" else a.float().t()
    B = b.float().t() if b_layout == "K" else b.float()
    ref = A @ B
    assert out.shape == (M, N) and out.dtype == torch.bfloat16
    assert _rel_err(out, ref) < 1e-2, _rel_err(out, ref)


@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_epilogues_and_batch(bn):
    from tyr_b200.ops.gemm import gemm
    g = torch.Generator(device="cuda").manual_seed(2)
    Bt, M, N, K = 3, 256, 384, 320
    a = torch.randn(Bt, M, K, device=_dev(), generator=g).bfloat16()
    b = torch.randn(Bt, N, K, device=_dev(), generator=g).bfloat16()
    aux = torch.randn(Bt, M, N, device=_dev(), generator=g).bfloat16()
    out = gemm(a, b, aux=aux, alpha=0.5, beta=-1.5, bn=bn)
    ref = 0.5 * torch.bmm(a.float(), b.float().transpose(1, 2)) - 1.5 * aux.float()
    assert _rel_err(out, ref) < 1e-2
    out = gemm(a, b, act="relu2", bn=bn)
    ref = torch.relu(torch.bmm(a.float(), b.float().transpose(1, 2))) ** 2
    assert _rel_err(out, ref) < 1e-2
    out32 = gemm(a, b, out_dtype=torch.float32, bn=bn)
    assert out32.dtype == torch.float32
    assert _rel_err(out32, torch.bmm(a.float(), b.float().transpose(1, 2))) < 2e-3
    y = torch.rand(Bt, M, N, device=_dev(), generator=g).bfloat16()
    outg = gemm(a, b, act="relu2_grad", aux=y, bn=bn)
    refg = torch.bmm(a.float(), b.float().transpose(1, 2)) * 2 * y.float().sqrt()
    assert _rel_err(outg, refg) < 1e-2


def _assert_elementwise(out, ref, K, what=""):
    """Per-element bound: the bf16 (or fp32) rounding of the result plus an accumulation term that grows like sqrt(K).
    One wrong output tile breaks it by orders of magnitude, which a norm ratio over a large matrix does not show."""
    out, ref = out.float(), ref.float()
    err = (out - ref).abs()
    bound = 2.0 ** -7 * ref.abs() + 4e-3 * math.sqrt(K) + 1e-3
    bad = err > bound
    assert not bool(bad.any()), (what, int(bad.sum()), float(err.max()), bad.nonzero()[:4].tolist())


@pytest.mark.parametrize("M,N,K,b_layout", [
    (65536, 3840, 1280, "K"),      # forward qkv projection of the d20 model (CTA pairs, 52 rounds of 256 x 256 tiles)
    (65536, 1280, 5120, "MN"),     # data gradient of the MLP up-projection
    (8192, 65536, 1280, "K"),      # lm_head chunk: row-fastest tile order
    (1000, 2000, 328, "K"),        # ragged edges in every dimension, second CTA of the last pair partly out of range
    (130, 384, 64, "MN"),          # the pair's second CTA holds 2 valid rows
])
def test_gemm_production_shapes_elementwise(M, N, K, b_layout):
    from tyr_b200.ops.gemm import gemm
    g = torch.Generator(device="cuda").manual_seed(11)
    a = torch.randn(M, K, device=_dev(), generator=g).bfloat16()
    b = torch.randn((N, K) if b_layout == "K" else (K, N), device=_dev(), generator=g).bfloat16()
    out = gemm(a, b, b_layout=b_layout)
    step = 8192
    for r0 in range(0, M, step):      # reference in row slabs: keeps the fp32 product small
        ref = a[r0:r0 + step].float() @ (b.float().t() if b_layout == "K" else b.float())
        _assert_elementwise(out[r0:r0 + step], ref, K, f"rows {r0}")
    assert _rel_err(out[:4096], a[:4096].float() @ (b.float().t() if b_layout == "K" else b.float())) < 5e-3


def test_gemm_wgrad_production_shape_elementwise():
    """K = 65536 weight gradient (MN/MN, fp32 accumulate): whole-tile rounds plus a k-slab remainder on all SMs."""
    from tyr_b200.ops.gemm import gemm
    g = torch.Generator(device="cuda").manual_seed(12)
    Kt, M, N = 65536, 5120, 1280
    dy = torch.randn(Kt, M, device=_dev(), generator=g).bfloat16()
    x = torch.randn(Kt, N, device=_dev(), generator=g).bfloat16()
    acc = torch.zeros(M, N, device=_dev(), dtype=torch.float32)
    gemm(dy, x, a_layout="MN", b_layout="MN", out=acc, accumulate=True)
    ref = dy.float().t() @ x.float()
    err = (acc - ref).abs()
    assert float(err.max()) < 0.05 * math.sqrt(Kt) * 2.0 ** -8 + 1e-1, float(err.max())
    assert _rel_err(acc, ref) < 1e-3


@pytest.mark.parametrize("Kt,M,N", [(4096, 384, 256), (1024, 2048, 2560), (704, 1344, 520), (64, 19072, 256)])
def test_gemm_stream_k_accumulate(Kt, M, N):
    """Fewer tiles than SMs, a whole round of tiles plus a remainder, ragged edges, and a single k block."""
    from tyr_b200.ops.gemm import gemm
    g = torch.Generator(device="cuda").manual_seed(3)
    dy = torch.randn(Kt, M, device=_dev(), generator=g).bfloat16()
    x = torch.randn(Kt, N, device=_dev(), generator=g).bfloat16()
    acc = torch.ones(M, N, device=_dev(), dtype=torch.float32)
    gemm(dy, x, a_layout="MN", b_layout="MN", out=acc, accumulate=True)
    ref = 1.0 + dy.float().t() @ x.float()
    assert _rel_err(acc, ref) < 2e-3
    # deterministic partition: a second run into a fresh buffer agrees to fp32 rounding
    acc2 = torch.ones(M, N, device=_dev(), dtype=torch.float32)
    gemm(dy, x, a_layout="MN", b_layout="MN", out=acc2, accumulate=True)
    assert _rel_err(acc2, acc) < 1e-5


def test_linear_autograd():
    from tyr_b200.ops.gemm import linear
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(512, 256, device=_dev(), generator=g).bfloat16().requires_grad_(True)
    w = (torch.randn(384, 256, device=_dev(), generator=g) * 0.1).bfloat16().requires_grad_(True)
    dy = torch.randn(512, 384, device=_dev(), generator=g).bfloat16()
    y = linear(x, w)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    (xr @ wr.t()).backward(dy.float())
    assert _rel_err(y, xr @ wr.t()) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 1e-2


@pytest.mark.parametrize("n_in", [1, 2, 3, 4])
def test_lincomb_rmsnorm(n_in):
    from tyr_b200.ops.norm import lincomb_rmsnorm, rms_norm_ref
    g = torch.Generator(device="cuda").manual_seed(5)
    rows, D = 300, 1280
    ts = [torch.randn(rows, D, device=_dev(), generator=g).bfloat16().requires_grad_(True) for _ in range(n_in)]
    sc = (torch.rand(n_in, device=_dev(), generator=g) + 0.5).requires_grad_(True)
    out, normed = lincomb_rmsnorm(ts, sc)
    d_out = torch.randn(rows, D, device=_dev(), generator=g).bfloat16()
    d_n = torch.randn(rows, D, device=_dev(), generator=g).bfloat16()
    torch.autograd.backward([out, normed], [d_out, d_n])
    tr = [t.detach().float().requires_grad_(True) for t in ts]
    sr = sc.detach().clone().requires_grad_(True)
    o_ref = sum(sr[i] * tr[i] for i in range(n_in))
    n_ref = rms_norm_ref(o_ref)
    torch.autograd.backward([o_ref, n_ref], [d_out.float(), d_n.float()])
    assert _rel_err(out, o_ref) < 1e-2 and _rel_err(normed, n_ref) < 1e-2
    for t, r in zip(ts, tr):
        assert _rel_err(t.grad, r.grad) < 2e-2
    assert _rel_err(sc.grad, sr.grad) < 2e-2


def test_qkv_post_fwd_bwd():
    from tyr_b200.ops.rope import qkv_post, qkv_post_ref, rotary_freqs
    g = torch.Generator(device="cuda").manual_seed(6)
    B, T, H, D = 2, 96, 3, 128
    qkv = torch.randn(B * T, 3 * H * D, device=_dev(), generator=g).bfloat16().requires_grad_(True)
    ve = torch.randn(B * T, H * D, device=_dev(), generator=g).bfloat16().requires_grad_(True)
    mix = torch.tensor(0.7, device=_dev()).requires_grad_(True)
    cos, sin = rotary_freqs(T, D, 500000.0, device=_dev())
    out = qkv_post(qkv, ve, mix, cos, sin, T, H, D)
    dy = torch.randn_like(out)
    out.backward(dy)
    q_r = qkv.detach().float().requires_grad_(True)
    v_r = ve.detach().float().requires_grad_(True)
    m_r = mix.detach().clone().requires_grad_(True)
    ref = qkv_post_ref(q_r, v_r, m_r, cos, sin, T, H, D)
    ref.backward(dy.float())
    assert _rel_err(out, ref) < 1e-2
    assert _rel_err(qkv.grad, q_r.grad) < 2e-2
    assert _rel_err(ve.grad, v_r.grad) < 2e-2
    assert abs(mix.grad.item() - m_r.grad.item()) < 2e-2 * abs(m_r.grad.item()) + 1e-2


def test_softcap_ce_kernel_and_lm_head():
    from tyr_b200.ops.ce import lm_head_ce, softcap_ce_, softcap_ce_ref
    g = torch.Generator(device="cuda").manual_seed(7)
    rows, V = 64, 4096
    logits = (torch.randn(rows, V, device=_dev(), generator=g) * 4).bfloat16()
    t = torch.randint(0, V, (rows,), device=_dev(), generator=g)
    t[3] = -100
    lr = logits.detach().float().requires_grad_(True)
    ref = softcap_ce_ref(lr, t, 15.0)
    ref.sum().backward()
    work = logits.clone()
    loss = softcap_ce_(work, t, 15.0, 1.0)
    assert torch.allclose(loss, ref, rtol=2e-3, atol=2e-3)
    assert _rel_err(work, lr.grad) < 2e-2
    # fused head
    N, d = 512, 256
    x = torch.randn(N, d, device=_dev(), generator=g).bfloat16().requires_grad_(True)
    w = (torch.randn(V, d, device=_dev(), generator=g) * 0.1).bfloat16().requires_grad_(True)
    tt = torch.randint(0, V, (N,), device=_dev(), generator=g)
    l = lm_head_ce(x, w, tt, cap=15.0, chunk_rows=200)
    l.backward()
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    lref = torch.nn.functional.cross_entropy(15 * torch.tanh((xr @ wr.t()) / 15), tt)
    lref.backward()
    assert abs(l.item() - lref.item()) < 2e-2
    assert _rel_err(x.grad, xr.grad) < 3e-2
    assert _rel_err(w.grad, wr.grad) < 3e-2


def test_adamw_and_muon_kernels():
    from tyr_b200.ops import optim_kernels as ok
    from tyr_b200.ops import polar
    g = torch.Generator(device="cuda").manual_seed(8)
    n = 1000 * 37 + 3
    p = torch.randn(n, device=_dev(), generator=g)
    grad = torch.randn(n, device=_dev(), generator=g).bfloat16()
    m = torch.zeros(n, device=_dev())
    v = torch.zeros(n, device=_dev())
    pb = torch.empty(n, device=_dev(), dtype=torch.bfloat16)
    pc, mc, vc = p.cpu().clone(), m.cpu().clone(), v.cpu().clone()
    for step in (1, 2, 3):
        ok.adamw_step_(p, grad, m, v, lr=0.01, beta1=0.8, beta2=0.95, eps=1e-10, weight_decay=0.1, step=step, p_bf16=pb)
        ok.adamw_step_(pc, grad.cpu(), mc, vc, lr=0.01, beta1=0.8, beta2=0.95, eps=1e-10, weight_decay=0.1, step=step)
    assert torch.allclose(p.cpu(), pc, rtol=1e-4, atol=1e-5)
    assert torch.allclose(pb.float().cpu(), pc.bfloat16().float(), rtol=1e-2, atol=1e-2)
    # Muon pieces
    Bm, R, C = 3, 256, 512
    gr = torch.randn(Bm, R, C, device=_dev(), generator=g)
    mom = torch.randn(Bm, R, C, device=_dev(), generator=g) * 0.1
    u = torch.empty(Bm, R, C, device=_dev(), dtype=torch.bfloat16)
    ss = torch.zeros(Bm, device=_dev())
    mom_ref = 0.9 * mom + 0.1 * gr
    u_ref = 0.1 * gr + 0.9 * mom_ref
    ok.muon_momentum_(gr, mom, u, ss, 0.9)
    assert torch.allclose(mom, mom_ref, rtol=1e-5, atol=1e-6)
    assert _rel_err(u, u_ref) < 1e-2
    assert torch.allclose(ss, u.float().pow(2).sum((1, 2)), rtol=1e-3)
    ok.scale_by_inv_norm_(u, ss)
    assert torch.allclose(u.float().pow(2).sum((1, 2)), torch.ones(Bm, device=_dev()), rtol=2e-2)
    o = polar.newton_schulz_(u, 5)
    # oracle: same iteration in fp32
    x = u.float()
    a, b, c = polar.MUON_COEFFS
    for _ in range(5):
        A = x @ x.transpose(1, 2)
        x = a * x + (b * A + c * A @ A) @ x
    assert _rel_err(o, x) < 5e-2
    sv = torch.linalg.svdvals(o.float())
    assert sv.max() < 1.35 and sv.min() > 0.3
    # tall matrices go through the transposed-operand path
    ut = u.transpose(1, 2).contiguous()
    ot = polar.newton_schulz_(ut, 5)
    assert _rel_err(ot, x.transpose(1, 2)) < 5e-2
    pm = torch.randn(Bm, R, C, device=_dev(), generator=g)
    pm_ref = pm * (1 - 0.02 * 0.5) - (o.float() * 0.02).bfloat16().float()
    pbf = torch.empty(Bm, R, C, device=_dev(), dtype=torch.bfloat16)
    ok.muon_apply_(pm, o.contiguous(), 0.02, 0.5, pbf)
    assert torch.allclose(pm, pm_ref, rtol=1e-5, atol=1e-6)


def test_rmsnorm_weighted_and_rope_norm():
    from tyr_b200.ops.norm import rms_norm_weighted
    from tyr_b200.ops.rope import rope_norm, rotary_freqs
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn(100, 2048, device=_dev(), generator=g).bfloat16()
    w = torch.randn(2048, device=_dev(), generator=g).bfloat16()
    r = torch.randn(100, 2048, device=_dev(), generator=g).bfloat16()
    gate = torch.randn(100, 2048, device=_dev(), generator=g).bfloat16()
    y, ro = rms_norm_weighted(x, w, one_plus_w=True, gate=gate, residual=r, return_residual=True)
    y_ref, ro_ref = rms_norm_weighted(x.cpu(), w.cpu(), one_plus_w=True, gate=gate.cpu(), residual=r.cpu(), return_residual=True)
    assert _rel_err(y.cpu(), y_ref) < 1e-2 and _rel_err(ro.cpu(), ro_ref) < 1e-2
    rows, H, D, rot = 50, 4, 256, 64
    xx = torch.randn(rows, H, D, device=_dev(), generator=g).bfloat16()
    wn = torch.randn(D, device=_dev(), generator=g).bfloat16()
    cos, sin = rotary_freqs(128, rot, 10000.0, device=_dev())
    pos = torch.randint(0, 128, (rows,), device=_dev(), generator=g)
    yy = rope_norm(xx, cos, sin, weight=wn, positions=pos, rot=rot, one_plus_w=True)
    yy_ref = rope_norm(xx.cpu(), cos.cpu(), sin.cpu(), weight=wn.cpu(), positions=pos.cpu(), rot=rot, one_plus_w=True)
    assert _rel_err(yy.cpu(), yy_ref) < 1e-2


@pytest.mark.parametrize("rows,D", [(64, 5120), (7, 8192), (33, 1024), (3000, 2048), (64, 512)])
def test_rmsnorm_weighted_row_and_warp_kernels(rows, D):
    """Decode-sized inputs take the one-CTA-per-row kernel, the rest one warp per row; both against the fp32 formula."""
    from tyr_b200.ops.norm import rms_norm_weighted
    g = torch.Generator(device="cuda").manual_seed(rows + D)
    x = torch.randn(rows, D, device=_dev(), generator=g).bfloat16()
    w = (0.1 * torch.randn(D, device=_dev(), generator=g)).bfloat16()
    r = torch.randn(rows, D, device=_dev(), generator=g).bfloat16()
    y, ro = rms_norm_weighted(x, w, 1e-6, one_plus_w=True, residual=r, return_residual=True)
    s_ref = (x.float() + r.float()).bfloat16()
    y_ref = s_ref.float() * torch.rsqrt(s_ref.float().pow(2).mean(-1, keepdim=True) + 1e-6) * (1 + w.float())
    assert torch.equal(ro, s_ref)
    assert (y.float() - y_ref).abs().max().item() < 2e-2 * max(1.0, y_ref.abs().max().item())
    y2 = rms_norm_weighted(x, w, 1e-6)
    y2_ref = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    assert (y2.float() - y2_ref).abs().max().item() < 2e-2 * max(1.0, y2_ref.abs().max().item())


def test_embedding_grad_sorted_matches_index_add():
    """Zipf-like tokens (a few ids own most rows), row strides of a packed buffer, ids at both ends of the table."""
    from tyr_b200.ops import embed
    g = torch.Generator(device="cuda").manual_seed(4)
    N, d, V = 5000, 256, 1000
    idx = (torch.rand(N, device=_dev(), generator=g) ** 6 * V).long().clamp(0, V - 1)
    idx[:3] = torch.tensor([0, V - 1, V - 1], device=_dev())
    big = torch.randn(N, 3 * d, device=_dev(), generator=g).bfloat16()
    dy = big[:, d:2 * d]                                   # strided rows
    table = torch.randn(V, d, device=_dev(), generator=g)
    want = table.clone().index_add_(0, idx, dy.float())
    got = table.clone()
    embed.embedding_grad_(got, dy, idx)
    torch.cuda.synchronize()
    assert (got - want).abs().max().item() < 1e-3 * max(1.0, want.abs().max().item())
    untouched = torch.ones(V, dtype=torch.bool, device=_dev())
    untouched[idx] = False
    assert torch.equal(got[untouched], table[untouched])


def test_nanochat_step_graph_matches_eager_steps():
    """Forward + backward replayed from a CUDA graph (after two eager steps) trains like the eager step: same losses and
    parameters over six steps on changing batches, up to the fp32 summation order of the split-K weight gradients."""
    from tyr_b200.models import nanochat as nc
    from tyr_b200.train import nanochat_engine as eng
    cfg = nc.Config(vocab_size=2048, n_layer=7, n_head=2, half_head_dim=64, max_seq_len=128)
    hp = eng.Hyperparameters(device_batch_size=4, max_seq_len=128, total_batch_size_tokens=512)
    gen = torch.Generator().manual_seed(5)
    toks = [torch.randint(0, cfg.vocab_size, (4, 129), generator=gen).to(_dev()) for _ in range(6)]
    runs = []
    for graphed in (False, True):
        tr = eng.NanoChatTrainer(cfg, hp, device=_dev(), compute_dtype=torch.bfloat16, seed=3, ce_chunk_rows=256)
        tr._graph_enabled = graphed
        losses = [float(tr.step([(t[:, :-1], t[:, 1:])]).loss.item()) for t in toks]
        torch.cuda.synchronize()
        if graphed:
            assert tr._graph is not None and tr._graph_launches > 50, "the step graph was not captured"
        runs.append((losses, {k: v.detach().clone() for k, v in tr.params.master.items()}))
    (l0, p0), (l1, p1) = runs
    for a, b in zip(l0, l1):
        assert abs(a - b) < 2e-2 * max(1.0, abs(a)), (l0, l1)
    assert l0[-1] < l0[0]
    for k in p0:
        assert _rel_err(p1[k], p0[k]) < 2e-2, k


def test_nanochat_fused_vs_reference_gpu():
    from tyr_b200.models import nanochat as nc
    cfg = nc.Config(vocab_size=2048, n_layer=7, n_head=2, half_head_dim=64, max_seq_len=128)
    params = nc.ModdedGPTParams(cfg, device=_dev(), compute_dtype=torch.bfloat16, seed=1)
    gen = torch.Generator().manual_seed(0)
    with torch.no_grad():
        for k, v in params.master.items():
            if k == "scalars":
                v.copy_((1.1 + 0.3 * torch.randn(v.shape, generator=gen)).to(v.device))
            else:
                v.copy_((torch.randn(v.shape, generator=gen) * 0.05).to(v.device))
    params.sync_work_from_master()
    params.refresh_leaves()
    B, T = 4, 128
    x = torch.randint(0, cfg.vocab_size, (B, T), generator=gen).to(_dev())
    y = torch.randint(0, cfg.vocab_size, (B, T), generator=gen).to(_dev())
    params.zero_grads()
    loss = nc.loss_fused(params, x, y, ce_chunk_rows=200)
    loss.backward()
    ref_p = {k: v.detach().clone().requires_grad_(True) for k, v in params.named_parameters("master").items()}
    ref_loss = nc.loss_reference(ref_p, cfg, x, y, params.cos, params.sin)
    ref_loss.backward()
    assert abs(loss.item() - ref_loss.item()) < 3e-2, (loss.item(), ref_loss.item())
    grads = params.named_parameters("grad")
    for name in ("blocks.0.attn.wQ", "blocks.3.attn.wO", "blocks.5.mlp.cFc", "blocks.6.mlp.cProj",
                 "lmHead.weight", "embed", "valueEmbeds.1"):
        e = _rel_err(grads[name], ref_p[name].grad)
        assert e < 8e-2, (name, e)
    e = _rel_err(params.work["scalars"].grad, ref_p["scalars.values"].grad)
    assert e < 8e-2, ("scalars", e)


@pytest.mark.parametrize("B,Hq,Hkv,Tq,Tk,causal,window", [
    (2, 2, 2, 256, 256, True, None),
    (1, 4, 2, 384, 384, True, None),
    (2, 2, 2, 512, 512, True, 200),
    (1, 2, 2, 200, 200, True, None),
    (1, 2, 1, 300, 300, False, None),
    (1, 2, 2, 128, 640, True, None),
    (2, 3, 3, 1024, 1024, True, None),
    (2, 6, 2, 1, 190, False, None),
    (2, 4, 2, 1, 128, False, None),
    (1, 8, 8, 1, 191, True, None),
    (2, 6, 2, 16, 300, True, None),
])
def test_flash_attention_forward(B, Hq, Hkv, Tq, Tk, causal, window):
    from tyr_b200.ops import flash
    from tyr_b200.ops.attention import attention_ref
    if not flash.has_fwd():
        pytest.skip("flash forward kernel not built")
    g = torch.Generator(device="cuda").manual_seed(11)
    D = 128
    q = torch.randn(B, Tq, Hq, D, device=_dev(), generator=g).bfloat16()
    k = torch.randn(B, Tk, Hkv, D, device=_dev(), generator=g).bfloat16()
    v = torch.randn(B, Tk, Hkv, D, device=_dev(), generator=g).bfloat16()
    o, lse = flash.flash_fwd_bthd(q, k, v, causal=causal, window=window, scale=None)
    ref = attention_ref(q.transpose(1, 2).float(), k.transpose(1, 2).float(), v.transpose(1, 2).float(),
                        causal=causal, window=window).transpose(1, 2)
    assert _rel_err(o, ref) < 2e-2, _rel_err(o, ref)
    # log-sum-exp against the explicit scores
    rep = Hq // Hkv
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float().repeat_interleave(rep, dim=2)) / math.sqrt(D)
    qi = torch.arange(Tq, device=_dev())[:, None] + (Tk - Tq)
    ki = torch.arange(Tk, device=_dev())[None, :]
    m = torch.ones(Tq, Tk, dtype=torch.bool, device=_dev())
    if causal:
        m &= ki <= qi
    if window:
        m &= ki > qi - window
    s = s.masked_fill(~m, float("-inf"))
    assert torch.allclose(lse, torch.logsumexp(s, -1), rtol=1e-2, atol=2e-2)


@pytest.mark.parametrize("B,Hq,Hkv,Tq,Tk,causal,window", [
    (2, 2, 2, 256, 256, True, None),
    (1, 4, 2, 384, 384, True, None),
    (2, 2, 2, 512, 512, True, 200),
    (1, 2, 2, 200, 200, True, None),
    (1, 2, 1, 300, 300, False, None),
    (1, 2, 2, 128, 640, True, None),
    (1, 3, 3, 1024, 1024, True, None),
    (2, 6, 2, 16, 300, True, None),
])
def test_flash_attention_backward(B, Hq, Hkv, Tq, Tk, causal, window):
    """dQ, dK, dV of the tcgen05 backward against fp32 autograd through the explicit masked softmax."""
    from tyr_b200.ops import flash
    from tyr_b200.ops._common import err_word
    from tyr_b200.ops.attention import attention_ref
    if not (flash.has_fwd() and flash.has_bwd()):
        pytest.skip("flash kernels not built")
    g = torch.Generator(device="cuda").manual_seed(5)
    D = 128
    q = torch.randn(B, Tq, Hq, D, device=_dev(), generator=g).bfloat16()
    k = torch.randn(B, Tk, Hkv, D, device=_dev(), generator=g).bfloat16()
    v = torch.randn(B, Tk, Hkv, D, device=_dev(), generator=g).bfloat16()
    do = torch.randn(B, Tq, Hq, D, device=_dev(), generator=g).bfloat16()
    o, lse = flash.flash_fwd_bthd(q, k, v, causal=causal, window=window, scale=None)
    dq, dk, dv, _ = flash.flash_bwd_bthd(do, q, k, v, o, lse, causal=causal, window=window, scale=None)
    torch.cuda.synchronize()
    assert err_word(_dev()).tolist()[0] == 0, err_word(_dev()).tolist()
    qf, kf, vf = (t.float().transpose(1, 2).requires_grad_() for t in (q, k, v))
    ref = attention_ref(qf, kf, vf, causal=causal, window=window)
    ref.backward(do.float().transpose(1, 2))
    for name, got, want in (("dq", dq, qf.grad), ("dk", dk, kf.grad), ("dv", dv, vf.grad)):
        e = _rel_err(got, want.transpose(1, 2))
        assert e < 3e-2, (name, e)


@pytest.mark.parametrize("B,Hq,Hkv,D,cap,pos,ring,window,splits", [
    (2, 6, 1, 128, 700, 513, False, None, None), (3, 8, 2, 256, 300, 299, False, 100, 4), (2, 4, 4, 64, 64, 200, True, None, 2),
    (64, 48, 8, 128, 1100, 1024, False, None, None), (1, 8, 1, 128, 96, 5, True, None, 3), (2, 12, 2, 128, 50, 0, False, None, 1),
    (4, 72, 8, 128, 512, 777, True, None, None), (2, 16, 1, 64, 200, 150, False, 64, 2), (1, 9, 1, 128, 40, 17, False, None, 1)])
def test_decode_attention_matches_reference(B, Hq, Hkv, D, cap, pos, ring, window, splits):
    from tyr_b200.ops.decode_attention import decode_attention
    g = torch.Generator().manual_seed(pos + D)
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16)
    q, kn, vn, kc, vc = mk(B, Hq, D), mk(B, Hkv, D), mk(B, Hkv, D), mk(B, Hkv, cap, D), mk(B, Hkv, cap, D)
    pt = torch.tensor([pos], dtype=torch.int32)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    ref = decode_attention(q, kn, vn, kc_ref, vc_ref, pt, ring=ring, window=window)
    kd, vd = kc.cuda(), vc.cuda()
    wide = torch.randn(B, (Hq + 2 * Hkv) * D + 8, generator=g).to(torch.bfloat16).cuda()      # q / k / v as column slices of one projection
    wide[:, :Hq * D], wide[:, Hq * D:(Hq + Hkv) * D], wide[:, (Hq + Hkv) * D:(Hq + 2 * Hkv) * D] = q.reshape(B, -1).cuda(), kn.reshape(B, -1).cuda(), vn.reshape(B, -1).cuda()
    qv = wide[:, :Hq * D].view(B, Hq, D)
    kv = wide[:, Hq * D:(Hq + Hkv) * D].view(B, Hkv, D)
    vv = wide[:, (Hq + Hkv) * D:(Hq + 2 * Hkv) * D].view(B, Hkv, D)
    for _ in range(2):                                   # a second launch checks that the ticket counters were reset
        out = decode_attention(qv, kv, vv, kd, vd, pt.cuda(), ring=ring, window=window, splits=splits)
    torch.cuda.synchronize()
    assert torch.equal(kd.cpu(), kc_ref) and torch.equal(vd.cpu(), vc_ref)
    assert (out.float().cpu() - ref.float()).abs().max() < 2e-2
    # output gates folded into the final write: per head softplus, per element sigmoid (strided views of wider rows)
    hg = torch.randn(B, Hq + 3, generator=g).to(torch.bfloat16).cuda()[:, 1:Hq + 1]
    eg = torch.randn(B, Hq, 2 * D, generator=g).to(torch.bfloat16).cuda()[..., D:]
    for kw, factor in (({"head_gate": hg}, torch.nn.functional.softplus(hg.float()).unsqueeze(-1)), ({"elem_gate": eg}, torch.sigmoid(eg.float()))):
        got = decode_attention(qv, kv, vv, kd, vd, pt.cuda(), ring=ring, window=window, splits=splits, append=False, **kw)
        want = out.float() * factor
        assert (got.float() - want).abs().max().item() < 2e-2 * max(1.0, want.abs().max().item()), list(kw)


@pytest.mark.parametrize("M,N,K", [(17, 512, 1024), (32, 2176, 5120), (33, 300, 192), (64, 1152, 4096), (48, 128, 64)])
def test_decode_gemm_tensor_core_matches_reference(M, N, K):
    """Weights on the 128-row side of tcgen05.mma, 17 .. 64 tokens on the narrow side: plain and gated, ragged row counts
    (the last CTA's weight tile runs past N), strided output and strided weight rows."""
    from tyr_b200.ops import decode_gemm as DG
    g = torch.Generator().manual_seed(M * 7 + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    wcat = (torch.randn(2 * N, K + 8, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    wg, wu = wcat[:N, :K], wcat[N:, :K]                                # row stride K + 8: a window of a wider matrix
    assert DG.supported(x, wg, wu, min_tiles=1) and DG.supported(x, wg, min_tiles=1)
    ref_g, ref_u = x.float() @ wg.float().T, x.float() @ wu.float().T
    buf = torch.zeros(M, N + 16, dtype=torch.bfloat16, device="cuda")
    DG.decode_linear(x, wg, out=buf[:, 8:8 + N])
    assert (buf[:, 8:8 + N].float() - ref_g).abs().max().item() < 2e-2 * max(1.0, ref_g.abs().max().item())
    assert torch.equal(buf[:, :8], torch.zeros_like(buf[:, :8])) and torch.equal(buf[:, 8 + N:], torch.zeros_like(buf[:, 8 + N:]))
    ref = torch.nn.functional.silu(ref_g) * ref_u
    got = DG.decode_swiglu(x, wg, wu)
    assert (got.float() - ref).abs().max().item() < 2e-2 * max(1.0, ref.abs().max().item())
    # contraction split over the CTAs of a cluster, partial sums through distributed shared memory
    for split in (1, 2, 3, 4):
        if K // 64 < split or (split == 4 and M > 32):
            continue
        got = DG.decode_swiglu(x, wg, wu, split=split)
        assert (got.float() - ref).abs().max().item() < 2e-2 * max(1.0, ref.abs().max().item()), split
        got = DG.decode_linear(x, wg, split=split)
        assert (got.float() - ref_g).abs().max().item() < 2e-2 * max(1.0, ref_g.abs().max().item()), split
    from tyr_b200.ops._common import raise_on_device_error
    torch.cuda.synchronize()
    raise_on_device_error(x.device)


@pytest.mark.parametrize("M,N,K", [(17, 512, 1024), (32, 2176, 5120), (25, 100, 96)])
def test_skinny_swiglu_up_to_32_rows_and_strided_out(M, N, K):
    from tyr_b200.ops import skinny
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    wg = (torch.randn(N, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    wu = (torch.randn(N, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    assert skinny.swiglu_supported(x, wg, wu) and not skinny.supported(x, wg)       # plain products stop at 16 rows
    ref = torch.nn.functional.silu(x.float() @ wg.float().T) * (x.float() @ wu.float().T)
    got = skinny.skinny_swiglu(x, wg, wu)
    assert (got.float() - ref).abs().max().item() < 2e-2 * max(1.0, ref.abs().max().item())
    # the plain kernel itself handles 32 rows (used through out= by callers that choose it) and strided outputs
    buf = torch.zeros(M, N + 16, dtype=torch.bfloat16, device="cuda")
    skinny.skinny_linear(x, wg, out=buf[:, 8:8 + N])
    ref2 = x.float() @ wg.float().T
    assert (buf[:, 8:8 + N].float() - ref2).abs().max().item() < 2e-2 * max(1.0, ref2.abs().max().item())
    assert torch.equal(buf[:, :8], torch.zeros_like(buf[:, :8])) and torch.equal(buf[:, 8 + N:], torch.zeros_like(buf[:, 8 + N:]))


@pytest.mark.parametrize("M,N,K", [(1, 3072, 9216), (3, 100, 64), (8, 4096, 1024), (9, 1000, 2048), (16, 272, 3072)])
def test_skinny_gemm_matches_reference(M, N, K):
    from tyr_b200.ops.skinny import skinny_linear, supported
    g = torch.Generator().manual_seed(M * 7 + N)
    wide = (torch.randn(N, K + 64, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    w = wide[:, 32:32 + K]                                   # strided rows, 16-byte aligned start
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(N, generator=g).to(torch.bfloat16).cuda()
    assert supported(x, w)
    for bias in (None, b):
        y = skinny_linear(x, w, bias).float()
        ref = x.float() @ w.float().T + (0 if bias is None else bias.float())
        assert (y - ref).abs().max() < 2e-2 * max(1.0, ref.abs().max().item())


def test_flag_wait_runs_out_and_reports_without_losing_the_context():
    """A wait on a flag that nothing sets ends after its cycle budget (about 0.1 s here), records the timeout in the
    device error record, and leaves the device usable."""
    from tyr_b200.distributed.symm import wait_flags_bounded
    from tyr_b200.ops._common import err_word, ptr, raise_on_device_error
    dev = torch.device("cuda", 0)
    flags = torch.zeros(8, dtype=torch.int64, device=dev)
    flags[0] = 5                                            # rank 0 signalled, rank 1 never does
    err = err_word(dev)
    err.zero_()
    wait_flags_bounded(flags, 2, 0, 5, ptr(err), 200_000_000)
    with pytest.raises(RuntimeError, match="code=2 .*detail=1"):
        raise_on_device_error(dev)
    assert err.tolist()[0] == 0                             # the record was cleared by the read
    flags[1] = 5
    wait_flags_bounded(flags, 2, 0, 5, ptr(err), 200_000_000)
    raise_on_device_error(dev)                              # satisfied wait: no error
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0


def test_checked_build_records_a_bad_index_and_skips_it():
    """The -DTYR_BOUNDS_CHECK library: a rotary position outside the table and a pair index outside the batch are
    recorded (tag, index, limit) without faulting; clean inputs leave the record empty."""
    import ctypes
    from tyr_b200._native.checked import bounds_status, checked
    lib = checked()
    dev = torch.device("cuda", 0)
    st = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    x = torch.randn(4, 2, 32, device=dev).bfloat16()
    y = torch.empty_like(x)
    cos, sin = torch.ones(16, 8, device=dev), torch.zeros(16, 8, device=dev)
    assert bounds_status("rope")[0] == 0
    pos = torch.tensor([0, 3, 15, 7], dtype=torch.int32, device=dev)
    assert lib.tyr_rope_norm(p(x), p(y), None, p(cos), p(sin), p(pos), 64, 64, 4, 16, 2, 32, 16, 1e-6, 0, st) == 0
    torch.cuda.synchronize()
    assert bounds_status("rope") == (0, 0, 0, 0) and torch.equal(x, y)              # cos 1 / sin 0: identity rotation
    pos[2] = 99
    assert lib.tyr_rope_norm(p(x), p(y), None, p(cos), p(sin), p(pos), 64, 64, 4, 16, 2, 32, 16, 1e-6, 0, st) == 0
    torch.cuda.synchronize()
    assert bounds_status("rope") == (3, 21, 99, 16) and bounds_status("rope")[0] == 0   # read clears
    src = torch.randn(3, 16, device=dev).bfloat16()
    dst = torch.zeros(6, 16, device=dev).bfloat16()
    order = torch.tensor([0, 1, 2, 77, 4, 5], dtype=torch.int32, device=dev)
    assert lib.tyr_moe_gather_rows(p(src), p(order), p(dst), 6, 2, 16, st) == 0
    torch.cuda.synchronize()
    assert bounds_status("moe") == (3, 12, 77, 6)
    assert torch.equal(dst[0], src[0]) and torch.equal(dst[4], src[2]) and bool((dst[3] == 0).all())     # the bad row was skipped


@pytest.mark.parametrize("T,E,k,h,softmax", [(1, 256, 10, 3072, False), (64, 256, 10, 3072, False), (7, 64, 8, 2048, True), (33, 512, 4, 1024, False)])
def test_moe_route_fused_matches_separate_gemm_and_route(T, E, k, h, softmax):
    """Router GEMV + routing in one launch against fp32 logits from a library GEMM fed to the plain routing kernel."""
    from tyr_b200.ops import moe
    g = torch.Generator(device="cuda").manual_seed(T + E)
    x = torch.randn(T, h, device=_dev(), generator=g).bfloat16()
    wr = torch.randn(E, h, device=_dev(), generator=g) * h ** -0.5
    bias = torch.randn(E, device=_dev(), generator=g) * 0.01
    assert moe.route_fused_supported(x, wr)
    ids, w, counts = moe.route_fused(x, wr, k, softmax=softmax, bias=bias, renorm=True, softcap=0.0, scale=2.5)
    logits = x.double() @ wr.double().t()
    rid, rw, rc = moe.route(logits.float(), k, softmax=softmax, bias=bias, renorm=True, softcap=0.0, scale=2.5)
    same = (ids.sort(1).values == rid.sort(1).values).all(1)
    assert float(same.float().mean()) >= 0.95                      # a near-tie at the k-th place may resolve differently
    rows = same.nonzero().flatten()
    assert torch.allclose(w[rows].sort(1).values, rw[rows].sort(1).values, rtol=2e-3, atol=1e-5)
    assert int(counts.sum()) == T * k and torch.equal(counts, torch.bincount(ids.flatten().long(), minlength=E).int())


@pytest.mark.parametrize("B,S,Hk,Hv,dv,with_state", [(2, 256, 2, 4, 128, False), (1, 200, 1, 2, 64, True), (1, 64, 2, 2, 128, True), (4, 128, 16, 48, 128, False)])
def test_gated_delta_rule_chunk_scan_kernel_matches_recurrence(B, S, Hk, Hv, dv, with_state):
    """Chunked prefill with the chunk recurrence in one launch (TF32 tensor cores) against the token-by-token fp32 recurrence."""
    from tyr_b200.ops import delta_rule as DR
    g = torch.Generator(device="cuda").manual_seed(S + dv)
    dk = 128
    rn = lambda *s: torch.randn(*s, device=_dev(), generator=g)
    q, k = rn(B, S, Hk, dk).bfloat16(), rn(B, S, Hk, dk).bfloat16()
    rep = Hv // Hk
    qr, kr = q.repeat_interleave(rep, dim=2), k.repeat_interleave(rep, dim=2)
    v = rn(B, S, Hv, dv).bfloat16()
    gl = -torch.nn.functional.softplus(rn(B, S, Hv)) * 0.3
    beta = torch.sigmoid(rn(B, S, Hv))
    st0 = rn(B, Hv, dk, dv) * 0.1 if with_state else None
    assert DR.chunk_kernels_supported(q, k, v)
    out, st = DR.chunk_gated_delta_rule(q, k, v, gl, beta, 64, st0)                 # grouped keys: both chunk kernels
    ref, rst = DR.recurrent_gated_delta_rule(qr, kr, v, gl, beta, st0)
    torch.cuda.synchronize()
    assert out.shape == ref.shape and _rel_err(out, ref) < 2e-2, _rel_err(out, ref)
    assert _rel_err(st, rst) < 2e-2, _rel_err(st, rst)
    import os
    os.environ["TYR_GDR_CHUNK_KERNEL"] = "0"
    try:
        DR._CHUNK_KERNEL = False
        lib_out, lib_st = DR.chunk_gated_delta_rule(q, k, v, gl, beta, 64, st0)     # library-op form of the same algorithm
    finally:
        DR._CHUNK_KERNEL = True
        os.environ.pop("TYR_GDR_CHUNK_KERNEL", None)
    assert _rel_err(out, lib_out) < 2e-2 and _rel_err(st, lib_st) < 2e-2


@pytest.mark.parametrize("B,S,C,K,bias", [(2, 300, 256, 4, True), (1, 5, 64, 4, False), (3, 64, 10240, 4, True), (1, 2, 8, 2, True)])
def test_causal_conv1d_silu_matches_library(B, S, C, K, bias):
    from tyr_b200.ops import delta_rule as DR
    g = torch.Generator(device="cuda").manual_seed(C + S)
    wide = torch.randn(B, S, C + 16, device=_dev(), generator=g).bfloat16()
    x = wide[:, :, 8:8 + C]                                  # strided rows, 16-byte aligned
    w = torch.randn(C, K, device=_dev(), generator=g) * 0.5
    b = torch.randn(C, device=_dev(), generator=g) if bias else None
    y = DR.causal_conv1d_silu(x, w, b)
    xc = x.float().transpose(1, 2)
    ref = torch.nn.functional.silu(torch.nn.functional.conv1d(torch.nn.functional.pad(xc, (K - 1, 0)), w.reshape(C, 1, K), b, groups=C)).transpose(1, 2)
    assert y.shape == (B, S, C) and (y.float() - ref).abs().max() < 1e-2 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("act", ["swiglu", "geglu"])
def test_moe_dense_grouped_gemm_gate_epilogues(act):
    """Dense expert banks through the grouped tcgen05 GEMM with the SiLU / tanh-GELU gate in the epilogue against the fp32 expert loop."""
    from tyr_b200.ops import moe
    g = torch.Generator(device="cuda").manual_seed(3)
    T, E, k, h, mi = 200, 8, 2, 256, 384
    x = torch.randn(T, h, device=_dev(), generator=g).bfloat16()
    gate_up = (torch.randn(E, 2 * mi, h, device=_dev(), generator=g) * h ** -0.5).bfloat16()
    down = (torch.randn(E, h, mi, device=_dev(), generator=g) * mi ** -0.5).bfloat16()
    ids, w, cnt = moe.route(torch.randn(T, E, device=_dev(), generator=g), k)
    y = moe.moe_dense_forward(x, ids, w, gate_up, down, counts=cnt, act=act)
    ref = moe.moe_eager(x, ids.cpu().to(_dev()), w, gate_up[:, :mi], gate_up[:, mi:], down, act=act)
    assert _rel_err(y, ref) < 3e-2, _rel_err(y, ref)


@pytest.mark.parametrize("M,N,K", [(1, 1024, 512), (8, 17408, 5120), (13, 272, 2048), (2, 128, 64), (2, 64, 64), (16, 48, 32)])
def test_skinny_swiglu_matches_reference(M, N, K):
    from tyr_b200.ops.skinny import skinny_swiglu, swiglu_supported
    g = torch.Generator(device="cuda").manual_seed(M + N)
    x = torch.randn(M, K, device=_dev(), generator=g).bfloat16()
    wg = (torch.randn(N, K, device=_dev(), generator=g) * K ** -0.5).bfloat16()
    wu = (torch.randn(N, K, device=_dev(), generator=g) * K ** -0.5).bfloat16()
    assert swiglu_supported(x, wg, wu)
    y = skinny_swiglu(x, wg, wu).float()
    ref = torch.nn.functional.silu(x.float() @ wg.float().T) * (x.float() @ wu.float().T)
    assert (y - ref).abs().max() < 2e-2 * max(1.0, ref.abs().max().item())
