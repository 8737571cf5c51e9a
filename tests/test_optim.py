"""Optimizer stack (Tests/TestManifoldMuon.lean:64-227, TestDualOptimizerDispatch.lean:17-215,
schedule / NorMuon / DistAdam local-fallback tests)."""
import math

import pytest
import torch

from tyr_b200 import manifolds as mf
from tyr_b200 import modular as md
from tyr_b200 import optim
from tyr_b200.optim import distadam, dual, manifold_muon, normuon, polar_express, riemannian, schedule
from tyr_b200.struct import tensor_struct


@tensor_struct
class P:
    w: torch.Tensor
    b: torch.Tensor


def test_adamw_chain_matches_torch():
    torch.manual_seed(0)
    p = P(torch.randn(4, 3), torch.randn(3))
    ref = [p.w.clone().requires_grad_(True), p.b.clone().requires_grad_(True)]
    topt = torch.optim.AdamW(ref, lr=0.01, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
    opt = optim.adamw(lr=0.01, weight_decay=0.0)
    state = opt.init(p)
    for i in range(3):
        g = P(torch.randn(4, 3), torch.randn(3))
        ref[0].grad, ref[1].grad = g.w.clone(), g.b.clone()
        topt.step()
        p, state = optim.step(opt, p, g, state)
    assert torch.allclose(p.w, ref[0], atol=1e-6) and torch.allclose(p.b, ref[1], atol=1e-6)
    assert p.w.requires_grad and state.fst.count == 3


def test_weight_decay_sgd_and_schedule_chain():
    p = P(torch.ones(2, 2), torch.ones(2))
    g = P(torch.zeros(2, 2), torch.zeros(2))
    opt = optim.chain(optim.add_decayed_weights(0.5), optim.scale(-0.1))
    q, _ = optim.step(opt, p, g, opt.init(p))
    assert torch.allclose(q.w, torch.full((2, 2), 0.95))
    opt = optim.sgd_schedule(schedule.linear_decay(1.0, 2))
    s = opt.init(p)
    p1, s = optim.step(opt, p, P(torch.ones(2, 2), torch.ones(2)), s)
    p2, s = optim.step(opt, p1, P(torch.ones(2, 2), torch.ones(2)), s)
    assert torch.allclose(p1.w, torch.zeros(2, 2)) and torch.allclose(p2.w, torch.full((2, 2), -0.5))


def test_schedules():
    c = schedule.cosine_decay(1.0, 100, 0.1, warmup_steps=10)
    assert c(0) == 0.0 and abs(c(10) - 1.0) < 1e-12 and abs(c(55) - 0.55) < 1e-9 and c(100) == 0.1
    assert schedule.step_decay(1.0, 0.1, 30)(65) == pytest.approx(0.01)
    oc = schedule.one_cycle(1.0, 100, 0.0, 0.3)
    assert oc(30) == pytest.approx(1.0) and oc(100) == 0.0 and oc(15) == pytest.approx(0.5)
    w = schedule.warmup_plateau_cosine(2.0, 100, 10, 20)
    assert w(5) == 1.0 and w(25) == 2.0 and w(100) == 0.0
    assert schedule.sequence(schedule.constant(1.0), 5, schedule.constant(2.0))(7) == 2.0
    assert schedule.clamp(schedule.exponential_decay(1.0, 0.5), 0.2, 0.9)(0) == 0.9
    assert schedule.polynomial_decay(1.0, 10, 0.0, 2.0)(5) == pytest.approx(0.25)
    assert schedule.linear_weight_decay(1.2, 10)(5) == pytest.approx(0.6)


def test_muon_orthogonalize_and_polar_express():
    torch.manual_seed(1)
    g = torch.randn(32, 64)
    o = polar_express.muon_orthogonalize(g, 5).float()
    assert o.dtype == torch.float32 and polar_express.muon_orthogonalize(g).dtype == torch.bfloat16
    sv = torch.linalg.svdvals(o)
    assert sv.max() < 1.35 and sv.min() > 0.3
    tall = polar_express.muon_orthogonalize(g.T.contiguous(), 5).float()
    assert torch.allclose(tall, o.T, atol=5e-2)
    pe = polar_express.apply(g, polar_express.Config(5))
    sv = torch.linalg.svdvals(pe)
    assert sv.max() < 1.2 and sv.min() > 0.6
    assert len(polar_express.apply_batch([g, g])) == 2


def test_normuon_step_single():
    torch.manual_seed(2)
    p = torch.randn(16, 8)
    g = torch.randn(16, 8)
    cfg = normuon.Config(lr=0.1, weight_decay=0.5, momentum=0.9)
    q, st = normuon.step_single(p, g, normuon.init_param_state(), cfg)
    mom = 0.1 * g
    nes = 0.1 * g + 0.9 * mom
    eff = 0.1 * math.sqrt(2.0)
    expect = p - p * (eff * 0.5) - (polar_express.muon_orthogonalize(nes).float() * eff)
    assert torch.allclose(q, expect, atol=2e-2) and torch.allclose(st.momentum_buffer, mom) and st.step == 1
    z, _ = normuon.step_single(p, torch.zeros_like(p), normuon.init_param_state(), normuon.Config(weight_decay=0.0))
    assert torch.equal(z.detach(), p)      # zero gradients stay zero
    ps, ss = normuon.step_distributed_group([p, p], [g, g], [normuon.init_param_state()] * 2, cfg)
    assert torch.allclose(ps[0], q)        # no process group -> local fallback
    assert normuon.get_momentum(0) == 0.85 and normuon.get_momentum(400) == 0.95


def test_distadam_local_and_sharded_fallback():
    torch.manual_seed(3)
    p = torch.randn(6, 4)
    g = torch.randn(6, 4)
    cfg = distadam.Config(lr=0.01, beta1=0.8, beta2=0.95, eps=1e-10, weight_decay=0.1)
    q, st = distadam.step_distributed(p, g, distadam.init_param_state(p), cfg)
    m = 0.2 * g
    v = 0.05 * g * g
    expect = p - p * 0.001 - 0.01 * (m / 0.2) / ((v / 0.05).sqrt() + 1e-10)
    assert torch.allclose(q, expect, atol=1e-6) and st.step == 1
    emb = distadam.ShardedEmbeddingAdam(p, cfg)
    emb.step(g)
    assert torch.allclose(emb.gather(), expect, atol=1e-6)


def test_manifold_muon_keeps_stiefel_constraint():
    torch.manual_seed(4)
    W = manifold_muon.retract_stiefel(torch.randn(12, 4))
    st = manifold_muon.init_param_state()
    for solver in (manifold_muon.SolverKind.dual_ascent, manifold_muon.SolverKind.fixed_point):
        cfg = manifold_muon.Config(lr=0.05, solver=solver, dual_ascent_steps=3)
        W2, st2, diag = manifold_muon.step_single_with_diagnostics(W, torch.randn(12, 4), st, cfg)
        assert mf.Stiefel().check(W2.detach(), 1e-4) and diag.iterations >= 1 and st2.dual_var.shape == (4, 4)
        assert (W2.detach() - W).norm() > 1e-3
    wide = manifold_muon.retract_stiefel(torch.randn(4, 12))
    W3, _ = manifold_muon.step_single(wide, torch.randn(4, 12), manifold_muon.init_param_state(),
                                      manifold_muon.Config(dual_ascent_steps=0))
    assert mf.Stiefel().check(W3.detach(), 1e-4)
    t = manifold_muon.tangent_project(W, torch.randn(12, 4))
    assert manifold_muon.tangent_residual(W, t).abs().max() < 1e-5
    assert manifold_muon.benchmark_local_step(16, 8, iters=1) > 0


def test_dual_optimizer_dispatch():
    torch.manual_seed(5)
    cfg = dual.Config(model_dim=1536)
    assert dual.dim_lr_scale(cfg) == pytest.approx(2 ** -0.5)
    assert dual.label_to_group(normuon.ParamLabel.mlp) is dual.ParamGroup.matrix
    assert dual.label_to_group(normuon.ParamLabel.value_embed) is dual.ParamGroup.embedding
    w = torch.randn(8, 8)
    st = dual.init_matrix_state(cfg)
    p, st = dual.step_matrix_single(w, torch.randn(8, 8), st, cfg)
    assert st.step == 1
    mcfg = dual.Config(matrix_optimizer=dual.MatrixOptimizerKind.manifold_muon,
                       manifold_family=dual.MatrixManifoldFamily.orthogonal)
    with pytest.raises(RuntimeError, match="produced by"):
        dual.step_matrix_single(w, w, st, mcfg)                      # state/optimizer mismatch
    q = mf.Orthogonal().project(w)
    ost = dual.init_matrix_state(mcfg)
    q2, ost = dual.step_matrix_single(q, torch.randn(8, 8), ost, mcfg)
    assert mf.Orthogonal().check(q2.detach(), 1e-4)
    gcfg = dual.Config(matrix_optimizer=dual.MatrixOptimizerKind.manifold_muon,
                       manifold_family=dual.MatrixManifoldFamily.grassmann)
    y = mf.Grassmann().project(torch.randn(8, 3))
    y2, _ = dual.step_matrix_single(y, torch.randn(8, 3), dual.init_matrix_state(gcfg), gcfg)
    assert mf.Grassmann().check(y2.detach(), 1e-4)
    opt = dual.DualOptimizer({"w": (w, normuon.ParamLabel.attn), "e": (torch.randn(5, 4), normuon.ParamLabel.embed)}, cfg)
    out = opt.step({"w": w, "e": torch.randn(5, 4)}, {"w": torch.randn(8, 8), "e": torch.randn(5, 4)})
    assert set(out) == {"w", "e"}


def test_manifolds_constraints_preserved():
    torch.manual_seed(6)
    for man, x in ((mf.Sphere(), mf.Sphere().project(torch.randn(7))),
                   (mf.Oblique(), mf.Oblique().project(torch.randn(5, 3))),
                   (mf.Elliptope(), mf.Elliptope().project(torch.randn(6, 2))),
                   (mf.FixedRankEmbedded(2), mf.FixedRankEmbedded(2).project(torch.randn(6, 5)))):
        y = mf.gradient_step(man, x, torch.randn_like(x), 0.1)
        assert man.check(y, 1e-3), man.name
    pos = mf.Positive()
    assert pos.check(mf.gradient_step(pos, torch.rand(5) + 0.1, torch.randn(5), 0.1))
    spd = mf.SymmetricPositiveDefinite()
    A = torch.randn(4, 4)
    X = A @ A.T + torch.eye(4)
    assert torch.allclose(spd.expm(spd.logm(X)), X, atol=1e-4)
    with pytest.raises(ValueError):
        spd.logm(-X)
    s = mf.Sphere()
    a, b = s.project(torch.randn(4)), s.project(torch.randn(4))
    v = s.tangent_project(a, b - a)
    v = v / v.norm() * s.distance(a, b)
    assert torch.allclose(s.exp(a, v), b, atol=1e-4)
    sd = mf.SignDualMap()
    assert torch.equal(sd.dual_map_step(torch.zeros(3), torch.tensor([2.0, -3.0, 0.0]), 0.5), torch.tensor([-0.5, 0.5, 0.0]))


def test_modular_norms_and_budget():
    torch.manual_seed(7)
    l1, l2 = md.Linear.init(16, 8), md.Linear.init(8, 4)
    assert l1.norm() == pytest.approx(1.0, abs=1e-4) and l1.is_well_normed()
    seq = md.compose(l1, l2)
    assert seq.nu() == pytest.approx(1.0, abs=1e-3)
    g = torch.randn(8, 16)
    d = l1.normalize_dual(g)
    assert md.Linear(d).norm() == pytest.approx(1.0, abs=1e-4)
    assert (d * g).sum() == pytest.approx(l1.dual_norm(g), rel=1e-4)      # saturates the dual pairing
    upd = l1.normalized_update(0.1, g)
    assert md.Linear(upd).norm() == pytest.approx(0.1, abs=1e-4)
    e = md.Embedding.init(10, 6)
    assert e.norm() == pytest.approx(1.0, abs=1e-5)
    lrs = md.budgeted_sequential_lrs(1.0, [md.Linear(l1.weight * 2), l2])
    assert lrs[1] == 1.0 and lrs[0] == pytest.approx(1.0)
    assert md.multiplier_from_sensitivity(md.BudgetConfig(), 4.0) == 0.25
    K = md.MetricFactor(torch.randn(3, 6))
    D = md.DiagonalMass.of_scalar(6, 0.5)
    b = torch.randn(6)
    assert torch.allclose(K.solve_woodbury(D, b), torch.linalg.solve(K.dense_metric(D), b), atol=1e-4)
    ml = md.StiefelLinear(8, 4)
    assert ml.apply_dual_map_update(torch.randn(4, 8), 0.1).on_manifold(1e-3)
    hv = md.HyperbolicVector.init(3)
    assert mf.Hyperbolic().check(hv.apply_dual_map_update(torch.randn(4), 0.1).value, 1e-3)


def test_riemannian_sgd_and_tree_sgd():
    torch.manual_seed(8)
    layer = md.RiemannianLinear(torch.randn(3, 4) * 0.3, mass=0.5)
    x, t = torch.randn(4), torch.randn(3)
    losses = []
    for _ in range(5):
        r = riemannian.step_mse(layer, x, t, 0.5)
        layer = r.params
        losses.append(r.loss)
    assert losses[-1] < 0.2 * losses[0]
    layers = [md.RiemannianLinear(torch.randn(5, 4) * 0.3), md.RiemannianLinear(torch.randn(3, 5) * 0.3)]
    l0 = riemannian.step_sequential_mse(layers, x, t, 0.0).loss
    for _ in range(8):
        layers = riemannian.step_sequential_mse(layers, x, t, 0.3).params
    assert riemannian.step_sequential_mse(layers, x, t, 0.0).loss < l0
    params = P(torch.randn(3, 5) * 0.1, torch.zeros(5))
    xs, ys = torch.randn(4, 3), torch.tensor([0, 2, 1, 4])
    fn = lambda p: xs @ p.w + p.b
    prev = None
    for _ in range(4):
        params, loss, diag = riemannian.step_cross_entropy(fn, params, ys, lr=0.5, mass=1e-2, max_step_norm=5.0)
        assert prev is None or loss < prev + 1e-6
        prev = loss
    g = torch.Generator().manual_seed(0)
    _, loss2, _ = riemannian.step_cross_entropy_sampled_fisher(fn, params, ys, lr=0.1, samples=3, generator=g)
    assert math.isfinite(loss2)
    f = riemannian.TreeMetricFactor([P(torch.randn(3, 5), torch.randn(5)) for _ in range(2)])
    b = P(torch.randn(3, 5), torch.randn(5))
    sol = f.solve_woodbury(0.7, b)
    back = f.apply_regularized(0.7, sol)
    assert torch.allclose(back.w, b.w, atol=1e-4) and torch.allclose(back.b, b.b, atol=1e-4)
