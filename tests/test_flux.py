"""Flux DiT: rope / modulation algebra, block shapes, schedule, pack/unpack, loader, VAE decoder."""
import math

import pytest
import torch

from tyr_b200.io import safetensors as st
from tyr_b200.models import flux as FX
from tyr_b200.models import vae as V
from tyr_b200.ops.modulate import gate_residual, layernorm_modulate


def tiny():
    return FX.FluxConfig(hidden_size=64, num_heads=2, half_head_dim=16, num_double_layers=2, num_single_layers=2,
                         context_in_dim=48, in_channels=16, time_dim=32, mlp_hidden_dim=96, half_axes_dims=(4, 4, 4, 4))


def test_config_validation_and_defaults():
    c = FX.FluxConfig.klein4b()
    assert c.head_dim == 128 and c.mlp_hidden_dim == 3 * c.hidden_size
    with pytest.raises(ValueError, match="sum to half_head_dim"):
        FX.FluxConfig(half_axes_dims=(16, 16, 16, 8))


def test_rope_is_a_rotation_per_axis():
    ids = FX.compute_image_position_ids(3, 5)
    assert ids.shape == (1, 15, 4) and ids[0, 7].tolist() == [0, 1, 2, 0]
    assert FX.compute_text_position_ids(4)[0, 3].tolist() == [0, 0, 0, 3]
    cos, sin = FX.rope_embed(ids, (4, 4, 4, 4), 2000)
    assert cos.shape == (1, 15, 16)
    assert torch.allclose(cos[0, :, :4], torch.ones(15, 4))            # axis 0 id is always 0
    w = 2000.0 ** (-2.0 / 8)
    assert abs(cos[0, 7, 5].item() - math.cos(1 * w)) < 1e-6           # axis 1 (row), j = 1
    x = torch.randn(1, 15, 2, 32)
    y = FX.apply_rope(x, (cos, sin))
    assert torch.allclose(y.pow(2).sum(-1), x.pow(2).sum(-1), atol=1e-4)
    assert torch.allclose(y[0, 7, 0, 10], cos[0, 7, 5] * x[0, 7, 0, 10] - sin[0, 7, 5] * x[0, 7, 0, 11], atol=1e-6)


def test_timestep_embedding_and_schedule():
    e = FX.timestep_embedding(torch.tensor([0.5]), 8)
    assert e.shape == (1, 8) and abs(e[0, 0].item() - math.cos(500.0)) < 1e-4
    ts = FX.compute_timesteps(256, 4)
    assert len(ts) == 4 and ts[0][0] == 1.0 and ts[-1][1] == 0.0
    assert all(a > b for a, b in ts) and all(ts[i][1] == ts[i + 1][0] for i in range(3))
    mu = FX.compute_empirical_mu(256, 4)
    assert abs(ts[1][0] - math.exp(mu) / (math.exp(mu) + (1 / 0.75 - 1))) < 1e-12
    assert abs(FX.compute_empirical_mu(5000, 4) - (0.00016927 * 5000 + 0.45666666)) < 1e-12


def test_pack_unpack_roundtrip():
    z = torch.randn(2, 12, 128)
    u = FX.unpack_latents(z, 3, 4)
    assert u.shape == (2, 32, 6, 8) and torch.equal(FX.pack_latents(u), z)
    assert u[0, 5, 3, 2] == z[0, 1 * 4 + 1, 5 * 4 + 1 * 2 + 0]


def test_modulation_helpers_match_formula():
    x, sc, sh, g = torch.randn(2, 5, 16), torch.randn(2, 16), torch.randn(2, 16), torch.randn(2, 16)
    y = layernorm_modulate(x, sc, sh)
    ref = (1 + sc[:, None]) * torch.nn.functional.layer_norm(x, (16,), eps=1e-6) + sh[:, None]
    assert torch.allclose(y, ref, atol=1e-5)
    assert torch.allclose(gate_residual(x, y, g), x + g[:, None] * y, atol=1e-6)


def test_forward_denoise_and_zero_gates():
    cfg = tiny()
    m = FX.init(cfg)
    img, txt = torch.randn(2, 12, 16), torch.randn(2, 5, 48)
    iid, tid = FX.compute_image_position_ids(3, 4).expand(2, -1, -1), FX.compute_text_position_ids(5).expand(2, -1, -1)
    out = FX.forward(m, img, txt, torch.tensor([1.0, 0.3]), iid, tid)
    assert out.shape == (2, 12, 16) and torch.isfinite(out).all()
    # batch rows are independent
    out0 = FX.forward(m, img[:1], txt[:1], torch.tensor([1.0]), iid[:1], tid[:1])
    assert torch.allclose(out[:1], out0, atol=1e-4)
    # zero modulation weights => gates are zero => blocks are identities => output depends only on the final layer
    m.double_stream_modulation_img.zero_(); m.double_stream_modulation_txt.zero_(); m.single_stream_modulation.zero_()
    h = torch.nn.functional.linear(img, m.img_in)
    vec = torch.nn.functional.linear(torch.nn.functional.silu(torch.nn.functional.linear(FX.timestep_embedding(torch.tensor([1.0, 0.3]), 32), m.time_in_layer)), m.time_out_layer)
    mod2 = torch.nn.functional.linear(torch.nn.functional.silu(vec), m.final_modulation)
    ref = torch.nn.functional.linear((1 + mod2[:, None, 64:]) * torch.nn.functional.layer_norm(h, (64,), eps=1e-6) + mod2[:, None, :64], m.final_linear)
    assert torch.allclose(FX.forward(m, img, txt, torch.tensor([1.0, 0.3]), iid, tid), ref, atol=1e-4)
    x = FX.denoise(FX.init(cfg), img, txt, iid, tid, num_steps=2)
    assert x.shape == img.shape and torch.isfinite(x).all()


def test_loader_roundtrip(tmp_path):
    cfg = tiny()
    m = FX.init(cfg)
    p = str(tmp_path / "flux.safetensors")
    st.save_file({k: v.contiguous() for k, v in FX.state_dict(m).items()}, p)
    m2 = FX.load(cfg, p, dtype=torch.float32)
    img, txt = torch.randn(1, 4, 16), torch.randn(1, 3, 48)
    iid, tid = FX.compute_image_position_ids(2, 2), FX.compute_text_position_ids(3)
    t = torch.tensor([0.7])
    assert torch.equal(FX.forward(m, img, txt, t, iid, tid), FX.forward(m2, img, txt, t, iid, tid))


def test_vae_decoder_shapes_and_latent_denormalisation():
    dec = V.init_decoder(stages=((64, 64, True), (64, 32, False)), z_channels=8)
    ae = V.AutoEncoder(dec, torch.arange(32.0), torch.full((32,), 3.0))
    z = torch.randn(1, 32, 4, 4)
    zn = ae.inv_normalize(z)
    assert torch.allclose(zn[0, 5], z[0, 5] * math.sqrt(3.0 + 1e-4) + 5.0, atol=1e-5)
    u = V.AutoEncoder.unpack_packed(z)
    assert u.shape == (1, 8, 8, 8) and u[0, 2, 3, 5] == z[0, 2 * 4 + 1 * 2 + 1, 1, 2]
    img = ae.decode(z)
    assert img.shape == (1, 3, 16, 16) and torch.isfinite(img).all()
    full = V.init_decoder()
    assert sum(len(s) for s in full.ups) == 15 and full.conv_in.weight.shape == (512, 32, 3, 3)


@pytest.mark.gpu
def test_gpu_modulate_kernels_match_reference():
    x = torch.randn(3, 70, 3072, device="cuda").bfloat16()
    mod = torch.randn(3, 6, 3072, device="cuda").bfloat16()
    y = layernorm_modulate(x, mod[:, 1], mod[:, 0])
    ref = (1 + mod[:, 1].float()[:, None]) * torch.nn.functional.layer_norm(x.float(), (3072,), eps=1e-6) + mod[:, 0].float()[:, None]
    assert torch.allclose(y.float(), ref, atol=3e-2, rtol=2e-2)
    o = gate_residual(x, y, mod[:, 2])
    assert torch.allclose(o.float(), x.float() + mod[:, 2].float()[:, None] * y.float(), atol=3e-2, rtol=2e-2)


@pytest.mark.gpu
def test_gpu_flux_qk_post_matches_unfused_ops():
    """QK-norm + RoPE kernel against the fp32 formula, into a joint buffer at a row offset (with the v copy) and in place."""
    from tyr_b200.ops.modulate import flux_qk_post
    B, S, H, D, extra = 2, 200, 3, 128, 256
    g = torch.Generator(device="cuda").manual_seed(3)
    src = torch.randn(B, S, 3 * H * D + extra, device="cuda", generator=g).bfloat16()
    wq = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).bfloat16()
    wk = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).bfloat16()
    ids = torch.randint(0, 50, (B, S, 4), device="cuda", generator=g)
    cos, sin = FX.rope_embed(ids, (16, 16, 16, 16), 2000)

    def ref(x, w):
        xf = x.float().reshape(B, S, H, D)
        n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
        return FX.apply_rope(n, (cos, sin)).reshape(B, S, H * D)
    rq, rk = ref(src[..., :H * D], wq), ref(src[..., H * D:2 * H * D], wk)
    dst = torch.zeros(B, S + 40, 3 * H * D, device="cuda", dtype=torch.bfloat16)
    flux_qk_post(src, dst, wq, wk, cos, sin, H, dst_row0=40, copy_v=True)
    assert torch.equal(dst[:, :40], torch.zeros_like(dst[:, :40]))
    assert (dst[:, 40:, :H * D].float() - rq).abs().max().item() < 2e-2 * rq.abs().max().item()
    assert (dst[:, 40:, H * D:2 * H * D].float() - rk).abs().max().item() < 2e-2 * rk.abs().max().item()
    assert torch.equal(dst[:, 40:, 2 * H * D:], src[..., 2 * H * D:3 * H * D])
    inplace = src.clone()
    flux_qk_post(inplace, inplace, wq, wk, cos, sin, H)
    assert torch.equal(inplace[..., :2 * H * D], dst[:, 40:, :2 * H * D]) and torch.equal(inplace[..., 2 * H * D:], src[..., 2 * H * D:])


@pytest.mark.gpu
def test_gpu_gated_gemm_matches_reference():
    """SwiGLU in the epilogue of a dense product, written into a column window of a wider buffer."""
    from tyr_b200.ops.gemm import gemm, interleave_gate_up
    g = torch.Generator(device="cuda").manual_seed(5)
    M, K, Mh = 1000, 512, 384
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w1 = (torch.randn(2 * Mh, K, device="cuda", generator=g) * K ** -0.5).bfloat16()
    gu = x.float() @ w1.float().T
    ref = torch.nn.functional.silu(gu[:, :Mh]) * gu[:, Mh:]
    buf = torch.zeros(M, 128 + Mh, device="cuda", dtype=torch.bfloat16)
    gemm(x, interleave_gate_up(w1), act="swiglu", out=buf[:, 128:])
    assert torch.equal(buf[:, :128], torch.zeros_like(buf[:, :128]))
    assert (buf[:, 128:].float() - ref).abs().max().item() < 2e-2 * ref.abs().max().item()
    cpu = gemm(x.cpu().float(), interleave_gate_up(w1).cpu().float(), act="swiglu")
    assert torch.allclose(cpu, ref.cpu(), atol=1e-3, rtol=1e-3)


@pytest.mark.gpu
def test_gpu_flux_bf16_matches_fp32_cpu():
    cfg = FX.FluxConfig(hidden_size=256, num_heads=2, half_head_dim=64, num_double_layers=1, num_single_layers=1, context_in_dim=64,
                        in_channels=32, time_dim=64, mlp_hidden_dim=512)
    m = FX.init(cfg)
    img, txt = torch.randn(1, 192, 32), torch.randn(1, 64, 64)
    iid, tid = FX.compute_image_position_ids(12, 16), FX.compute_text_position_ids(64)
    t = torch.tensor([0.6])
    ref = FX.forward(m, img, txt, t, iid, tid)
    mg = _to_cuda(m)
    with torch.no_grad():
        out = FX.forward(mg, img.cuda().bfloat16(), txt.cuda().bfloat16(), t.cuda(), iid.cuda(), tid.cuda()).float().cpu()
    assert (out - ref).abs().max().item() < 0.08 * ref.abs().max().item()


def _to_cuda(m):
    import dataclasses

    def conv(o):
        if isinstance(o, torch.Tensor):
            return o.to(device="cuda", dtype=torch.bfloat16)
        if dataclasses.is_dataclass(o) and not isinstance(o, FX.FluxConfig):
            return type(o)(**{f.name: conv(getattr(o, f.name)) for f in dataclasses.fields(o)})
        if isinstance(o, list):
            return [conv(v) for v in o]
        return o
    return conv(m)
