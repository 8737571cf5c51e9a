"""Kernel micro-benchmarks: `python -m benchmarks.kernel_bench [gemm|attention|attention-bwd|moe|moe-decode|decode-attn|skinny|elementwise|ns|gdr|qwen3-decode|all]`
(plus `*-small` cases sized for a profiler: gemm-fwd-small, attention-fwd-small, attention-bwd-small, elementwise-small,
ns-small, fp4-small, gdr-small, decode-attn-small).

Times the hand-written kernels with CUDA events (5 warm-up + 20 timed iterations, a 256 MB
buffer written between iterations to flush the 126 MB L2) on the NanoChat d20 shapes and prints
achieved TFLOP/s next to the library kernel for the same product (cuBLAS through torch.matmul,
SDPA) measured the same way.
"""
from __future__ import annotations

import json
import sys

import torch


def _time(fn, iters=20, warmup=5, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    evs = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        evs.append((e0, e1))
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) for a, b in evs)
    return ts[len(ts) // 2]


def bench_gemm(results):
    from tyr_b200.ops.gemm import gemm
    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    N = 65536
    shapes = [
        ("fwd qkv   [65536x1280]x[3840x1280]^T", "K", "K", (N, 1280), (3840, 1280), N, 3840, 1280),
        ("fwd fc    [65536x1280]x[5120x1280]^T", "K", "K", (N, 1280), (5120, 1280), N, 5120, 1280),
        ("fwd proj  [65536x5120]x[5120x1280]  ", "K", "MN", (N, 5120), (5120, 1280), N, 1280, 5120),
        ("dgrad fc  [65536x5120]x[5120x1280]  ", "K", "MN", (N, 5120), (5120, 1280), N, 1280, 5120),
        ("wgrad fc  [65536x5120]^Tx[65536x1280]", "MN", "MN", (N, 5120), (N, 1280), 5120, 1280, N),
        ("wgrad qkv [65536x3840]^Tx[65536x1280]", "MN", "MN", (N, 3840), (N, 1280), 3840, 1280, N),
        ("lm_head   [8192x1280]x[65536x1280]^T", "K", "K", (8192, 1280), (65536, 1280), 8192, 65536, 1280),
    ]
    for name, la, lb, sa, sb, M, Nn, K in shapes:
        a = torch.randn(sa, device=dev).bfloat16()
        b = torch.randn(sb, device=dev).bfloat16()
        flops = 2.0 * M * Nn * K
        if la == "MN":
            out32 = torch.zeros(M, Nn, device=dev, dtype=torch.float32)
            ours = _time(lambda: gemm(a, b, a_layout=la, b_layout=lb, out=out32, accumulate=True), flush=flush)
            lib = _time(lambda: torch.matmul(a.t(), b), flush=flush)
        else:
            ours = _time(lambda: gemm(a, b, a_layout=la, b_layout=lb), flush=flush)
            lib = _time(lambda: torch.matmul(a, b.t() if lb == "K" else b), flush=flush)
        results.append({"kernel": "gemm", "shape": name.strip(), "ours_ms": ours, "ours_tflops": flops / ours / 1e9,
                        "cublas_ms": lib, "cublas_tflops": flops / lib / 1e9})
        print(f"{name}  ours {ours:7.3f} ms {flops/ours/1e9:7.1f} TF/s | cuBLAS {lib:7.3f} ms {flops/lib/1e9:7.1f} TF/s", flush=True)
    # batched Newton-Schulz shapes
    for name, Bt, R, C in (("NS xxt 76x[1280x1280]", 76, 1280, 1280), ("NS xxt 40x[1280x5120]", 40, 1280, 5120)):
        x = torch.randn(Bt, R, C, device=dev).bfloat16()
        flops = 2.0 * Bt * R * R * C
        ours = _time(lambda: gemm(x, x), flush=flush)
        lib = _time(lambda: torch.bmm(x, x.transpose(1, 2)), flush=flush)
        results.append({"kernel": "gemm", "shape": name, "ours_ms": ours, "ours_tflops": flops / ours / 1e9,
                        "cublas_ms": lib, "cublas_tflops": flops / lib / 1e9})
        print(f"{name:38s}  ours {ours:7.3f} ms {flops/ours/1e9:7.1f} TF/s | cuBLAS {lib:7.3f} ms {flops/lib/1e9:7.1f} TF/s", flush=True)


def bench_attention(results):
    import torch.nn.functional as F
    from tyr_b200.ops import flash
    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for B, H, T, causal in ((32, 10, 2048, True), (4, 24, 4608, False), (8, 16, 4096, True)):
        D = 128
        qkv = torch.randn(B, T, 3, H, D, device=dev).bfloat16()
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        flops = 4.0 * B * H * T * T * D * (0.5 if causal else 1.0)
        ours = _time(lambda: flash.flash_fwd_bthd(q, k, v, causal=causal, window=None, scale=None), flush=flush)
        qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        lib = _time(lambda: F.scaled_dot_product_attention(qt, kt, vt, is_causal=causal), flush=flush)
        results.append({"kernel": "flash_fwd", "shape": f"B{B} H{H} T{T} D{D} causal={causal}", "ours_ms": ours,
                        "ours_tflops": flops / ours / 1e9, "sdpa_ms": lib, "sdpa_tflops": flops / lib / 1e9})
        print(f"flash fwd B{B} H{H} T{T} causal={causal}: ours {ours:7.3f} ms {flops/ours/1e9:7.1f} TF/s | SDPA {lib:7.3f} ms {flops/lib/1e9:7.1f} TF/s", flush=True)


def bench_attention_bwd(results):
    """Backward of causal / joint attention: the tcgen05 kernel (with its prepare and finish launches) against the
    library's backward, both through their public entry points."""
    import torch.nn.functional as F
    from tyr_b200.ops import flash
    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for B, H, T, causal in ((32, 10, 2048, True), (4, 24, 4608, False), (8, 16, 4096, True)):
        D = 128
        qkv = torch.randn(B, T, 3, H, D, device=dev).bfloat16()
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        do = torch.randn(B, T, H, D, device=dev).bfloat16()
        flops = 10.0 * B * H * T * T * D * (0.5 if causal else 1.0)
        o, lse = flash.flash_fwd_bthd(q, k, v, causal=causal, window=None, scale=None)
        ours = _time(lambda: flash.flash_bwd_bthd(do, q, k, v, o, lse, causal=causal, window=None, scale=None), flush=flush)
        qt, kt, vt = (t.transpose(1, 2).detach().requires_grad_() for t in (q, k, v))
        ol = F.scaled_dot_product_attention(qt, kt, vt, is_causal=causal)
        dot = do.transpose(1, 2)
        lib = _time(lambda: torch.autograd.grad(ol, (qt, kt, vt), dot, retain_graph=True), flush=flush)
        results.append({"kernel": "flash_bwd", "shape": f"B{B} H{H} T{T} D{D} causal={causal}", "ours_ms": ours,
                        "ours_tflops": flops / ours / 1e9, "sdpa_ms": lib, "sdpa_tflops": flops / lib / 1e9})
        print(f"flash bwd B{B} H{H} T{T} causal={causal}: ours {ours:7.3f} ms {flops/ours/1e9:7.1f} TF/s | SDPA {lib:7.3f} ms {flops/lib/1e9:7.1f} TF/s", flush=True)


def bench_attention_fwd_small(results):
    """One small forward case for profiler captures: B 8, H 10, T 2048 causal, two warm-up and three timed calls."""
    from tyr_b200.ops import flash
    dev = torch.device("cuda")
    B, H, T, D = 8, 10, 2048, 128
    qkv = torch.randn(B, T, 3, H, D, device=dev).bfloat16()
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    ms = _time(lambda: flash.flash_fwd_bthd(q, k, v, causal=True, window=None, scale=None), iters=3, warmup=2)
    flops = 2.0 * B * H * T * T * D
    results.append({"kernel": "flash_fwd_small", "ms": ms, "tflops": flops / ms / 1e9})
    print(f"flash fwd small B{B} H{H} T{T}: {ms:7.3f} ms {flops / ms / 1e9:7.1f} TF/s", flush=True)


def bench_attention_bwd_small(results):
    """One small backward case for profiler captures: B 8, H 10, T 2048 causal (q, k, v, o, dO and the gradients hold about
    0.3 GB), two warm-up and three timed calls."""
    from tyr_b200.ops import flash
    dev = torch.device("cuda")
    B, H, T, D = 8, 10, 2048, 128
    qkv = torch.randn(B, T, 3, H, D, device=dev).bfloat16()
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    do = torch.randn(B, T, H, D, device=dev).bfloat16()
    o, lse = flash.flash_fwd_bthd(q, k, v, causal=True, window=None, scale=None)
    ms = _time(lambda: flash.flash_bwd_bthd(do, q, k, v, o, lse, causal=True, window=None, scale=None), iters=3, warmup=2)
    flops = 5.0 * B * H * T * T * D
    results.append({"kernel": "flash_bwd_small", "ms": ms, "tflops": flops / ms / 1e9})
    print(f"flash bwd small B{B} H{H} T{T}: {ms:7.3f} ms {flops / ms / 1e9:7.1f} TF/s", flush=True)


def _gdr_inputs(B, S, Hk, Hv, dv, dev):
    g = torch.Generator(device=dev).manual_seed(0)
    rn = lambda *shape: torch.randn(*shape, device=dev, generator=g)
    q, k, v = rn(B, S, Hk, 128).bfloat16(), rn(B, S, Hk, 128).bfloat16(), rn(B, S, Hv, dv).bfloat16()
    return q, k, v, -torch.nn.functional.softplus(rn(B, S, Hv)) * 0.3, torch.sigmoid(rn(B, S, Hv))


def bench_gdr(results, small=False):
    """Gated delta rule prefill (chunk 64): the two chunk kernels against the library-op form of the same algorithm
    (Qwen3.5-27B head counts: 16 key / 48 value heads of 128).  ``small``: one case for profiler captures."""
    from tyr_b200.ops import delta_rule as DR
    dev = torch.device("cuda")
    flush = None if small else torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for B, S in (((2, 2048),) if small else ((8, 2048), (1, 8192))):
        q, k, v, gl, beta = _gdr_inputs(B, S, 16, 48, 128, dev)
        iters, warm = (3, 2) if small else (10, 3)
        ours = _time(lambda: DR.chunk_gated_delta_rule(q, k, v, gl, beta), iters=iters, warmup=warm, flush=flush)
        row = {"kernel": "gdr_chunk", "B": B, "S": S, "ours_ms": ours}
        if not small:
            DR._CHUNK_KERNEL = False
            try:
                row["library_ms"] = _time(lambda: DR.chunk_gated_delta_rule(q, k, v, gl, beta), iters=5, warmup=2, flush=flush)
            finally:
                DR._CHUNK_KERNEL = True
        results.append(row)
        print(f"gated delta rule prefill B{B} S{S} 16/48 heads x 128: ours {ours:7.3f} ms" + (f" | library ops {row['library_ms']:7.3f} ms" if "library_ms" in row else ""), flush=True)


def bench_gdr_decode(results, small=False):
    """Gated delta rule, one token per row (decode): bound by one read and one write of the fp32 state
    [B, value heads, 128, 128]; reports the fraction of the measured copy bandwidth."""
    from tyr_b200.ops import delta_rule as DR
    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    peak = 6538.0                      # measured copy bandwidth of this pool, GB/s
    for B, Hk, Hv in (((32, 8, 24),) if small else ((32, 8, 24), (32, 16, 48), (8, 16, 48), (64, 16, 48))):
        q, k, v, gl, beta = _gdr_inputs(B, 1, Hk, Hv, 128, dev)
        state = torch.randn(B, Hv, 128, 128, device=dev) * 0.1
        gl, beta = gl.float().contiguous(), beta.float().contiguous()
        fn = lambda: DR.gdr_decode_step(q, k, v, gl, beta, state)
        ms = _time(fn, iters=3 if small else 20, warmup=2 if small else 5, flush=flush)
        gbs = 2.0 * state.numel() * 4 / ms / 1e6
        results.append({"kernel": "gdr_decode", "B": B, "Hv": Hv, "ms": ms, "gbs": gbs, "of_measured_copy": gbs / peak})
        print(f"gated delta rule decode B{B} {Hk}/{Hv} heads x 128: {ms * 1e3:7.1f} us  {gbs:7.0f} GB/s  ({gbs / peak:.2f} of measured copy)", flush=True)


def bench_moe(results, cases=None):
    """Fused NVFP4 MoE op at Laguna-S-2.1 shapes (hidden 3072, 256 experts, top-10, FFN 1024): effective
    FP4 weight-read bandwidth for decode-sized batches (the reference's bar is >= 150 GB/s at one token,
    Tests/RunLagunaFused.lean:373-386) and tokens/s for prefill-sized batches."""
    from tyr_b200.models import laguna as L
    from tyr_b200.ops import moe
    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    cfg = L.LagunaConfig()
    gen = torch.Generator().manual_seed(0)
    ex = L.random_packed_experts(cfg, dev, gen)
    E, k, h, mi = cfg.num_experts, cfg.num_experts_per_tok, cfg.hidden_size, cfg.moe_intermediate_size
    for T, path in cases or ((1, "gemv"), (4, "gemv"), (16, "gemv"), (64, "gemv"), (32, "gemm_sorted"), (32, "gemm"), (64, "gemm_sorted"), (64, "gemm"), (128, "gemm_sorted"), (128, "gemm"), (512, "gemm"), (4096, "gemm")):
        x = torch.randn(T, h, device=dev).bfloat16()
        ids, w, cnt = moe.route(torch.randn(T, E, device=dev), k)
        fn = lambda: moe.moe_fp4_forward(x, ids, w, ex, counts=cnt, force_path=path)
        ms = _time(fn, flush=flush)
        active = int((cnt > 0).sum())
        fp4_bytes = ex.weight_bytes_per_pair() * (T * k if path == "gemv" and T == 1 else active)
        flops = 6.0 * T * k * h * mi
        row = {"kernel": "moe_fp4_" + path, "tokens": T, "ms": ms, "active_experts": active,
               "fp4_gbs": fp4_bytes / ms / 1e6, "tflops": flops / ms / 1e9, "tokens_per_s": T / ms * 1e3}
        results.append(row)
        print(f"moe {path} T={T:5d}: {ms:8.3f} ms  unique-expert FP4 read {row['fp4_gbs']:8.1f} GB/s  {row['tflops']:7.1f} TF/s  "
              f"{row['tokens_per_s']:10.0f} tok/s", flush=True)


def bench_decode_attention_small(results):
    """One small case for profiler captures: K/V of 134 MB (larger than L2), two warm-up and three timed launches."""
    from tyr_b200.ops.decode_attention import decode_attention
    dev = torch.device("cuda")
    B, Hq, Hkv, D, pos = 8, 48, 8, 128, 4096
    q, kn, vn = (torch.randn(B, n, D, device=dev).bfloat16() for n in (Hq, Hkv, Hkv))
    kc, vc = torch.randn(B, Hkv, pos + 64, D, device=dev).bfloat16(), torch.randn(B, Hkv, pos + 64, D, device=dev).bfloat16()
    pt = torch.tensor([pos], dtype=torch.int32, device=dev)
    ms = _time(lambda: decode_attention(q, kn, vn, kc, vc, pt), iters=3, warmup=2)
    gb = 2.0 * B * Hkv * (pos + 1) * D * 2 / 1e9
    results.append({"kernel": "decode_attention", "case": "small b8", "ms": ms, "gbs": gb / ms * 1e3})
    print(f"decode attention small b8: {ms:7.3f} ms {gb / ms * 1e3:7.0f} GB/s", flush=True)


def bench_decode_attention(results):
    """Split-KV decode attention with fused append against the library SDPA over the sliced store: Laguna-S-2.1
    (48 q / 8 kv heads x 128) and Qwen3.5-27B (24 q / 4 kv heads x 256) geometries; bandwidth counts the K/V bytes read."""
    import torch.nn.functional as F
    from tyr_b200.ops.decode_attention import decode_attention
    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for name, B, Hq, Hkv, D, pos in (("laguna b64", 64, 48, 8, 128, 4096), ("laguna b1", 1, 48, 8, 128, 4096), ("qwen27b b32", 32, 24, 4, 256, 2048),
                                     ("laguna b64 long", 64, 48, 8, 128, 16384)):
        cap = pos + 64
        q, kn, vn = (torch.randn(B, n, D, device=dev).bfloat16() for n in (Hq, Hkv, Hkv))
        kc, vc = torch.randn(B, Hkv, cap, D, device=dev).bfloat16(), torch.randn(B, Hkv, cap, D, device=dev).bfloat16()
        pt = torch.tensor([pos], dtype=torch.int32, device=dev)
        ours = _time(lambda: decode_attention(q, kn, vn, kc, vc, pt), flush=flush)

        def lib_path():
            kc[:, :, pos] = kn
            vc[:, :, pos] = vn
            return F.scaled_dot_product_attention(q.unsqueeze(2), kc[:, :, :pos + 1], vc[:, :, :pos + 1], enable_gqa=True)
        libms = _time(lib_path, flush=flush)
        gb = 2.0 * B * Hkv * (pos + 1) * D * 2 / 1e9
        results.append({"kernel": "decode_attention", "case": name, "ms": ours, "gbs": gb / ours * 1e3, "sdpa_ms": libms, "sdpa_gbs": gb / libms * 1e3})
        print(f"decode attention {name:16s}: ours {ours:7.3f} ms {gb / ours * 1e3:7.0f} GB/s | append+SDPA {libms:7.3f} ms {gb / libms * 1e3:7.0f} GB/s", flush=True)


def bench_skinny(results):
    """Weight-streaming linear for decode-sized batches against the library GEMM: Laguna / Qwen3.5 projection shapes and
    the Laguna lm_head; bandwidth counts the weight bytes."""
    import torch.nn.functional as F
    from tyr_b200.ops.skinny import skinny_linear
    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for M, N, K in ((1, 11336, 3072), (1, 3072, 9216), (1, 100352, 3072), (8, 11336, 3072), (8, 34816, 5120), (16, 5120, 17408)):
        w = (torch.randn(N, K, device=dev) * K ** -0.5).bfloat16()
        x = torch.randn(M, K, device=dev).bfloat16()
        ours = _time(lambda: skinny_linear(x, w), flush=flush)
        libms = _time(lambda: F.linear(x, w), flush=flush)
        gb = N * K * 2 / 1e9
        results.append({"kernel": "skinny_gemm", "M": M, "N": N, "K": K, "ms": ours, "gbs": gb / ours * 1e3, "lib_ms": libms, "lib_gbs": gb / libms * 1e3})
        print(f"skinny M={M:2d} N={N:6d} K={K:5d}: ours {ours * 1e3:7.1f} us {gb / ours * 1e3:6.0f} GB/s | library {libms * 1e3:7.1f} us {gb / libms * 1e3:6.0f} GB/s", flush=True)


def bench_decode_gemm(results, small=False):
    """Tensor-core weight-streaming linear for 17 .. 64 rows (csrc/decode_gemm.cu) against the library GEMM and, for the
    gated form at up to 32 rows, against the mma.sync weight-streaming kernel; Qwen3.5-27B MLP shapes, whole and halved
    (tensor parallel over two GPUs).  Bandwidth counts the weight bytes; fraction of the measured copy bandwidth."""
    import torch.nn.functional as F
    from tyr_b200.ops import decode_gemm as DG
    from tyr_b200.ops import skinny
    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    cases = ((32, 17408, 5120, True),) if small else ((32, 17408, 5120, True), (64, 17408, 5120, True), (32, 8704, 5120, True),
                                                      (32, 17408, 5120, False), (32, 5120, 17408, False), (64, 5120, 17408, False),
                                                      (32, 12288, 5120, False))
    for M, N, K, gated in cases:
        w = (torch.randn(N, K, device=dev) * K ** -0.5).bfloat16()
        w2 = (torch.randn(N, K, device=dev) * K ** -0.5).bfloat16() if gated else None
        x = torch.randn(M, K, device=dev).bfloat16()
        it, wu = (3, 2) if small else (20, 5)
        if gated:
            ours = _time(lambda: DG.decode_swiglu(x, w, w2), iters=it, warmup=wu, flush=flush)
            libms = _time(lambda: F.silu(F.linear(x, w)) * F.linear(x, w2), iters=it, warmup=wu, flush=flush)
            old = _time(lambda: skinny.skinny_swiglu(x, w, w2), iters=it, warmup=wu, flush=flush) if M <= 32 else float("nan")
        else:
            ours = _time(lambda: DG.decode_linear(x, w), iters=it, warmup=wu, flush=flush)
            libms = _time(lambda: F.linear(x, w), iters=it, warmup=wu, flush=flush)
            old = float("nan")
        gb = (2 if gated else 1) * N * K * 2 / 1e9
        results.append({"kernel": "decode_gemm_" + ("swiglu" if gated else "plain"), "M": M, "N": N, "K": K, "ms": ours, "gbs": gb / ours * 1e3,
                        "of_measured_copy": gb / ours * 1e3 / 6538.0, "lib_ms": libms, "mma_sync_ms": old})
        print(f"decode gemm {'swiglu' if gated else 'plain '} M={M:2d} N={N:6d} K={K:5d}: ours {ours * 1e3:7.1f} us {gb / ours * 1e3:6.0f} GB/s "
              f"({gb / ours * 1e3 / 6538.0:.2f} of measured copy) | library {libms * 1e3:7.1f} us | mma.sync kernel {old * 1e3:7.1f} us", flush=True)


def bench_gemm_fwd_small(results):
    """The forward qkv projection of NanoChat d20 alone, few launches: the case to put under a profiler."""
    from tyr_b200.ops.gemm import gemm
    dev = torch.device("cuda")
    a = torch.randn(65536, 1280, device=dev).bfloat16()
    b = torch.randn(3840, 1280, device=dev).bfloat16()
    ms = _time(lambda: gemm(a, b, a_layout="K", b_layout="K"), iters=3, warmup=2)
    results.append({"kernel": "gemm", "shape": "fwd qkv [65536x1280]x[3840x1280]^T", "ours_ms": ms, "ours_tflops": 2.0 * 65536 * 3840 * 1280 / ms / 1e9})
    print(f"fwd qkv: {ms:.3f} ms", flush=True)


def bench_qwen3_decode(results):
    """Greedy decode through ``Qwen3Session`` (random-init Qwen3-4B shape, 1024-token prompt, 64 timed steps) for
    batch 1 and 8, once replaying the captured step graph and once launching the same kernels eagerly."""
    import os
    from tyr_b200.models import qwen as Q
    dev = torch.device("cuda")
    cfg = Q.QwenConfig.qwen3_4b()
    lm = Q.Qwen3ForCausalLM.init(cfg, device=dev, dtype=torch.bfloat16, seed=0)
    saved = os.environ.get("TYR_DECODE_GRAPH")
    try:
        for B in (1, 8):
            ids = torch.randint(0, cfg.vocab_size, (B, 1024), device=dev)
            for graph in ("1", "0"):
                os.environ["TYR_DECODE_GRAPH"] = graph
                with torch.no_grad():
                    s = Q.Qwen3Session(lm, B, 1024 + 80)
                    tok = s.prefill(ids).argmax(-1)
                    for _ in range(3):                       # the first step of a session captures its graph
                        tok = s.step(tok).argmax(-1)
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    torch.cuda.synchronize()
                    e0.record()
                    for _ in range(64):
                        tok = s.step(tok).argmax(-1)
                    e1.record()
                    torch.cuda.synchronize()
                ms = e0.elapsed_time(e1) / 64
                results.append({"kernel": "qwen3_4b_decode", "batch": B, "graph": graph == "1", "ms_per_step": ms, "tok_s": B / ms * 1e3})
                print(f"qwen3-4b decode batch {B} graph={graph}: {B / ms * 1e3:8.1f} tok/s, {ms:.2f} ms/step", flush=True)
                del s
    finally:
        if saved is None:
            os.environ.pop("TYR_DECODE_GRAPH", None)
        else:
            os.environ["TYR_DECODE_GRAPH"] = saved


def bench_elementwise(results, small=False):
    """Bandwidth-bound kernels of the NanoChat and Flux steps at their production shapes (``small``: an eighth of the
    rows, still larger than L2, few launches: the case to put under a profiler).  Achieved GB/s counts the algorithmic
    bytes (every operand read once, every result written once) against the measured copy bandwidth of 6538 GB/s."""
    from tyr_b200 import ops
    from tyr_b200.ops import ce as CE
    from tyr_b200.ops import modulate as MOD
    dev = torch.device("cuda")
    flush = None if small else torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    it = dict(iters=3, warmup=2) if small else dict()
    N, d, H, D, T = (8192 if small else 65536), 1280, 10, 128, 2048
    g = torch.Generator(device="cuda").manual_seed(0)
    rnd = lambda *sh: torch.randn(*sh, device=dev, generator=g).bfloat16()

    def row(name, ms, nbytes):
        results.append({"kernel": name, "ms": ms, "gbs": nbytes / ms / 1e6, "fraction_of_copy_bw": nbytes / ms / 1e6 / 6538.0})
        print(f"{name:34s} {ms:8.3f} ms  {nbytes / ms / 1e6:8.1f} GB/s  {nbytes / ms / 1e6 / 6538.0:5.2f} of measured copy bandwidth", flush=True)

    # lincomb + RMSNorm, three inputs, forward and backward
    xs = [rnd(N, d).requires_grad_(True) for _ in range(3)]
    sc = torch.tensor([0.7, 0.3, 0.5], device=dev, requires_grad=True)
    t = N * d * 2
    row("lincomb_rmsnorm_fwd<3>", _time(lambda: ops.lincomb_rmsnorm(xs, sc), flush=flush, **it), 5 * t)
    out, normed = ops.lincomb_rmsnorm(xs, sc)
    go, gn = rnd(N, d), rnd(N, d)
    row("lincomb_rmsnorm_bwd<3>", _time(lambda: torch.autograd.grad([out, normed], xs + [sc], [go, gn], retain_graph=True),
                                        flush=flush, **it), 8 * t)
    # RoPE + QK norm + value-embedding blend on the packed projection, forward and backward
    qkv = rnd(N, 3 * H * D).requires_grad_(True)
    ve = rnd(N, H * D).requires_grad_(True)
    mix = torch.tensor(0.4, device=dev, requires_grad=True)
    cos, sin = ops.rotary_freqs(T, D, 500000.0, device=dev)
    q3 = N * 3 * H * D * 2
    row("qkv_post_fwd", _time(lambda: ops.qkv_post(qkv, ve, mix, cos, sin, T, H, D), flush=flush, **it), 2 * q3 + q3 // 3)
    y = ops.qkv_post(qkv, ve, mix, cos, sin, T, H, D)
    gy = rnd(N, 3 * H * D)
    row("qkv_post_bwd", _time(lambda: torch.autograd.grad(y, [qkv, ve, mix], gy, retain_graph=True), flush=flush, **it),
        3 * q3 + 2 * (q3 // 3))
    # soft-capped cross-entropy with the gradient written in place
    rows_ce, V = (1024 if small else 8192), 65536
    logits = rnd(rows_ce, V)
    tg = torch.randint(0, V, (rows_ce,), device=dev, generator=g)
    row("softcap_ce (fwd + grad in place)", _time(lambda: CE.softcap_ce_(logits, tg, 15.0), flush=flush, **it), 2 * rows_ce * V * 2)
    # Flux modulation kernels
    B, S, Df = (1 if small else 4), 4608, 3072
    x = rnd(B, S, Df)
    mod = rnd(B, 3 * Df)
    xb = B * S * Df * 2
    row("layernorm_modulate", _time(lambda: MOD.layernorm_modulate(x, mod[:, :Df], mod[:, Df:2 * Df]), flush=flush, **it), 2 * xb)
    yv = rnd(B, S, Df)
    row("gate_residual", _time(lambda: MOD.gate_residual(x, yv, mod[:, 2 * Df:]), flush=flush, **it), 3 * xb)


def bench_ns(results, small=False):
    """Newton-Schulz chain (5 iterations, 15 batched tcgen05 GEMMs with the scale / add terms in their epilogues) on the two
    Muon shape classes of NanoChat d20; ``small``: 8 matrices, few launches, for a profiler."""
    from tyr_b200.ops import polar
    dev = torch.device("cuda")
    flush = None if small else torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    it = dict(iters=3, warmup=2) if small else dict()
    for name, (Bm, R, C) in (("attention matrices", (8 if small else 76, 1280, 1280)), ("MLP matrices", (4 if small else 40, 5120, 1280))):
        x = torch.randn(Bm, R, C, device=dev)
        x = (x / x.pow(2).sum((1, 2), keepdim=True).sqrt()).bfloat16().contiguous()
        ms = _time(lambda: polar.newton_schulz_(x.clone(), 5), flush=flush, **it)
        S = min(R, C)
        flops = 5 * Bm * (2.0 * S * S * max(R, C) + 2.0 * S * S * S + 2.0 * S * S * max(R, C))
        results.append({"kernel": "newton_schulz", "shape": f"{Bm}x[{R}x{C}]", "ms": ms, "tflops": flops / ms / 1e9})
        print(f"newton_schulz {name:20s} {Bm}x[{R}x{C}]: {ms:8.3f} ms  {flops / ms / 1e9:7.1f} TF/s", flush=True)


def bench_fp4_small(results):
    """The block-scaled FP4 expert path on a case sized for a profiler: 2048 tokens, 64 experts top-8, hidden 2048, FFN 768."""
    from tyr_b200.models import laguna as L
    from tyr_b200.ops import moe
    dev = torch.device("cuda")
    cfg = L.LagunaConfig(hidden_size=2048, num_experts=64, num_experts_per_tok=8, moe_intermediate_size=768)
    ex = L.random_packed_experts(cfg, dev, torch.Generator().manual_seed(0))
    T = 2048
    x = torch.randn(T, 2048, device=dev).bfloat16()
    ids, w, cnt = moe.route(torch.randn(T, 64, device=dev), 8)
    ms = _time(lambda: moe.moe_fp4_forward(x, ids, w, ex, counts=cnt, force_path="gemm"), iters=3, warmup=2)
    flops = 6.0 * T * 8 * 2048 * 768
    results.append({"kernel": "moe_fp4_tensor_core", "tokens": T, "ms": ms, "tflops": flops / ms / 1e9})
    print(f"moe fp4 tensor-core path T={T}: {ms:.3f} ms {flops / ms / 1e9:.1f} TF/s", flush=True)


def main(argv):
    what = argv[1] if len(argv) > 1 else "all"
    results = []
    if what == "gemm-fwd-small":
        bench_gemm_fwd_small(results)
    if what == "qwen3-decode":
        bench_qwen3_decode(results)
    if what in ("gemm", "all"):
        bench_gemm(results)
    if what in ("attention", "all"):
        bench_attention(results)
    if what in ("attention-bwd", "all"):
        bench_attention_bwd(results)
    if what in ("gdr", "all"):
        bench_gdr(results)
    if what in ("decode-gemm", "all"):
        bench_decode_gemm(results)
    if what == "decode-gemm-small":
        bench_decode_gemm(results, small=True)
    if what in ("gdr-decode", "all"):
        bench_gdr_decode(results)
    if what == "gdr-decode-small":
        bench_gdr_decode(results, small=True)
    if what == "gdr-small":
        bench_gdr(results, small=True)
    if what == "attention-fwd-small":
        bench_attention_fwd_small(results)
    if what == "attention-bwd-small":
        bench_attention_bwd_small(results)
    if what in ("moe", "all"):
        bench_moe(results)
    if what in ("decode-attn", "all"):
        bench_decode_attention(results)
    if what == "decode-attn-small":
        bench_decode_attention_small(results)
    if what in ("skinny", "all"):
        bench_skinny(results)
    if what in ("elementwise", "all"):
        bench_elementwise(results)
    if what == "elementwise-small":
        bench_elementwise(results, small=True)
    if what in ("ns", "all"):
        bench_ns(results)
    if what == "ns-small":
        bench_ns(results, small=True)
    if what == "fp4-small":
        bench_fp4_small(results)
    if what == "moe-decode":
        bench_moe(results, ((1, "gemv"), (64, "gemv")))
    print(json.dumps(results))


if __name__ == "__main__":
    main(sys.argv)
