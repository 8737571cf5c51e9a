"""Kernel micro-benchmarks: `python -m benchmarks.kernel_bench [gemm|attention|moe|moe-decode|decode-attn|skinny|qwen3-decode|all]`.

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
    for T, path in cases or ((1, "gemv"), (4, "gemv"), (16, "gemv"), (64, "gemv"), (64, "gemm"), (512, "gemm"), (4096, "gemm")):
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
    if what == "moe-decode":
        bench_moe(results, ((1, "gemv"), (64, "gemv")))
    print(json.dumps(results))


if __name__ == "__main__":
    main(sys.argv)
