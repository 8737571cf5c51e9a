// Decode-step attention with the KV append fused in and the sequence position read from device memory, so that a
// whole decode step can be replayed from a CUDA graph.
//
// One new query row per (batch, head); K/V stores [B, Hkv, cap, D] bf16 (plain or ring).  Grid (splits, Hkv, B): a CTA
// owns the G = Hq / Hkv <= 16 query heads of one K/V head over one slice of the retained keys (split-KV, 4 warps, 16 keys
// per warp step).  Both products run on mma.sync m16n8k16 with the operand fragments loaded straight from global
// memory, 16 bytes per lane (see the kernel's comment for the channel / key permutations that make this possible).
// The key at the new position is taken from k_new / v_new rather than from the store, so the append (done by split 0)
// cannot race with readers.  Split partials {m, l, acc} go to a workspace; the last CTA to arrive for a
// (batch, K/V head) combines them (atomic ticket, counter reset for the next launch).
//
// The reference takes the library SDPA over a sliced cache for this step (cc/include/tyr_attention.h:58-130,
// Tyr/Inference/KVCache.lean:41-215).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace tyr {

constexpr int kDecWarps = 4;

struct DecodeAttnArgs {
  const __nv_bfloat16* q;        // [B, Hq, D], batch stride q_bs, head stride D
  const __nv_bfloat16* k_new;    // [B, Hkv, D], batch stride kn_bs, head stride D
  const __nv_bfloat16* v_new;    // same strides (vn_bs)
  __nv_bfloat16* k_cache;        // [B, Hkv, cap, D]
  __nv_bfloat16* v_cache;
  const int* pos;                // absolute position of the new token
  __nv_bfloat16* out;            // [B, Hq, D] contiguous
  float* part_acc;               // [B, Hq, splits, D]
  float* part_ml;                // [B, Hq, splits, 2]
  int* counters;                 // [B * Hkv], zero on entry, zero on exit
  long long q_bs, kn_bs, vn_bs;
  int B, Hq, Hkv, cap, ring, window, splits, append;
  float scale_log2;
  int* err;
  // optional output gate, applied when the result is written: mode 1 = one value per (batch, head), out *= softplus(g)
  // (Laguna); mode 2 = one value per element, out *= sigmoid(g) (Qwen3.5).  Element (b, h, d) is at gate + b * gate_bs +
  // h * gate_hs (+ d in mode 2).
  const __nv_bfloat16* gate;
  long long gate_bs, gate_hs;
  int gate_mode;
};

__device__ __forceinline__ float decode_gate(const DecodeAttnArgs& a, int b, int h, int d) {
  if (a.gate_mode == 1) {
    const float g = __bfloat162float(a.gate[b * a.gate_bs + h * a.gate_hs]);
    return g > 20.f ? g : log1pf(__expf(g));
  }
  if (a.gate_mode == 2) {
    const float g = __bfloat162float(a.gate[b * a.gate_bs + h * a.gate_hs + d]);
    return 1.f / (1.f + __expf(-g));
  }
  return 1.f;
}

// One m16n8k16 step.  `lo` accumulates the tile's rows 0..7 (query head g of the lane), `hi` rows 8..15 (head g + 8).
// With at most 8 query heads per K/V head the upper rows are padding: their A registers are zero and their accumulators
// scratch, which halves the live registers.
template <bool WIDE>
__device__ __forceinline__ void mma_bf16_16816(float (&lo)[2], float (&hi)[2], uint32_t a_lo0, uint32_t a_lo2, uint32_t a_hi0, uint32_t a_hi2,
                                               uint32_t b0, uint32_t b1) {
  if constexpr (WIDE) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(lo[0]), "+f"(lo[1]), "+f"(hi[0]), "+f"(hi[1])
                 : "r"(a_lo0), "r"(a_hi0), "r"(a_lo2), "r"(a_hi2), "r"(b0), "r"(b1));
  } else {
    float z0 = 0.f, z1 = 0.f;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(lo[0]), "+f"(lo[1]), "+f"(z0), "+f"(z1)
                 : "r"(a_lo0), "r"(0u), "r"(a_lo2), "r"(0u), "r"(b0), "r"(b1));
  }
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

// Tensor-core formulation (mma.sync m16n8k16, bf16 in, fp32 accumulate); one warp consumes 16 keys per step.
//   S = Q K^T : M = query heads of the group (<= 8 real rows), N = 8 keys, K = 16 channels.  The reduction over channels
//   is order-free, so lane (g, t) feeds the B fragment straight from one 16-byte load of key row g (channels
//   32j + 8t .. +8) and Q is loaded once with the same addressing.
//   O += P V  : M = heads, N = 8 channels, K = 16 keys.  Lane (g, t) loads 16 bytes (8 channels) of the four key rows
//   {2t, 2t+1, 2t+8, 2t+9}; byte permutes pair the rows per channel.  The channel order of the accumulators is permuted
//   (undone when they are written out): accumulator (c, e, u) of lane (g, t) is channel 64c + 16t + 8u + e of head g.
template <int D, bool WIDE>
__global__ void __launch_bounds__(kDecWarps * 32) decode_attention_kernel(DecodeAttnArgs a) {
  pdl_entry();
  constexpr int NJ = D / 32;                     // 16-byte chunks per lane of a K (or Q) row
  constexpr int NC = D / 64;                     // 64-channel blocks of a V row
  constexpr int R = WIDE ? 2 : 1;                // query heads per lane: g, and g + 8 when more than 8 heads share a K/V head
  constexpr int GM = 8 * R;
  __shared__ float s_m[kDecWarps][GM], s_l[kDecWarps][GM];
  __shared__ float s_acc[kDecWarps][GM][D];
  __shared__ int s_ticket;

  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int G = a.Hq / a.Hkv;
  const int pos = *a.pos;
  if (pos < 0 || (!a.ring && pos >= a.cap)) {    // position outside the store: report, leave the output untouched
    if (tid == 0) report_error(a.err, ERR_BOUNDS, pos);
    return;
  }
  int start, n_keys, slot_new;
  if (a.ring) {
    start = 0;
    n_keys = pos + 1 < a.cap ? pos + 1 : a.cap;
    slot_new = pos % a.cap;
  } else {
    start = (a.window > 0 && pos + 1 > a.window) ? pos + 1 - a.window : 0;
    n_keys = pos + 1 - start;
    slot_new = pos;
  }
  int chunk = (n_keys + a.splits - 1) / a.splits;
  chunk = (chunk + 63) & ~63;
  const int lo = start + split * chunk;
  int hi = lo + chunk;
  if (hi > start + n_keys) hi = start + n_keys;

  const long long kv_base = (static_cast<long long>(b) * a.Hkv + hkv) * a.cap * D;
  const __nv_bfloat16* kc = a.k_cache + kv_base;
  const __nv_bfloat16* vc = a.v_cache + kv_base;
  const __nv_bfloat16* kn = a.k_new + b * a.kn_bs + static_cast<long long>(hkv) * D;
  const __nv_bfloat16* vn = a.v_new + b * a.vn_bs + static_cast<long long>(hkv) * D;

  if (a.append && split == 0) {                  // fused append; nobody reads this slot from the store in this launch
    for (int i = tid; i < D / 8; i += kDecWarps * 32) {
      reinterpret_cast<uint4*>(a.k_cache + kv_base + static_cast<long long>(slot_new) * D)[i] = reinterpret_cast<const uint4*>(kn)[i];
      reinterpret_cast<uint4*>(a.v_cache + kv_base + static_cast<long long>(slot_new) * D)[i] = reinterpret_cast<const uint4*>(vn)[i];
    }
  }

  uint4 qf[R][NJ];                               // A fragments of heads g (and g + 8); zero rows beyond G
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int head = g + 8 * r;
    const __nv_bfloat16* qrow = a.q + b * a.q_bs + static_cast<long long>(hkv * G + (head < G ? head : 0)) * D;
#pragma unroll
    for (int j = 0; j < NJ; ++j) qf[r][j] = head < G ? *reinterpret_cast<const uint4*>(qrow + 32 * j + 8 * t) : make_uint4(0u, 0u, 0u, 0u);
  }
  float m[R], l[R];                              // running max (same in the four lanes of a head) and per-lane partial sum
  float o[R][NC][8][2];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
      for (int e = 0; e < 8; ++e) o[r][c][e][0] = o[r][c][e][1] = 0.f;
  }

  for (int base = lo + warp * 16; base < hi; base += kDecWarps * 16) {
    // ---- S for 16 keys: key tiles base + [0, 8) and base + [8, 16) ----
    float s[R][2][2];
#pragma unroll
    for (int tile = 0; tile < 2; ++tile) {
      int row = base + 8 * tile + g;
      row = row < hi ? row : hi - 1;             // clamped rows are masked below
      const __nv_bfloat16* krow = (row == slot_new) ? kn : kc + static_cast<long long>(row) * D;
      uint4 kf[NJ];
#pragma unroll
      for (int j = 0; j < NJ; ++j) kf[j] = *reinterpret_cast<const uint4*>(krow + 32 * j + 8 * t);
      float c_lo[2] = {0.f, 0.f}, c_hi[2] = {0.f, 0.f};
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        mma_bf16_16816<WIDE>(c_lo, c_hi, qf[0][j].x, qf[0][j].y, qf[R - 1][j].x, qf[R - 1][j].y, kf[j].x, kf[j].y);
        mma_bf16_16816<WIDE>(c_lo, c_hi, qf[0][j].z, qf[0][j].w, qf[R - 1][j].z, qf[R - 1][j].w, kf[j].z, kf[j].w);
      }
      const int key0 = base + 8 * tile + 2 * t;
      s[0][tile][0] = key0 < hi ? c_lo[0] * a.scale_log2 : -INFINITY;
      s[0][tile][1] = key0 + 1 < hi ? c_lo[1] * a.scale_log2 : -INFINITY;
      if constexpr (WIDE) {
        s[1][tile][0] = key0 < hi ? c_hi[0] * a.scale_log2 : -INFINITY;
        s[1][tile][1] = key0 + 1 < hi ? c_hi[1] * a.scale_log2 : -INFINITY;
      }
    }
    // ---- V rows of this lane's four keys (issued before the softmax arithmetic so the loads overlap it) ----
    const __nv_bfloat16* vrow[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int row = base + 2 * t + (i & 1) + 8 * (i >> 1);
      row = row < hi ? row : hi - 1;
      vrow[i] = (row == slot_new) ? vn : vc + static_cast<long long>(row) * D;
    }
    uint4 vf[NC][4];
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
      for (int i = 0; i < 4; ++i) vf[c][i] = *reinterpret_cast<const uint4*>(vrow[i] + 64 * c + 8 * g);

    // ---- online softmax per head (its 16 scores live in the four lanes t = 0..3) ----
    uint32_t pa0[R], pa2[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float mx = fmaxf(fmaxf(s[r][0][0], s[r][0][1]), fmaxf(s[r][1][0], s[r][1][1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m[r], mx);       // finite: key `base` is always in range
      const float alpha = exp2f(m[r] - m_new);
      const float p00 = exp2f(s[r][0][0] - m_new), p01 = exp2f(s[r][0][1] - m_new);
      const float p10 = exp2f(s[r][1][0] - m_new), p11 = exp2f(s[r][1][1] - m_new);
      l[r] = l[r] * alpha + (p00 + p01) + (p10 + p11);
      if (__any_sync(0xffffffffu, m_new > m[r])) {
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
          for (int e = 0; e < 8; ++e) { o[r][c][e][0] *= alpha; o[r][c][e][1] *= alpha; }
      }
      m[r] = m_new;
      pa0[r] = pack_bf16x2(p00, p01);
      pa2[r] = pack_bf16x2(p10, p11);
    }

    // ---- O += P V ----
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const uint32_t v0[4] = {vf[c][0].x, vf[c][0].y, vf[c][0].z, vf[c][0].w};
      const uint32_t v1[4] = {vf[c][1].x, vf[c][1].y, vf[c][1].z, vf[c][1].w};
      const uint32_t v2[4] = {vf[c][2].x, vf[c][2].y, vf[c][2].z, vf[c][2].w};
      const uint32_t v3[4] = {vf[c][3].x, vf[c][3].y, vf[c][3].z, vf[c][3].w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;
        mma_bf16_16816<WIDE>(o[0][c][e], o[R - 1][c][e], pa0[0], pa2[0], pa0[R - 1], pa2[R - 1],
                             prmt(v0[e >> 1], v1[e >> 1], sel), prmt(v2[e >> 1], v3[e >> 1], sel));
      }
    }
  }

  // publish this warp's state: heads g (and g + 8), channels as laid out above
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float lr = l[r];
    lr += __shfl_xor_sync(0xffffffffu, lr, 1);
    lr += __shfl_xor_sync(0xffffffffu, lr, 2);
    const int head = g + 8 * r;
    if (head < G) {
      if (t == 0) { s_m[warp][head] = m[r]; s_l[warp][head] = lr; }
#pragma unroll
      for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          s_acc[warp][head][64 * c + 16 * t + e] = o[r][c][e][0];
          s_acc[warp][head][64 * c + 16 * t + 8 + e] = o[r][c][e][1];
        }
    }
  }

  // ---- combine the four warps -------------------------------------------------------------------------------
  __syncthreads();
  const int hq0 = hkv * G;
  for (int i = tid; i < G * D; i += kDecWarps * 32) {
    const int g = i / D, d = i - g * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) M = fmaxf(M, s_m[w][g]);
    float L = 0.f, A = 0.f;
    if (M > -INFINITY) {
#pragma unroll
      for (int w = 0; w < kDecWarps; ++w) {
        const float f = exp2f(s_m[w][g] - M);
        L += s_l[w][g] * f;
        A += s_acc[w][g][d] * f;
      }
    }
    const long long row = static_cast<long long>(b) * a.Hq + hq0 + g;
    if (a.splits == 1) {
      a.out[row * D + d] = __float2bfloat16((L > 0.f ? A / L : 0.f) * decode_gate(a, b, hq0 + g, d));
    } else {
      a.part_acc[(row * a.splits + split) * D + d] = A;
      if (d == 0) {
        a.part_ml[(row * a.splits + split) * 2] = M;
        a.part_ml[(row * a.splits + split) * 2 + 1] = L;
      }
    }
  }
  if (a.splits == 1) return;

  // ---- last CTA of this (batch, K/V head) merges the splits ---------------------------------------------------
  __threadfence();
  __syncthreads();
  if (tid == 0) s_ticket = atomicAdd(&a.counters[b * a.Hkv + hkv], 1);
  __syncthreads();
  if (s_ticket != a.splits - 1) return;
  __threadfence();
  for (int i = tid; i < G * D; i += kDecWarps * 32) {
    const int g = i / D, d = i - g * D;
    const long long row = static_cast<long long>(b) * a.Hq + hq0 + g;
    float M = -INFINITY;
    for (int sp = 0; sp < a.splits; ++sp) M = fmaxf(M, __ldcg(&a.part_ml[(row * a.splits + sp) * 2]));
    float L = 0.f, A = 0.f;
    if (M > -INFINITY) {
      for (int sp = 0; sp < a.splits; ++sp) {
        const float f = exp2f(__ldcg(&a.part_ml[(row * a.splits + sp) * 2]) - M);
        L += __ldcg(&a.part_ml[(row * a.splits + sp) * 2 + 1]) * f;
        A += __ldcg(&a.part_acc[(row * a.splits + sp) * D + d]) * f;
      }
    }
    a.out[row * D + d] = __float2bfloat16((L > 0.f ? A / L : 0.f) * decode_gate(a, b, hq0 + g, d));
  }
  if (tid == 0) a.counters[b * a.Hkv + hkv] = 0;
}

}  // namespace tyr

// Workspace: floats for the split partials followed by the ticket counters.
extern "C" TYR_EXPORT long long tyr_decode_attention_workspace_bytes(int B, int Hq, int Hkv, int D, int splits) {
  return static_cast<long long>(B) * Hq * splits * (D + 2) * 4 + static_cast<long long>(B) * Hkv * 4;
}

extern "C" TYR_EXPORT int tyr_decode_attention_gated(const void* q, const void* k_new, const void* v_new, void* k_cache,
                                                     void* v_cache, const void* pos, void* out, void* workspace, long long q_bs,
                                                     long long kn_bs, long long vn_bs, int B, int Hq, int Hkv, int D, int cap,
                                                     int ring, int window, int splits, int append, float scale, const void* gate,
                                                     long long gate_bs, long long gate_hs, int gate_mode, void* err, void* stream);

// `workspace` must be zero-filled once after allocation (the kernel leaves the counters at zero).
extern "C" TYR_EXPORT int tyr_decode_attention(const void* q, const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                                               const void* pos, void* out, void* workspace, long long q_bs, long long kn_bs,
                                               long long vn_bs, int B, int Hq, int Hkv, int D, int cap, int ring, int window,
                                               int splits, int append, float scale, void* err, void* stream) {
  return tyr_decode_attention_gated(q, k_new, v_new, k_cache, v_cache, pos, out, workspace, q_bs, kn_bs, vn_bs, B, Hq, Hkv, D, cap,
                                    ring, window, splits, append, scale, nullptr, 0, 0, 0, err, stream);
}

// The same with an output gate folded into the final write (see DecodeAttnArgs::gate).
extern "C" TYR_EXPORT int tyr_decode_attention_gated(const void* q, const void* k_new, const void* v_new, void* k_cache,
                                                     void* v_cache, const void* pos, void* out, void* workspace, long long q_bs,
                                                     long long kn_bs, long long vn_bs, int B, int Hq, int Hkv, int D, int cap,
                                                     int ring, int window, int splits, int append, float scale, const void* gate,
                                                     long long gate_bs, long long gate_hs, int gate_mode, void* err, void* stream) {
  using namespace tyr;
  if (gate_mode < 0 || gate_mode > 2 || (gate_mode != 0 && gate == nullptr)) return -5;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || Hq / Hkv > 16 || cap <= 0 || splits < 1 || splits > 64) return -1;
  if (D != 64 && D != 128 && D != 256) return -2;
  const bool wide = Hq / Hkv > 8;
  if (wide && D == 256) return -4;                                  // 16 heads x 256 channels of accumulators do not fit a warp
  if ((q_bs | kn_bs | vn_bs) & 7) return -3;                       // 16-byte rows
  DecodeAttnArgs a;
  a.q = (const __nv_bfloat16*)q; a.k_new = (const __nv_bfloat16*)k_new; a.v_new = (const __nv_bfloat16*)v_new;
  a.k_cache = (__nv_bfloat16*)k_cache; a.v_cache = (__nv_bfloat16*)v_cache;
  a.pos = (const int*)pos; a.out = (__nv_bfloat16*)out;
  a.part_acc = (float*)workspace;
  a.part_ml = a.part_acc + static_cast<long long>(B) * Hq * splits * D;
  a.counters = (int*)(a.part_ml + static_cast<long long>(B) * Hq * splits * 2);
  a.q_bs = q_bs; a.kn_bs = kn_bs; a.vn_bs = vn_bs;
  a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.cap = cap; a.ring = ring; a.window = window; a.splits = splits; a.append = append;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.err = (int*)err;
  a.gate = (const __nv_bfloat16*)gate; a.gate_bs = gate_bs; a.gate_hs = gate_hs; a.gate_mode = gate == nullptr ? 0 : gate_mode;
  const dim3 grid(splits, Hkv, B);
  const cudaStream_t st = (cudaStream_t)stream;
  const dim3 block(kDecWarps * 32);
  if (D == 64 && !wide) return (int)launch_dependent(decode_attention_kernel<64, false>, grid, block, 0, st, a);
  if (D == 64) return (int)launch_dependent(decode_attention_kernel<64, true>, grid, block, 0, st, a);
  if (D == 128 && !wide) return (int)launch_dependent(decode_attention_kernel<128, false>, grid, block, 0, st, a);
  if (D == 128) return (int)launch_dependent(decode_attention_kernel<128, true>, grid, block, 0, st, a);
  return (int)launch_dependent(decode_attention_kernel<256, false>, grid, block, 0, st, a);
}
