// Decode-step attention with the KV append fused in and the sequence position read from device memory, so that a
// whole decode step can be replayed from a CUDA graph.
//
// One new query row per (batch, head); K/V stores [B, Hkv, cap, D] bf16 (plain or ring).  Grid (splits, Hkv, B): a CTA
// owns the G = Hq / Hkv query heads of one K/V head over one slice of the retained keys (split-KV, 4 warps).  Scores
// are computed lane-per-key (the key row streams through registers 16 B at a time, the queries sit in shared memory
// as fp32 pre-scaled by scale * log2 e), probabilities are then broadcast by shuffle and the value rows are consumed
// lane-per-channel (coalesced).  The key at the new position is taken from k_new / v_new rather than from the store,
// so the append (done by split 0) cannot race with readers.  Split partials {m, l, acc} go to a workspace; the last
// CTA to arrive for a (batch, K/V head) combines them (atomic ticket, counter reset for the next launch).
//
// The reference takes the library SDPA over a sliced cache for this step (cc/include/tyr_attention.h:58-130,
// Tyr/Inference/KVCache.lean:41-215).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace tyr {

constexpr int kDecWarps = 4;
constexpr int kDecGMax = 8;

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
};

template <int D>
__device__ __forceinline__ void load_row_chunk(const __nv_bfloat16* row, int lane, float (&v)[D / 32]) {
  if constexpr (D == 64) {
    const float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(row + lane * 2));
    v[0] = a.x; v[1] = a.y;
  } else if constexpr (D == 128) {
    const uint2 u = *reinterpret_cast<const uint2*>(row + lane * 4);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  } else {
    const uint4 u = *reinterpret_cast<const uint4*>(row + lane * 8);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  }
}

template <int D>
__global__ void __launch_bounds__(kDecWarps * 32) decode_attention_kernel(DecodeAttnArgs a) {
  constexpr int E = D / 32;                      // channels per lane in the value phase
  __shared__ __align__(16) float sq[kDecGMax * D];
  __shared__ float s_m[kDecWarps][kDecGMax], s_l[kDecWarps][kDecGMax];
  __shared__ float s_acc[kDecWarps][kDecGMax][D];
  __shared__ int s_ticket;

  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
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
  chunk = (chunk + 31) & ~31;
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
  for (int i = tid; i < G * D; i += kDecWarps * 32) {
    const int g = i / D, d = i - g * D;
    sq[i] = __bfloat162float(a.q[b * a.q_bs + static_cast<long long>(hkv * G + g) * D + d]) * a.scale_log2;
  }
  __syncthreads();

  float m[kDecGMax], l[kDecGMax], acc[kDecGMax][E];
#pragma unroll
  for (int g = 0; g < kDecGMax; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) acc[g][e] = 0.f;
  }

  for (int base = lo + warp * 32; base < hi; base += kDecWarps * 32) {
    const int slot = base + lane;
    const bool valid = slot < hi;
    float s[kDecGMax];
#pragma unroll
    for (int g = 0; g < kDecGMax; ++g) s[g] = 0.f;
    if (valid) {
      const __nv_bfloat16* krow = (slot == slot_new) ? kn : kc + static_cast<long long>(slot) * D;
#pragma unroll 4
      for (int c = 0; c < D / 8; ++c) {
        const uint4 u = *reinterpret_cast<const uint4*>(krow + c * 8);
        const float2 k0 = unpack_bf16x2(u.x), k1 = unpack_bf16x2(u.y), k2 = unpack_bf16x2(u.z), k3 = unpack_bf16x2(u.w);
#pragma unroll
        for (int g = 0; g < kDecGMax; ++g) {
          if (g < G) {
            const float4 qa = *reinterpret_cast<const float4*>(&sq[g * D + c * 8]);
            const float4 qb = *reinterpret_cast<const float4*>(&sq[g * D + c * 8 + 4]);
            s[g] += qa.x * k0.x + qa.y * k0.y + qa.z * k1.x + qa.w * k1.y + qb.x * k2.x + qb.y * k2.y + qb.z * k3.x + qb.w * k3.y;
          }
        }
      }
    }
    float p[kDecGMax];
#pragma unroll
    for (int g = 0; g < kDecGMax; ++g) {
      p[g] = 0.f;
      if (g < G) {
        const float sv = valid ? s[g] : -INFINITY;
        const float mx = fmaxf(m[g], warp_max(sv));          // finite: the chunk holds at least one key
        const float alpha = exp2f(m[g] - mx);
        p[g] = valid ? exp2f(sv - mx) : 0.f;
        l[g] = l[g] * alpha + p[g];                          // per-lane partial sum, reduced at the end
        m[g] = mx;
#pragma unroll
        for (int e = 0; e < E; ++e) acc[g][e] *= alpha;
      }
    }
    const int n_here = (hi - base) < 32 ? (hi - base) : 32;
#pragma unroll 4
    for (int j = 0; j < n_here; ++j) {
      const int sj = base + j;
      const __nv_bfloat16* vrow = (sj == slot_new) ? vn : vc + static_cast<long long>(sj) * D;
      float v[E];
      load_row_chunk<D>(vrow, lane, v);
#pragma unroll
      for (int g = 0; g < kDecGMax; ++g) {
        if (g < G) {
          const float pj = __shfl_sync(0xffffffffu, p[g], j);
#pragma unroll
          for (int e = 0; e < E; ++e) acc[g][e] += pj * v[e];
        }
      }
    }
  }

  // ---- combine the four warps -------------------------------------------------------------------------------
#pragma unroll
  for (int g = 0; g < kDecGMax; ++g) {
    if (g < G) {
      const float lw = warp_sum(l[g]);
      if (lane == 0) { s_m[warp][g] = m[g]; s_l[warp][g] = lw; }
#pragma unroll
      for (int e = 0; e < E; ++e) s_acc[warp][g][lane * E + e] = acc[g][e];
    }
  }
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
      a.out[row * D + d] = __float2bfloat16(L > 0.f ? A / L : 0.f);
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
    a.out[row * D + d] = __float2bfloat16(L > 0.f ? A / L : 0.f);
  }
  if (tid == 0) a.counters[b * a.Hkv + hkv] = 0;
}

}  // namespace tyr

// Workspace: floats for the split partials followed by the ticket counters.
extern "C" TYR_EXPORT long long tyr_decode_attention_workspace_bytes(int B, int Hq, int Hkv, int D, int splits) {
  return static_cast<long long>(B) * Hq * splits * (D + 2) * 4 + static_cast<long long>(B) * Hkv * 4;
}

// `workspace` must be zero-filled once after allocation (the kernel leaves the counters at zero).
extern "C" TYR_EXPORT int tyr_decode_attention(const void* q, const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                                               const void* pos, void* out, void* workspace, long long q_bs, long long kn_bs,
                                               long long vn_bs, int B, int Hq, int Hkv, int D, int cap, int ring, int window,
                                               int splits, int append, float scale, void* err, void* stream) {
  using namespace tyr;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || Hq / Hkv > kDecGMax || cap <= 0 || splits < 1 || splits > 64) return -1;
  if (D != 64 && D != 128 && D != 256) return -2;
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
  const dim3 grid(splits, Hkv, B);
  if (D == 64) decode_attention_kernel<64><<<grid, kDecWarps * 32, 0, (cudaStream_t)stream>>>(a);
  else if (D == 128) decode_attention_kernel<128><<<grid, kDecWarps * 32, 0, (cudaStream_t)stream>>>(a);
  else decode_attention_kernel<256><<<grid, kDecWarps * 32, 0, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}
