// NVFP4 mixture-of-experts kernels.
//
// Weight format (the reference's, Tyr/Model/Laguna/NvFp4.lean:44-72): e2m1 values packed two per
// byte (low nibble = even element), one e4m3 scale per 16 elements, one fp32 global scale per
// expert;  w = e2m1(nibble) * (e4m3(scale) / global).
//
//  * nvfp4_quantize / nvfp4_dequant: bf16 <-> packed banks (dequant is exact: fp32 product rounded
//    once to bf16, like the reference's LUT + embedding graph).
//  * moe_route: softcap -> sigmoid | softmax -> selection bias -> top-k -> renormalise -> scale, plus
//    per-expert counts; moe_layout: offsets + expert-major pair order.  No host synchronisation
//    (the reference's sm_12x path reads a row count back to the host,
//    cc/src/tyr_laguna_moe.cu:1054-1068; its SIMT path builds the layout with a <<<1,1>>> kernel).
//  * moe_fp4_stage_a / stage_b: weight-streaming grouped GEMV for decode-sized batches.  A CTA owns
//    (expert, row tile) and walks that expert's (token, slot) pairs eight at a time, so every
//    packed weight row is read once per eight pairs and decoded in registers; the reference's
//    stage_a/stage_b (:175-335) read the row once per pair.
//  * Prefill-sized batches dequantise the banks of the experts in use into a bf16 scratch and run
//    the grouped tcgen05 GEMM (gemm_tcgen05.cu, group offsets) with the SwiGLU in its epilogue.
#include "common.cuh"
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include <cuda_fp16.h>

namespace tyr {

__constant__ float kE2M1[16] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f,
                                -0.f, -0.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
__device__ __forceinline__ uint8_t float_to_e4m3(float v) {
  return __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}
// round-to-nearest-even onto the e2m1 grid {0, .5, 1, 1.5, 2, 3, 4, 6} (saturating)
__device__ __forceinline__ uint8_t float_to_e2m1(float v) {
  const float a = fabsf(v);
  uint8_t m;
  if (a <= 0.25f) m = 0;
  else if (a < 0.75f) m = 1;
  else if (a <= 1.25f) m = 2;
  else if (a < 1.75f) m = 3;
  else if (a <= 2.5f) m = 4;
  else if (a < 3.5f) m = 5;
  else if (a <= 5.0f) m = 6;
  else m = 7;
  return m | (v < 0.f ? 8 : 0);
}

// ---------------------------------------------------------------------------------------------
// quantise: one thread per 16-element block
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
nvfp4_quantize_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ packed,
                      uint8_t* __restrict__ scales, const float* __restrict__ global_scale,
                      long long blocks_per_mat, long long total_blocks) {
  for (long long b = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; b < total_blocks;
       b += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float G = global_scale[b / blocks_per_mat];
    const __nv_bfloat16* src = x + b * 16;
    float v[16];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint4 u = *reinterpret_cast<const uint4*>(src + i * 8);
      float2 p0 = unpack_bf16x2(u.x), p1 = unpack_bf16x2(u.y), p2 = unpack_bf16x2(u.z), p3 = unpack_bf16x2(u.w);
      v[i * 8 + 0] = p0.x; v[i * 8 + 1] = p0.y; v[i * 8 + 2] = p1.x; v[i * 8 + 3] = p1.y;
      v[i * 8 + 4] = p2.x; v[i * 8 + 5] = p2.y; v[i * 8 + 6] = p3.x; v[i * 8 + 7] = p3.y;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const uint8_t sb = float_to_e4m3(amax / 6.f * G);
    const float s = e4m3_to_float(sb);
    scales[b] = sb;
    const float inv = s > 0.f ? G / s : 0.f;
    uint8_t out[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      out[i] = float_to_e2m1(v[2 * i] * inv) | (float_to_e2m1(v[2 * i + 1] * inv) << 4);
    *reinterpret_cast<uint2*>(packed + b * 8) = *reinterpret_cast<uint2*>(out);
  }
}

// dequantise: one thread per 16-element block; `expert_map` (nullable) selects source experts
__global__ void __launch_bounds__(256)
nvfp4_dequant_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                     const float* __restrict__ global_scale, __nv_bfloat16* __restrict__ out,
                     long long blocks_per_mat, long long total_blocks) {
  for (long long b = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; b < total_blocks;
       b += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float sd = e4m3_to_float(scales[b]) / global_scale[b / blocks_per_mat];
    uint2 raw = *reinterpret_cast<const uint2*>(packed + b * 8);
    const uint8_t* by = reinterpret_cast<const uint8_t*>(&raw);
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = pack_bf16x2(sd * kE2M1[by[i] & 15], sd * kE2M1[by[i] >> 4]);
    uint4* dst = reinterpret_cast<uint4*>(out + b * 16);
    dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
    dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

// ---------------------------------------------------------------------------------------------
// routing: one warp per token, E <= 512
// ---------------------------------------------------------------------------------------------
struct RouteArgs {
  const float* logits;   // [T, E]
  const float* bias;     // [E] selection bias (nullable)
  int* ids;              // [T, k]
  float* weights;        // [T, k]
  int* counts;           // [E] (zero on entry)
  int T, E, k;
  int softmax;           // 0 = sigmoid scores, 1 = softmax scores
  int renorm;
  float softcap, scale;
};

// One warp routes one token from its row of logits.  The row may have been written by other CTAs of the same launch, so it is
// read with L2-coherent loads.
// kMaxPer experts per lane (E <= 32 * kMaxPer): the loops below are unrolled over it, so a 64-expert router instantiated
// with 2 does an eighth of the work of the 512-expert form (the routing of a decode step ran 23 us per layer with 16).
template <int kMaxPer>
__device__ __forceinline__ void route_token_n(const RouteArgs& a, const float* row, int tok, int lane) {
  float score[kMaxPer], sel[kMaxPer];
  const int per = (a.E + 31) / 32;
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kMaxPer; ++j) {
    const int e = lane + 32 * j;
    float l = (j < per && e < a.E) ? __ldcg(row + e) : -INFINITY;
    if (a.softcap > 0.f && l != -INFINITY) l = a.softcap * tanhf(l / a.softcap);
    score[j] = l;
    mx = fmaxf(mx, l);
  }
  if (a.softmax) {
    mx = warp_max(mx);
    float sum = 0.f;
    for (int j = 0; j < kMaxPer; ++j) {
      score[j] = score[j] == -INFINITY ? 0.f : __expf(score[j] - mx);
      sum += score[j];
    }
    sum = warp_sum(sum);
    for (int j = 0; j < kMaxPer; ++j) score[j] /= sum;
  } else {
    for (int j = 0; j < kMaxPer; ++j) score[j] = score[j] == -INFINITY ? 0.f : 1.f / (1.f + __expf(-score[j]));
  }
  for (int j = 0; j < kMaxPer; ++j) {
    const int e = lane + 32 * j;
    sel[j] = (j < per && e < a.E) ? score[j] + (a.bias ? a.bias[e] : 0.f) : -INFINITY;
  }
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int s = 0; s < a.k; ++s) {
    // warp argmax (ties -> lowest expert index, like a stable top-k)
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int j = 0; j < kMaxPer; ++j) {
      const int e = lane + 32 * j;
      if (sel[j] > best || (sel[j] == best && e < best_e)) { best = sel[j]; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    // owner lane fetches the unbiased score and retires the entry
    float sc = 0.f;
    if ((best_e & 31) == lane) {
      const int j = best_e >> 5;
      for (int q = 0; q < kMaxPer; ++q)
        if (q == j) { sc = score[q]; sel[q] = -INFINITY; }
    }
    sc = __shfl_sync(0xffffffffu, sc, best_e & 31);
    wsum += sc;
    if (lane == s) { my_w = sc; my_id = best_e; }
  }
  if (lane < a.k) {
    const float w = (a.renorm ? my_w / wsum : my_w) * a.scale;
    a.ids[static_cast<long long>(tok) * a.k + lane] = my_id;
    a.weights[static_cast<long long>(tok) * a.k + lane] = w;
    if (a.counts) atomicAdd(a.counts + my_id, 1);
  }
}

__device__ __forceinline__ void route_token(const RouteArgs& a, const float* row, int tok, int lane) {
  if (a.E <= 32) route_token_n<1>(a, row, tok, lane);
  else if (a.E <= 64) route_token_n<2>(a, row, tok, lane);
  else if (a.E <= 128) route_token_n<4>(a, row, tok, lane);
  else if (a.E <= 256) route_token_n<8>(a, row, tok, lane);
  else route_token_n<16>(a, row, tok, lane);       // E <= 512
}

__global__ void __launch_bounds__(256) moe_route_kernel(RouteArgs a) {
  const int lane = threadIdx.x & 31;
  const int tok = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (tok >= a.T) return;
  route_token(a, a.logits + static_cast<long long>(tok) * a.E, tok, lane);
}

// Decode-sized batches: router logits and routing in one launch.  CTA (token group, expert group) takes kRouteTok tokens and
// kRouteExp experts; two warps share an expert, each streaming half of its fp32 weight row and dotting it with the group's
// bf16 activation rows staged in shared memory (fp32 accumulation).  Logits go to a small global scratch; the last CTA of
// a token group to finish (atomic ticket) routes the group's tokens, one warp per token.  `tickets` holds one zeroed counter
// per token group.  Small groups on purpose: the kernel is a chain of dependent loads and FMAs per warp, so its duration is
// the instruction count of ONE warp; with 8 tokens x one whole row per warp it ran 20 - 24 us whatever the shape.
constexpr int kRouteTok = 4;
constexpr int kRouteExp = 4;

__global__ void __launch_bounds__(256) moe_route_fused_kernel(RouteArgs a, const __nv_bfloat16* __restrict__ x,
                                                              const float* __restrict__ wr, float* __restrict__ logits,
                                                              int* __restrict__ tickets, int h) {
  extern __shared__ __align__(16) uint8_t route_smem[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(route_smem);     // [kRouteTok][h]
  __shared__ int s_last;
  __shared__ float s_part[kRouteExp][kRouteTok];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tok0 = blockIdx.x * kRouteTok;
  const int nt = min(kRouteTok, a.T - tok0);
  pdl_entry();
#pragma unroll 4
  for (int i = threadIdx.x * 8; i < nt * h; i += blockDim.x * 8)
    *reinterpret_cast<uint4*>(xs + i) = *reinterpret_cast<const uint4*>(x + static_cast<long long>(tok0) * h + i);
  __syncthreads();
  const int el = warp >> 1, half = warp & 1;          // expert of this warp inside the CTA's group, half of the row
  const int e = blockIdx.y * kRouteExp + el;
  float acc[kRouteTok];
#pragma unroll
  for (int t = 0; t < kRouteTok; ++t) acc[t] = 0.f;
  if (e < a.E) {
    const float4* w4 = reinterpret_cast<const float4*>(wr + static_cast<long long>(e) * h);
    const int q4 = h >> 2;                            // float4 groups per row; this warp takes [half * q4 / 2, ...)
    const int lo = half * (q4 >> 1), hi = half ? q4 : (q4 >> 1);
#pragma unroll 4
    for (int i = lo + lane; i < hi; i += 32) {        // four weight loads in flight per lane
      const float4 w = __ldg(w4 + i);
#pragma unroll
      for (int t = 0; t < kRouteTok; ++t) {
        if (t < nt) {
          const uint2 u = *reinterpret_cast<const uint2*>(xs + t * h + 4 * i);
          const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y);
          acc[t] += w.x * f0.x + w.y * f0.y + w.z * f1.x + w.w * f1.y;
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < kRouteTok; ++t) acc[t] = warp_sum(acc[t]);
  if (half == 1 && lane == 0) {
#pragma unroll
    for (int t = 0; t < kRouteTok; ++t) s_part[el][t] = acc[t];
  }
  __syncthreads();
  if (half == 0 && lane == 0 && e < a.E) {
#pragma unroll
    for (int t = 0; t < kRouteTok; ++t)
      if (t < nt) logits[static_cast<long long>(tok0 + t) * a.E + e] = acc[t] + s_part[el][t];
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(tickets + blockIdx.x, 1) == static_cast<int>(gridDim.y) - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (warp < nt) route_token(a, logits + static_cast<long long>(tok0 + warp) * a.E, tok0 + warp, lane);
}

// offsets[E+1] from counts[E]; cursors[E] zeroed; tiles[E+1] (nullable) = prefix sum of
// ceil(count / 128), the m-tile table of the grouped GEMM.  One block.
// active[E + 1] (nullable): compact list of the experts with rows, followed by their number in active[E].
__global__ void moe_offsets_kernel(const int* counts, int* offsets, int* cursors, int* tiles, int* active, int E) {
  __shared__ int s[1024];
  __shared__ int s2[1024];
  __shared__ int s3[1024];
  const int t = threadIdx.x;
  const int v = t < E ? counts[t] : 0;
  s[t] = v;
  s2[t] = (v + 127) >> 7;
  s3[t] = v > 0 ? 1 : 0;
  __syncthreads();
  for (int o = 1; o < blockDim.x; o <<= 1) {
    const int add = t >= o ? s[t - o] : 0;
    const int add2 = t >= o ? s2[t - o] : 0;
    const int add3 = t >= o ? s3[t - o] : 0;
    __syncthreads();
    s[t] += add;
    s2[t] += add2;
    s3[t] += add3;
    __syncthreads();
  }
  if (t < E) {
    offsets[t + 1] = s[t];
    if (tiles) tiles[t + 1] = s2[t];
    if (active && v > 0) active[s3[t] - 1] = t;
    cursors[t] = 0;
  }
  if (t == 0) {
    offsets[0] = 0;
    if (tiles) tiles[0] = 0;
  }
  if (active && t == E - 1) active[E] = s3[t];
}

// pair_order[offsets[e] + slot] = pair index (expert-major); slot order within an expert is arbitrary
__global__ void moe_scatter_kernel(const int* ids, const int* offsets, int* cursors, int* pair_order,
                                   int* pair_pos, int pairs, int E) {
  for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < pairs; p += gridDim.x * blockDim.x) {
    const int e = ids[p];
    if (e < 0 || e >= E) {                           // not routed (expert-parallel padding rows carry id E): takes no slot
      (void)TYR_INDEX_OK(e, E + 1, 11);              // checked builds record ids beyond the padding marker
      if (pair_pos) pair_pos[p] = 0;
      continue;
    }
    const int slot = atomicAdd(cursors + e, 1);
    const int pos = offsets[e] + slot;
    pair_order[pos] = p;
    if (pair_pos) pair_pos[p] = pos;
  }
}

// counts[e] += number of pairs routed to expert e; ids outside [0, E) are not counted (counts zero on entry)
__global__ void moe_count_kernel(const int* ids, int* counts, int pairs, int E) {
  for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < pairs; p += gridDim.x * blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < E) atomicAdd(counts + e, 1);
  }
}

// gather rows: dst[pos] = src[pair_order[pos] / k]   (bf16 [pairs, h])
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const __nv_bfloat16* src, const int* pair_order, __nv_bfloat16* dst, int pairs, int k, int h) {
  const int vec = h >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
       i < static_cast<long long>(pairs) * vec; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int pos = static_cast<int>(i / vec), c = static_cast<int>(i % vec);
    const int tok = pair_order[pos] / k;
    if (!TYR_INDEX_OK(pair_order[pos], pairs, 12)) continue;
    reinterpret_cast<uint4*>(dst + static_cast<long long>(pos) * h)[c] =
        reinterpret_cast<const uint4*>(src + static_cast<long long>(tok) * h)[c];
  }
}

// combine: out[tok] = sum over its k slots of w * y[pair_pos[pair]]   (+ optional residual add-in)
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* y, const int* pair_pos, const float* weights, const __nv_bfloat16* add,
                   __nv_bfloat16* out, int T, int k, int h) {
  pdl_entry();
  const int vec = h >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
       i < static_cast<long long>(T) * vec; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int tok = static_cast<int>(i / vec), c = static_cast<int>(i % vec);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < k; ++s) {
      const int pair = tok * k + s;
      const float w = weights[pair];
      const int pp = pair_pos[pair];
      if (pp < 0) continue;                        // a pair that was not routed to an expert of this bank
      uint4 u = reinterpret_cast<const uint4*>(y + static_cast<long long>(pp) * h)[c];
      float2 a0 = unpack_bf16x2(u.x), a1 = unpack_bf16x2(u.y), a2 = unpack_bf16x2(u.z), a3 = unpack_bf16x2(u.w);
      acc[0] += w * a0.x; acc[1] += w * a0.y; acc[2] += w * a1.x; acc[3] += w * a1.y;
      acc[4] += w * a2.x; acc[5] += w * a2.y; acc[6] += w * a3.x; acc[7] += w * a3.y;
    }
    if (add) {
      uint4 u = reinterpret_cast<const uint4*>(add + static_cast<long long>(tok) * h)[c];
      float2 a0 = unpack_bf16x2(u.x), a1 = unpack_bf16x2(u.y), a2 = unpack_bf16x2(u.z), a3 = unpack_bf16x2(u.w);
      acc[0] += a0.x; acc[1] += a0.y; acc[2] += a1.x; acc[3] += a1.y;
      acc[4] += a2.x; acc[5] += a2.y; acc[6] += a3.x; acc[7] += a3.y;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + static_cast<long long>(tok) * h)[c] = o;
  }
}

// ---------------------------------------------------------------------------------------------
// Weight-streaming grouped GEMV (decode-sized batches).
//
// The op is bound by reading each active expert's FP4 rows once.  Up to 8 (token, slot) pairs of
// one expert form the N = 8 side of m16n8k16 tensor-core tiles, so one pass over the weights serves
// all of them (more pairs -> further passes that hit L2).  Every lane streams 16 contiguous bytes
// (32 weights = two scale groups) per row straight from global memory into registers, converts
// e2m1 -> f16 with the hardware cvt, multiplies by the e4m3 group scale (exact in f16: <= 6
// significant bits) and feeds the A fragment; the k order inside a 128-column step is permuted
// identically for A and B, which a dot product does not care about.  Activations are staged once
// per CTA in shared memory as f16 (clamped to the f16 range).  Four warps x 16 rows per CTA keep
// >= 148 CTAs busy even for a single token; each lane has 64-128 B of weights in flight.
// The synchronous mma form is used on purpose: N is 8 and the kernel is bandwidth bound, there
// is no operand reuse that shared-memory staging for tcgen05 could exploit.
// ---------------------------------------------------------------------------------------------
constexpr int kP = 8;            // pairs per pass (mma N)
constexpr int kWarpsA = 8;       // warps per CTA, stage A (eight warps share one staged activation block: 3 CTAs x 8 warps per SM)
constexpr int kWarpsB = 4;       // warps per CTA, stage B

struct StageArgs {
  const __nv_bfloat16* x;      // stage A: [T, h] activations
  const float* hid_g;          // stage B input / stage A output: raw gate sums [pairs, mi] (expert-major positions)
  const float* hid_u;          //                                  raw up sums
  const uint8_t* w0;           // stage A: gate packed; stage B: down packed
  const uint8_t* s0;
  const float* g0;             // global scale of w0's bank
  const uint8_t* w1;           // stage A: up packed
  const uint8_t* s1;
  const float* g1;
  const float* gg;             // stage B: gate / up global scales (to finish silu(g) * u while staging)
  const float* gu;
  const int* offsets;          // [E+1]
  const int* active;           // [E] compact list of experts with at least one pair
  const int* n_active;         // [1]
  const int* pair_order;       // [pairs] pair index at each expert-major position
  const float* pair_weight;    // [pairs] routing weight by pair index (stage B)
  float* out_g;                // stage A outputs (plain store when gridDim.z == 1, atomic otherwise)
  float* out_u;
  float* out;                  // stage B: [T, h] fp32, atomically accumulated
  int k, in_dim, out_dim;      // stage A: in = h, out = mi; stage B: in = mi, out = h
};

// e2m1 -> f16 without a table: with the nibble at bits [15:12] of a half, the sign stays at bit 15
// and the three magnitude bits move to [11:9] (low two exponent bits and the top mantissa bit).
// Read as f16 that is value * 2^-14, subnormal codes included; the group scale is applied as
// (scale * 2^7) in f16 (max 448 * 128 < 65504) and the missing 2^7 goes onto the fp32 accumulator.
// One 32-bit word holds nibbles n0..n7; register j pairs (n_j, n_{j+4}).
__device__ __forceinline__ void decode_word(uint32_t w, uint32_t scale2, uint32_t (&r)[4]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t tj = j == 3 ? w : (w << (12 - 4 * j));
    const uint32_t v = (tj & 0x80008000u) | ((tj >> 3) & 0x0E000E00u);
    __half2 h = __hmul2(*reinterpret_cast<const __half2*>(&v), *reinterpret_cast<const __half2*>(&scale2));
    r[j] = *reinterpret_cast<uint32_t*>(&h);
  }
}
__device__ __forceinline__ uint32_t e4m3_x128_to_f16x2(uint32_t byte) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3);
  __half v = __hmul(*reinterpret_cast<__half*>(&h), __float2half(128.f));
  return static_cast<uint32_t>(*reinterpret_cast<unsigned short*>(&v)) * 0x00010001u;
}
constexpr float kDecodeRebias = 128.f;     // 2^14 / 2^7 left to apply after the contraction

__device__ __forceinline__ void mma_f16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned short f16_sat(float a) {
  a = fminf(fmaxf(a, -65504.f), 65504.f);
  __half h = __float2half_rn(a);
  return *reinterpret_cast<unsigned short*>(&h);
}

// One 128-column step of one 16-row tile: rows (g, g+8) of one matrix.
//   wlo / whi: the lane's 16 bytes of row g / row g+8;  slo / shi: its two scale bytes per row.
// Word i of the 16 bytes feeds k-steps 2i and 2i+1; k-step s takes registers 2(s&1), 2(s&1)+1, i.e.
// elements {8i+j, 8i+j+4} and {8i+j+1, 8i+j+5} with j = 2(s&1); the activations are staged in the
// same order (position of element e inside its 8: ((e & 3) << 1) | (e >> 2)).
__device__ __forceinline__ void tile_step(float (&c)[4], const uint4& wlo, const uint4& whi, uint32_t slo, uint32_t shi,
                                          const uint32_t (&b)[16]) {
  const uint32_t lo[4] = {wlo.x, wlo.y, wlo.z, wlo.w};
  const uint32_t hi[4] = {whi.x, whi.y, whi.z, whi.w};
  const uint32_t sl[2] = {e4m3_x128_to_f16x2(slo & 0xff), e4m3_x128_to_f16x2(slo >> 8)};
  const uint32_t sh[2] = {e4m3_x128_to_f16x2(shi & 0xff), e4m3_x128_to_f16x2(shi >> 8)};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t rl[4], rh[4];
    decode_word(lo[i], sl[i >> 1], rl);
    decode_word(hi[i], sh[i >> 1], rh);
    mma_f16_16816(c, rl[0], rh[0], rl[1], rh[1], b[4 * i], b[4 * i + 1]);
    mma_f16_16816(c, rl[2], rh[2], rl[3], rh[3], b[4 * i + 2], b[4 * i + 3]);
  }
}

template <bool STAGE_A>
__global__ void __launch_bounds__(32 * (STAGE_A ? kWarpsA : kWarpsB), STAGE_A ? 3 : 8) moe_fp4_gemv_kernel(StageArgs a) {
  constexpr int kRowsCta = 16 * (STAGE_A ? kWarpsA : kWarpsB);
  extern __shared__ __align__(16) uint8_t smem_raw[];
  if (static_cast<int>(blockIdx.y) >= *a.n_active) return;
  const int e = a.active[blockIdx.y];
  const int begin = a.offsets[e], end = a.offsets[e + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int K = a.in_dim;
  // this CTA's slice of the contraction: steps [st0, st1) of 128 columns each
  const int steps = K >> 7;
  const int st0 = steps * blockIdx.z / gridDim.z, st1 = steps * (blockIdx.z + 1) / gridDim.z;
  const int kc0 = st0 << 7, kcols = (st1 - st0) << 7;
  const int xstride = kcols + 8;                              // halves; +16 B staggers rows across banks
  unsigned short* xs = reinterpret_cast<unsigned short*>(smem_raw);   // [kP][xstride] f16 bits
  const int row0 = blockIdx.x * kRowsCta + warp * 16;
  const bool rows_ok = row0 < a.out_dim;                      // out_dim is a multiple of 16
  const long long rbytes = K >> 1, sbytes = K >> 4;
  const long long r_lo = static_cast<long long>(e) * a.out_dim + row0 + g;
  const uint8_t* w0lo = a.w0 + r_lo * rbytes + t * 16 + (kc0 >> 1);
  const uint8_t* w0hi = w0lo + 8 * rbytes;
  const uint8_t* s0lo = a.s0 + r_lo * sbytes + t * 2 + (kc0 >> 4);
  const uint8_t* s0hi = s0lo + 8 * sbytes;
  const uint8_t* w1lo = STAGE_A ? a.w1 + r_lo * rbytes + t * 16 + (kc0 >> 1) : nullptr;
  const uint8_t* w1hi = STAGE_A ? w1lo + 8 * rbytes : nullptr;
  const uint8_t* s1lo = STAGE_A ? a.s1 + r_lo * sbytes + t * 2 + (kc0 >> 4) : nullptr;
  const uint8_t* s1hi = STAGE_A ? s1lo + 8 * sbytes : nullptr;
  float ig = 0.f, iu = 0.f;
  if (!STAGE_A) { ig = 1.f / a.gg[e]; iu = 1.f / a.gu[e]; }

  for (int base = begin; base < end; base += kP) {
    const int np = min(kP, end - base);
    __syncthreads();
    // stage this pass's activations as f16 in the k order of the decoded fragments, 8 at a time
    for (int i = threadIdx.x; i < np * (kcols >> 3); i += blockDim.x) {
      const int p = i / (kcols >> 3), c = (i % (kcols >> 3)) << 3;
      float v[8];
      if (STAGE_A) {
        const int tok = a.pair_order[base + p] / a.k;
        const uint4 u = *reinterpret_cast<const uint4*>(a.x + static_cast<long long>(tok) * K + kc0 + c);
        const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
        v[0] = f0.x; v[1] = f0.y; v[2] = f1.x; v[3] = f1.y; v[4] = f2.x; v[5] = f2.y; v[6] = f3.x; v[7] = f3.y;
      } else {
        const long long o = static_cast<long long>(base + p) * K + kc0 + c;
        const float4 g0 = *reinterpret_cast<const float4*>(a.hid_g + o), g1 = *reinterpret_cast<const float4*>(a.hid_g + o + 4);
        const float4 u0 = *reinterpret_cast<const float4*>(a.hid_u + o), u1 = *reinterpret_cast<const float4*>(a.hid_u + o + 4);
        const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const float uv[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float gs = gv[j] * ig;
          v[j] = gs / (1.f + __expf(-gs)) * (uv[j] * iu);
        }
      }
      // element e goes to position ((e & 3) << 1) | (e >> 2): order 0,4,1,5,2,6,3,7
      uint4 o4;
      o4.x = f16_sat(v[0]) | (static_cast<uint32_t>(f16_sat(v[4])) << 16);
      o4.y = f16_sat(v[1]) | (static_cast<uint32_t>(f16_sat(v[5])) << 16);
      o4.z = f16_sat(v[2]) | (static_cast<uint32_t>(f16_sat(v[6])) << 16);
      o4.w = f16_sat(v[3]) | (static_cast<uint32_t>(f16_sat(v[7])) << 16);
      *reinterpret_cast<uint4*>(xs + p * xstride + c) = o4;
    }
    __syncthreads();
    if (!rows_ok) continue;
    float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
    const unsigned short* xrow = xs + g * xstride + t * 32;
    const int nst = st1 - st0;
#pragma unroll 4
    for (int st = 0; st < nst; ++st) {
      const uint4 a_lo = __ldg(reinterpret_cast<const uint4*>(w0lo + st * 64));
      const uint4 a_hi = __ldg(reinterpret_cast<const uint4*>(w0hi + st * 64));
      const uint32_t sa_lo = __ldg(reinterpret_cast<const uint16_t*>(s0lo + st * 8));
      const uint32_t sa_hi = __ldg(reinterpret_cast<const uint16_t*>(s0hi + st * 8));
      uint4 b_lo, b_hi;
      uint32_t sb_lo = 0, sb_hi = 0;
      if (STAGE_A) {
        b_lo = __ldg(reinterpret_cast<const uint4*>(w1lo + st * 64));
        b_hi = __ldg(reinterpret_cast<const uint4*>(w1hi + st * 64));
        sb_lo = __ldg(reinterpret_cast<const uint16_t*>(s1lo + st * 8));
        sb_hi = __ldg(reinterpret_cast<const uint16_t*>(s1hi + st * 8));
      }
      uint32_t b[16];
      if (g < np) {
        const uint4* xp = reinterpret_cast<const uint4*>(xrow + st * 128);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 v = xp[j];
          b[4 * j] = v.x; b[4 * j + 1] = v.y; b[4 * j + 2] = v.z; b[4 * j + 3] = v.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) b[j] = 0u;
      }
      tile_step(c0, a_lo, a_hi, sa_lo, sa_hi, b);
      if (STAGE_A) tile_step(c1, b_lo, b_hi, sb_lo, sb_hi, b);
    }
    // c[0], c[1]: (row g, pairs 2t, 2t+1);  c[2], c[3]: (row g+8, pairs 2t, 2t+1)
    if (STAGE_A) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int n = 2 * t + (q & 1), row = row0 + g + (q >> 1) * 8;
        if (n < np) {
          const long long o = static_cast<long long>(base + n) * a.out_dim + row;
          if (gridDim.z == 1) {
            a.out_g[o] = c0[q] * kDecodeRebias;
            a.out_u[o] = c1[q] * kDecodeRebias;
          } else {
            atomicAdd(a.out_g + o, c0[q] * kDecodeRebias);
            atomicAdd(a.out_u + o, c1[q] * kDecodeRebias);
          }
        }
      }
    } else {
      const float id = kDecodeRebias / a.g0[e];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int n = 2 * t + (q & 1), row = row0 + g + (q >> 1) * 8;
        if (n < np) {
          const int pair = a.pair_order[base + n];
          atomicAdd(a.out + static_cast<long long>(pair / a.k) * a.out_dim + row, a.pair_weight[pair] * c0[q] * id);
        }
      }
    }
  }
}

// routed fp32 -> bf16 with optional add-in:  out = bf16(routed + add)
__global__ void __launch_bounds__(256)
moe_finalize_kernel(const float* routed, const __nv_bfloat16* add, __nv_bfloat16* out, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float v = routed[i];
    if (add) v += __bfloat162float(add[i]);
    out[i] = __float2bfloat16(v);
  }
}

static int blocks_for(long long items, int cap = 148 * 8) {
  long long b = (items + 255) / 256;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace tyr

using namespace tyr;

extern "C" TYR_EXPORT int tyr_nvfp4_quantize(const void* x, void* packed, void* scales, const float* global_scale,
                                             long long mats, long long elems_per_mat, void* stream) {
  if (mats <= 0 || elems_per_mat <= 0 || (elems_per_mat & 15)) return -1;
  const long long bpm = elems_per_mat / 16;
  nvfp4_quantize_kernel<<<blocks_for(mats * bpm), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (uint8_t*)packed, (uint8_t*)scales, global_scale, bpm, mats * bpm);
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_nvfp4_dequant(const void* packed, const void* scales, const float* global_scale,
                                            void* out, long long mats, long long elems_per_mat, void* stream) {
  if (mats <= 0 || elems_per_mat <= 0 || (elems_per_mat & 15)) return -1;
  const long long bpm = elems_per_mat / 16;
  nvfp4_dequant_kernel<<<blocks_for(mats * bpm), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)packed, (const uint8_t*)scales, global_scale, (__nv_bfloat16*)out, bpm, mats * bpm);
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_moe_route(const float* logits, const float* bias, int* ids, float* weights, int* counts,
                                        int T, int E, int k, int softmax, int renorm, float softcap, float scale,
                                        void* stream) {
  if (T <= 0 || E <= 0 || E > 512 || k <= 0 || k > 32 || k > E) return -1;
  RouteArgs a{logits, bias, ids, weights, counts, T, E, k, softmax, renorm, softcap, scale};
  moe_route_kernel<<<(T + 7) / 8, 256, 0, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

// Router GEMV + routing in one launch: x bf16 [T, h] (h a multiple of 8), router weight fp32 [E, h], `logits` a scratch of
// T * E floats, `tickets` ceil(T / 4) zeroed ints.
extern "C" TYR_EXPORT int tyr_moe_route_fused(const void* x, const float* router_w, const float* bias, float* logits,
                                              int* tickets, int* ids, float* weights, int* counts, int T, int E, int k,
                                              int h, int softmax, int renorm, float softcap, float scale, void* stream) {
  if (T <= 0 || E <= 0 || E > 512 || k <= 0 || k > 32 || k > E || h <= 0 || (h & 7)) return -1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(router_w)) & 15) return -2;
  const size_t smem = sizeof(__nv_bfloat16) * static_cast<size_t>(h) * kRouteTok;
  if (smem > 160 * 1024) return -3;
  static size_t configured = 0;
  if (smem + 1024 > 48 * 1024 && configured < smem) {       // the kernel also holds a few bytes of static shared memory
    cudaFuncSetAttribute(moe_route_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    configured = smem;
  }
  RouteArgs a{nullptr, bias, ids, weights, counts, T, E, k, softmax, renorm, softcap, scale};
  dim3 grid((T + kRouteTok - 1) / kRouteTok, (E + kRouteExp - 1) / kRouteExp);
  return (int)launch_dependent(moe_route_fused_kernel, grid, dim3(256), smem, (cudaStream_t)stream, a, (const __nv_bfloat16*)x,
                               router_w, logits, tickets, h);
}

extern "C" TYR_EXPORT int tyr_moe_layout(const int* ids, const int* counts, int* offsets, int* cursors,
                                         int* tiles, int* active, int* pair_order, int* pair_pos, int pairs,
                                         int E, void* stream) {
  if (pairs <= 0 || E <= 0 || E > 1024) return -1;
  int threads = 32;
  while (threads < E) threads <<= 1;
  moe_offsets_kernel<<<1, threads, 0, (cudaStream_t)stream>>>(counts, offsets, cursors, tiles, active, E);
  moe_scatter_kernel<<<blocks_for(pairs), 256, 0, (cudaStream_t)stream>>>(ids, offsets, cursors, pair_order,
                                                                         pair_pos, pairs, E);
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_moe_count(const int* ids, int* counts, int pairs, int E, void* stream) {
  if (pairs <= 0 || E <= 0) return -1;
  moe_count_kernel<<<blocks_for(pairs), 256, 0, (cudaStream_t)stream>>>(ids, counts, pairs, E);
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_moe_gather_rows(const void* src, const int* pair_order, void* dst, int pairs, int k,
                                              int h, void* stream) {
  if (pairs <= 0 || (h & 7)) return -1;
  moe_gather_rows_kernel<<<blocks_for(1LL * pairs * (h / 8)), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)src, pair_order, (__nv_bfloat16*)dst, pairs, k, h);
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_moe_combine(const void* y, const int* pair_pos, const float* weights, const void* add,
                                          void* out, int T, int k, int h, void* stream) {
  if (T <= 0 || (h & 7)) return -1;
  return (int)launch_dependent(moe_combine_kernel, dim3(blocks_for(1LL * T * (h / 8))), dim3(256), 0, (cudaStream_t)stream,
                               (const __nv_bfloat16*)y, pair_pos, weights, (const __nv_bfloat16*)add, (__nv_bfloat16*)out, T, k, h);
}

static int pick_split(int ctas, int steps, int sm_count) {
  // split the contraction until about four CTAs per SM exist; the split must divide the step count
  int z = 1;
  while (ctas * z < 4 * sm_count && z < steps) {
    int nz = z + 1;
    while (nz < steps && steps % nz) ++nz;
    z = nz;
  }
  return z;
}

// Decode path: routed[T, h] (fp32, zero on entry) += sum_k w * down(silu(gate x) * up x).
// `active` / `n_active` come from tyr_moe_layout; h and mi must be multiples of 128.
// `hid` holds 2 * pairs * mi floats (raw gate sums, then raw up sums) and must be zero on entry.
extern "C" TYR_EXPORT int tyr_moe_fp4_gemv(const void* x, const void* gate_p, const void* gate_s, const float* gate_g,
                                           const void* up_p, const void* up_s, const float* up_g,
                                           const void* down_p, const void* down_s, const float* down_g,
                                           const int* offsets, const int* active, const int* n_active,
                                           const int* pair_order, const float* pair_weight,
                                           float* hid, float* routed, int pairs, int E, int k, int h, int mi, void* stream) {
  if ((h & 127) || (mi & 127) || E <= 0 || pairs <= 0) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  const int slots = pairs < E ? pairs : E;
  if (slots > 65535) return -1;
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  float* hid_g = hid;
  float* hid_u = hid + static_cast<long long>(pairs) * mi;
  StageArgs a{};
  a.x = (const __nv_bfloat16*)x;
  a.w0 = (const uint8_t*)gate_p; a.s0 = (const uint8_t*)gate_s; a.g0 = gate_g;
  a.w1 = (const uint8_t*)up_p; a.s1 = (const uint8_t*)up_s; a.g1 = up_g;
  a.offsets = offsets; a.active = active; a.n_active = n_active; a.pair_order = pair_order; a.pair_weight = pair_weight;
  a.out_g = hid_g; a.out_u = hid_u; a.k = k; a.in_dim = h; a.out_dim = mi;
  const int rows_a = (mi + 16 * kWarpsA - 1) / (16 * kWarpsA), rows_b = (h + 16 * kWarpsB - 1) / (16 * kWarpsB);
  const int za = pick_split(rows_a * slots, h >> 7, sm_count);
  const int zb = pick_split(rows_b * slots, mi >> 7, sm_count);
  const size_t smem_a = sizeof(unsigned short) * kP * (((h >> 7) + za - 1) / za * 128 + 8);
  const size_t smem_b = sizeof(unsigned short) * kP * (((mi >> 7) + zb - 1) / zb * 128 + 8);
  if (smem_a > 200 * 1024 || smem_b > 200 * 1024) return -3;
  static size_t cfg_a = 0, cfg_b = 0;
  if (smem_a > 48 * 1024 && cfg_a < smem_a) {
    cudaFuncSetAttribute(moe_fp4_gemv_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a);
    cfg_a = smem_a;
  }
  if (smem_b > 48 * 1024 && cfg_b < smem_b) {
    cudaFuncSetAttribute(moe_fp4_gemv_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_b);
    cfg_b = smem_b;
  }
  moe_fp4_gemv_kernel<true><<<dim3(rows_a, slots, za), 32 * kWarpsA, smem_a, st>>>(a);
  StageArgs b{};
  b.hid_g = hid_g; b.hid_u = hid_u; b.gg = gate_g; b.gu = up_g;
  b.w0 = (const uint8_t*)down_p; b.s0 = (const uint8_t*)down_s; b.g0 = down_g;
  b.offsets = offsets; b.active = active; b.n_active = n_active; b.pair_order = pair_order; b.pair_weight = pair_weight;
  b.out = routed; b.k = k; b.in_dim = mi; b.out_dim = h;
  moe_fp4_gemv_kernel<false><<<dim3(rows_b, slots, zb), 32 * kWarpsB, smem_b, st>>>(b);
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_moe_finalize(const float* routed, const void* add, void* out, long long n, void* stream) {
  moe_finalize_kernel<<<blocks_for(n), 256, 0, (cudaStream_t)stream>>>(routed, (const __nv_bfloat16*)add,
                                                                       (__nv_bfloat16*)out, n);
  return (int)cudaGetLastError();
}

TYR_DEFINE_BOUNDS_STATUS(moe)
