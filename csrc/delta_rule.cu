// Gated delta rule (Qwen3.5 GatedDeltaNet): the single-token recurrent step for decode, and further down the sequential chunk
// pass of the chunked prefill form.
//
// Single-token step.
//
// Per (batch, value head) the state S is [dk, dv] fp32.  One step is
//   S <- exp(g) * S;  kv = S^T k;  delta = beta * (v - kv);  S <- S + k delta^T;  out = S^T q
// with q, k L2-normalised over dk and q scaled by dk^-1/2.  The step is bound by one read and one
// write of S (2 * dk * dv * 4 bytes); the kernel below does exactly that: a thread owns a quarter of one
// state column, keeps those values in registers between the two reductions (finished across the four row
// groups through shared memory), and the CTA's accesses to a state row are contiguous.  Semantics follow cc/src/tyr_qwen35.cpp:121-170 of the reference.
#include "common.cuh"

namespace tyr {

template <int DK>
__global__ void __launch_bounds__(512, 2)      // 64 registers: two CTAs per SM (at 128 registers one CTA kept a quarter of the warps busy)
gdr_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                  const __nv_bfloat16* __restrict__ v, const float* __restrict__ g,
                  const float* __restrict__ beta, float* __restrict__ state, __nv_bfloat16* __restrict__ out,
                  int Hk, int Hv, int dv, long long q_bstride, long long v_bstride,
                  const __nv_bfloat16* __restrict__ z, long long z_bstride, const __nv_bfloat16* __restrict__ norm_w,
                  float norm_eps) {
  // z != nullptr (dv == 128, one column pass): the layer's gated RMSNorm runs in the epilogue,
  //   out = rmsnorm_over_dv(o) * norm_w * silu(z),
  // with o rounded to bf16 first, as the separate kernels see it.
  // 128 state columns per pass.  A warp is one group of DK / 16 state rows; a lane owns four adjacent columns, so a warp's
  // access to a state row is one contiguous 512-byte line of 16-byte vectors.  The two column reductions (S^T k and S^T q) are
  // finished across the sixteen row groups through shared memory.
  constexpr int RPT = DK / 16;
  __shared__ float sq[DK], sk[DK];
  __shared__ float red[2][16];
  __shared__ __align__(16) float part[16][128];
  const int bh = blockIdx.x;
  const int b = bh / Hv, hv = bh % Hv;
  const int hk = hv / (Hv / Hk);
  const int tid = threadIdx.x;
  const int quad = tid & 31, rg = tid >> 5;
  float* S = state + static_cast<long long>(bh) * DK * dv;
  // The state was last written one decode step ago: ask the L2 for it while the kernel in front of this one still runs.
  pdl_trigger();
  if (dv == 128 && tid < 16) bulk_prefetch_l2(S + tid * (DK * 8), DK * 8 * 4);
  pdl_wait();
  const __nv_bfloat16* qp = q + b * q_bstride + static_cast<long long>(hk) * DK;
  const __nv_bfloat16* kp = k + b * q_bstride + static_cast<long long>(hk) * DK;
  float qs = 0.f, ks = 0.f;
  if (tid < DK) {
    const float a = __bfloat162float(qp[tid]), c = __bfloat162float(kp[tid]);
    sq[tid] = a; sk[tid] = c;
    qs = a * a; ks = c * c;
  }
  qs = warp_sum(qs); ks = warp_sum(ks);
  if ((tid & 31) == 0) { red[0][tid >> 5] = qs; red[1][tid >> 5] = ks; }
  __syncthreads();
  qs = 0.f; ks = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) { qs += red[0][i]; ks += red[1][i]; }
  const float qn = rsqrtf(qs + 1e-6f) * rsqrtf(static_cast<float>(DK));
  const float kn = rsqrtf(ks + 1e-6f);
  const float decay = __expf(g[bh]);
  const float bt = beta[bh];
  const int r0 = rg * RPT;
  const bool vec_ok = (dv & 3) == 0;               // 16-byte state accesses need dv to be a multiple of 4
  for (int col0 = blockIdx.y * 128; col0 < dv; col0 += gridDim.y * 128) {
    const int col = col0 + 4 * quad;
    float s[RPT][4];
    float kv[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      float* row = S + static_cast<long long>(r0 + r) * dv + col;
      if (vec_ok && col + 3 < dv) {
        const float4 t = *reinterpret_cast<const float4*>(row);
        s[r][0] = t.x; s[r][1] = t.y; s[r][2] = t.z; s[r][3] = t.w;
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) s[r][c] = col + c < dv ? row[c] : 0.f;
      }
      const float kk = sk[r0 + r];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        s[r][c] *= decay;
        kv[c] += s[r][c] * kk;
      }
    }
    *reinterpret_cast<float4*>(&part[rg][4 * quad]) = make_float4(kv[0], kv[1], kv[2], kv[3]);
    __syncthreads();
#pragma unroll
    for (int c = 0; c < 4; ++c) kv[c] = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float4 t = *reinterpret_cast<const float4*>(&part[i][4 * quad]);
      kv[0] += t.x; kv[1] += t.y; kv[2] += t.z; kv[3] += t.w;
    }
    __syncthreads();
    float delta[4], o[4] = {0.f, 0.f, 0.f, 0.f};
    const __nv_bfloat16* vp = v + b * v_bstride + static_cast<long long>(hv) * dv;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float vt = col + c < dv ? __bfloat162float(vp[col + c]) : 0.f;
      delta[c] = (vt - kv[c] * kn) * bt * kn;       // k enters normalised: k_hat = kn * k
    }
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      const float kk = sk[r0 + r], qq = sq[r0 + r];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        s[r][c] += kk * delta[c];
        o[c] += s[r][c] * qq;
      }
      float* row = S + static_cast<long long>(r0 + r) * dv + col;
      if (vec_ok && col + 3 < dv) {
        *reinterpret_cast<float4*>(row) = make_float4(s[r][0], s[r][1], s[r][2], s[r][3]);
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (col + c < dv) row[c] = s[r][c];
      }
    }
    *reinterpret_cast<float4*>(&part[rg][4 * quad]) = make_float4(o[0], o[1], o[2], o[3]);
    __syncthreads();
    if (rg == 0) {                                   // one warp finishes the 128 outputs of this pass, four per lane
#pragma unroll
      for (int c = 0; c < 4; ++c) o[c] = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float4 t = *reinterpret_cast<const float4*>(&part[i][4 * quad]);
        o[0] += t.x; o[1] += t.y; o[2] += t.z; o[3] += t.w;
      }
      __nv_bfloat16* op = out + static_cast<long long>(bh) * dv;
      if (z == nullptr) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (col + c < dv) op[col + c] = __float2bfloat16(o[c] * qn);
      } else {
        float ssq = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          o[c] = col + c < dv ? __bfloat162float(__float2bfloat16(o[c] * qn)) : 0.f;
          ssq += o[c] * o[c];
        }
        ssq = warp_sum(ssq);
        const float rstd = rsqrtf(ssq / static_cast<float>(dv) + norm_eps);
        const __nv_bfloat16* zp = z + b * z_bstride + static_cast<long long>(hv) * dv;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (col + c >= dv) continue;
          const float zz = __bfloat162float(zp[col + c]);
          const float y = o[c] * rstd * __bfloat162float(norm_w[col + c]);
          op[col + c] = __float2bfloat16(y * (zz / (1.f + __expf(-zz))));
        }
      }
    }
    __syncthreads();
  }
}

// The same step for dv == 128 with the state tile staged in shared memory.  The [DK, 128] fp32 state of one (batch, value
// head) is one contiguous block: a bulk copy brings it into shared memory while the threads normalise q and k, the two
// passes (S^T k, then update + S^T q) run on shared memory, and one bulk copy writes the tile back.  No thread keeps state
// in registers, so three CTAs (192 KB of tiles) fit an SM and their load / compute / store phases overlap.
__device__ __forceinline__ void gdr_bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void gdr_bulk_store(void* dst, const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src)), "r"(bytes)
               : "memory");
}

template <int DK>
__global__ void __launch_bounds__(256)
gdr_decode_tile_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                       const __nv_bfloat16* __restrict__ v, const float* __restrict__ g,
                       const float* __restrict__ beta, float* __restrict__ state, __nv_bfloat16* __restrict__ out,
                       int Hk, int Hv, long long q_bstride, long long v_bstride,
                       const __nv_bfloat16* __restrict__ z, long long z_bstride, const __nv_bfloat16* __restrict__ norm_w,
                       float norm_eps, int* err) {
  constexpr int DV = 128, RG = 8, RPT = DK / RG;
  constexpr uint32_t kBytes = DK * DV * 4, kPiece = kBytes / 4;
  extern __shared__ __align__(128) uint8_t gdr_smem[];
  float* tile = reinterpret_cast<float*>(gdr_smem);                      // [DK][128]
  __shared__ float sq[DK], sk[DK];
  __shared__ float red[2][RG];
  __shared__ __align__(16) float part[RG][DV];
  __shared__ __align__(8) uint64_t bar;
  const int bh = blockIdx.x;
  const int b = bh / Hv, hv = bh % Hv;
  const int hk = hv / (Hv / Hk);
  const int tid = threadIdx.x;
  const int quad = tid & 31, rg = tid >> 5;
  uint8_t* S = reinterpret_cast<uint8_t*>(state + static_cast<long long>(bh) * DK * DV);
  pdl_trigger();
  if (tid == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  if (tid < 4) bulk_prefetch_l2(S + tid * kPiece, kPiece);   // the state was last written a whole decode step ago
  pdl_wait();
  if (tid == 0) {
    mbar_expect_tx(&bar, kBytes);
#pragma unroll
    for (int i = 0; i < 4; ++i) gdr_bulk_load(gdr_smem + i * kPiece, S + i * kPiece, kPiece, &bar);
  }
  const __nv_bfloat16* qp = q + b * q_bstride + static_cast<long long>(hk) * DK;
  const __nv_bfloat16* kp = k + b * q_bstride + static_cast<long long>(hk) * DK;
  float qs = 0.f, ks = 0.f;
  if (tid < DK) {
    const float a = __bfloat162float(qp[tid]), c = __bfloat162float(kp[tid]);
    sq[tid] = a; sk[tid] = c;
    qs = a * a; ks = c * c;
  }
  qs = warp_sum(qs); ks = warp_sum(ks);
  if (quad == 0) { red[0][rg] = qs; red[1][rg] = ks; }
  __syncthreads();                                   // also orders the barrier's init before every thread's wait
  qs = 0.f; ks = 0.f;
#pragma unroll
  for (int i = 0; i < RG; ++i) { qs += red[0][i]; ks += red[1][i]; }
  const float qn = rsqrtf(qs + 1e-6f) * rsqrtf(static_cast<float>(DK));
  const float kn = rsqrtf(ks + 1e-6f);
  const float decay = __expf(g[bh]);
  const float bt = beta[bh];
  const int col = 4 * quad;
  const __nv_bfloat16* vp = v + b * v_bstride + static_cast<long long>(hv) * DV;
  float vt[4];
  {
    const uint2 u = *reinterpret_cast<const uint2*>(vp + col);
    const float2 a = unpack_bf16x2(u.x), c = unpack_bf16x2(u.y);
    vt[0] = a.x; vt[1] = a.y; vt[2] = c.x; vt[3] = c.y;
  }
  if (!mbar_wait(&bar, 0, err, 1600)) {
    mbar_wait(&bar, 0, nullptr, 0);                  // the copy still targets this CTA's shared memory: do not leave before it lands
    return;
  }
  float4* trow = reinterpret_cast<float4*>(tile) + static_cast<long long>(rg * RPT) * (DV / 4) + quad;
  float kv[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int r = 0; r < RPT; ++r) {
    const float4 t = trow[r * (DV / 4)];
    const float kk = sk[rg * RPT + r];
    kv[0] += t.x * kk; kv[1] += t.y * kk; kv[2] += t.z * kk; kv[3] += t.w * kk;
  }
  *reinterpret_cast<float4*>(&part[rg][col]) = make_float4(kv[0], kv[1], kv[2], kv[3]);
  __syncthreads();
#pragma unroll
  for (int c = 0; c < 4; ++c) kv[c] = 0.f;
#pragma unroll
  for (int i = 0; i < RG; ++i) {
    const float4 t = *reinterpret_cast<const float4*>(&part[i][col]);
    kv[0] += t.x; kv[1] += t.y; kv[2] += t.z; kv[3] += t.w;
  }
  __syncthreads();
  float delta[4], o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int c = 0; c < 4; ++c) delta[c] = (vt[c] - kv[c] * decay * kn) * bt * kn;     // k enters normalised: k_hat = kn * k
#pragma unroll
  for (int r = 0; r < RPT; ++r) {
    float4 t = trow[r * (DV / 4)];
    const float kk = sk[rg * RPT + r], qq = sq[rg * RPT + r];
    t.x = t.x * decay + kk * delta[0]; t.y = t.y * decay + kk * delta[1];
    t.z = t.z * decay + kk * delta[2]; t.w = t.w * decay + kk * delta[3];
    o[0] += t.x * qq; o[1] += t.y * qq; o[2] += t.z * qq; o[3] += t.w * qq;
    trow[r * (DV / 4)] = t;
  }
  *reinterpret_cast<float4*>(&part[rg][col]) = make_float4(o[0], o[1], o[2], o[3]);
  fence_proxy_async();                               // the tile's new values must be visible to the bulk copy engine
  __syncthreads();
  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) gdr_bulk_store(S + i * kPiece, gdr_smem + i * kPiece, kPiece);
    tma_store_commit();
  }
  if (rg == 0) {                                     // one warp finishes the 128 outputs, four per lane
#pragma unroll
    for (int c = 0; c < 4; ++c) o[c] = 0.f;
#pragma unroll
    for (int i = 0; i < RG; ++i) {
      const float4 t = *reinterpret_cast<const float4*>(&part[i][col]);
      o[0] += t.x; o[1] += t.y; o[2] += t.z; o[3] += t.w;
    }
    __nv_bfloat16* op = out + static_cast<long long>(bh) * DV + col;
    if (z != nullptr) {
      float ssq = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        o[c] = __bfloat162float(__float2bfloat16(o[c] * qn));
        ssq += o[c] * o[c];
      }
      ssq = warp_sum(ssq);
      const float rstd = rsqrtf(ssq / static_cast<float>(DV) + norm_eps);
      const __nv_bfloat16* zp = z + b * z_bstride + static_cast<long long>(hv) * DV + col;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float zz = __bfloat162float(zp[c]);
        o[c] = o[c] * rstd * __bfloat162float(norm_w[col + c]) * (zz / (1.f + __expf(-zz)));
      }
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c) o[c] *= qn;
    }
    uint2 u;
    u.x = pack_bf16x2(o[0], o[1]);
    u.y = pack_bf16x2(o[2], o[3]);
    *reinterpret_cast<uint2*>(op) = u;
  }
  if (tid == 0) tma_store_wait_read<0>();            // shared memory must outlive the copy engine's reads
}

// Everything in front of the recurrent step for one new token per row: the causal depthwise conv (window of K taps kept as
// the layer's conv state, shifted in place: a channel belongs to exactly one thread) with bias and SiLU, and the per-head
// gates beta = sigmoid(b), g = -softplus(a + dt_bias) * exp(a_log).  `mixed` / `b_in` / `a_in` are rows of projection outputs
// (column windows of one fused projection or separate tensors: row strides ld_m / ld_b / ld_a); outputs: conv_out bf16 [B, cd], g / beta fp32 [B, Hv].
// The reference runs this as about twenty library launches (cc/src/tyr_qwen35.cpp:121-170).
__global__ void __launch_bounds__(256)
gdn_conv_gates_kernel(const __nv_bfloat16* __restrict__ mixed, const __nv_bfloat16* __restrict__ b_in,
                      const __nv_bfloat16* __restrict__ a_in, long long ld_m, long long ld_b, long long ld_a,
                      __nv_bfloat16* __restrict__ conv_state,
                      const __nv_bfloat16* __restrict__ conv_w, const __nv_bfloat16* __restrict__ conv_b,
                      const float* __restrict__ dt_bias, const float* __restrict__ a_log, __nv_bfloat16* __restrict__ conv_out,
                      float* __restrict__ g, float* __restrict__ beta, int B, int cd, int K, int Hv) {
  pdl_entry();
  const long long idx = blockIdx.x * 256LL + threadIdx.x;
  const long long n_conv = static_cast<long long>(B) * cd;
  if (idx < n_conv) {
    const int b = static_cast<int>(idx / cd), c = static_cast<int>(idx - static_cast<long long>(b) * cd);
    __nv_bfloat16* st = conv_state + idx * K;
    const __nv_bfloat16* w = conv_w + static_cast<long long>(c) * K;
    const __nv_bfloat16 x_new = mixed[b * ld_m + c];
    float acc = conv_b ? __bfloat162float(conv_b[c]) : 0.f;
    for (int j = 0; j + 1 < K; ++j) {
      const __nv_bfloat16 t = st[j + 1];
      st[j] = t;
      acc += __bfloat162float(t) * __bfloat162float(w[j]);
    }
    st[K - 1] = x_new;
    acc += __bfloat162float(x_new) * __bfloat162float(w[K - 1]);
    conv_out[idx] = __float2bfloat16(acc / (1.f + __expf(-acc)));
  } else if (idx < n_conv + static_cast<long long>(B) * Hv) {
    const long long j = idx - n_conv;
    const int b = static_cast<int>(j / Hv), h = static_cast<int>(j - static_cast<long long>(b) * Hv);
    const float bv = __bfloat162float(b_in[b * ld_b + h]);
    const float av = __bfloat162float(a_in[b * ld_a + h]) + dt_bias[h];
    const float sp = av > 20.f ? av : log1pf(__expf(av));
    beta[j] = 1.f / (1.f + __expf(-bv));
    g[j] = -sp * __expf(a_log[h]);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Chunked prefill: the sequential pass over the chunks of one (batch, value head).
//
// The chunk-local quantities (u = "value" and w = "k_cumdecay" of the unit-lower-triangular solve, the decayed
// q K^T matrix `intra`, qg = q * exp(gc), kd = k * exp(g_last - gc)) are batched matrix work over all chunks at once and
// come in as fp32.  What is left is a recurrence over the chunks through the [dk, dv] state S,
//     v_new = u_i - w_i S;   out_i = qg_i S + intra_i v_new;   S <- exp(g_last_i) S + kd_i^T v_new,
// which the reference runs as a host loop of five small launches per chunk (cc/src/tyr_qwen35.cpp:89-110).  Here one CTA
// walks all chunks of one (batch, head, 64-column slice of dv): S lives in registers as the accumulator of the last product
// (each of the 4 warps owns 32 of the 128 state rows) and is mirrored into shared memory as the B operand of the first two;
// all five products run on tensor cores in TF32 (mma.sync m16n8k8, fp32 accumulate).  The chunk inputs are staged with
// cp.async in two groups so that the loads of w / qg for the next chunk overlap the last two products of this one.
// ------------------------------------------------------------------------------------------------------------------
constexpr int GC_C = 64;       // chunk length
constexpr int GC_DK = 128;     // key dim
constexpr int GC_DVS = 64;     // dv columns per CTA
constexpr int GC_LDW = GC_DK + 4;    // row-major A operands: 4 g + t hits 32 distinct banks
constexpr int GC_LDT = GC_DK + 8;    // kd is read transposed:  8 t + g
constexpr int GC_LDI = GC_C + 4;
constexpr int GC_LDS = GC_DVS + 8;   // B operands:              8 t + g

struct GdrChunkSmem {
  float w[GC_C * GC_LDW];
  float q[GC_C * GC_LDW];
  float kd[GC_C * GC_LDT];
  float intra[GC_C * GC_LDI];
  float s[GC_DK * GC_LDS];
  float v[GC_C * GC_LDS];
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma_tf32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// rows x cols floats from global (row stride = cols) into shared memory rows of `ld` floats, 16 bytes per copy
__device__ __forceinline__ void stage_tile(float* dst, const float* src, int rows, int cols, int ld) {
  const int per_row = cols >> 2;
  for (int i = threadIdx.x; i < rows * per_row; i += blockDim.x) {
    const int r = i / per_row, c = (i % per_row) << 2;
    cp_async16(dst + r * ld + c, src + static_cast<long long>(r) * cols + c);
  }
}

__global__ void __launch_bounds__(128, 1)
gdr_chunk_scan_kernel(const float* __restrict__ u, const float* __restrict__ w, const float* __restrict__ qg,
                      const float* __restrict__ kd, const float* __restrict__ intra, const float* __restrict__ glast,
                      const float* __restrict__ state_in, float* __restrict__ state_out, __nv_bfloat16* __restrict__ out, int n,
                      int dv, int seq, int Hv) {
  extern __shared__ __align__(16) uint8_t gdr_smem_raw[];
  GdrChunkSmem& sm = *reinterpret_cast<GdrChunkSmem*>(gdr_smem_raw);
  const int bh = blockIdx.y;
  const int col0 = blockIdx.x * GC_DVS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const long long chunk_k = static_cast<long long>(GC_C) * GC_DK;      // floats per chunk of w / qg / kd
  const float* w_p = w + static_cast<long long>(bh) * n * chunk_k;
  const float* q_p = qg + static_cast<long long>(bh) * n * chunk_k;
  const float* kd_p = kd + static_cast<long long>(bh) * n * chunk_k;
  const float* in_p = intra + static_cast<long long>(bh) * n * GC_C * GC_C;
  const float* u_p = u + static_cast<long long>(bh) * n * GC_C * dv + col0;
  // output rows go straight to the [B, S, Hv, dv] bf16 layout of the layer (rows past the sequence end are dropped)
  __nv_bfloat16* o_p = out + (static_cast<long long>(bh / Hv) * seq * Hv + (bh % Hv)) * dv + col0;

  // state rows [32 warp, 32 warp + 32) x 64 columns as two m-tiles x eight n-tiles of accumulators
  float S[2][8][4];
  {
    const float* si = state_in ? state_in + (static_cast<long long>(bh) * GC_DK) * dv + col0 : nullptr;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          const int r = warp * 32 + mt * 16 + g + h2 * 8, c = nt * 8 + 2 * t;
          float2 v = make_float2(0.f, 0.f);
          if (si) v = *reinterpret_cast<const float2*>(si + static_cast<long long>(r) * dv + c);
          S[mt][nt][2 * h2] = v.x;
          S[mt][nt][2 * h2 + 1] = v.y;
          *reinterpret_cast<float2*>(&sm.s[r * GC_LDS + c]) = v;
        }
  }
  stage_tile(sm.w, w_p, GC_C, GC_DK, GC_LDW);
  stage_tile(sm.q, q_p, GC_C, GC_DK, GC_LDW);
  cp_async_commit();

  for (int i = 0; i < n; ++i) {
    stage_tile(sm.kd, kd_p + i * chunk_k, GC_C, GC_DK, GC_LDT);
    stage_tile(sm.intra, in_p + static_cast<long long>(i) * GC_C * GC_C, GC_C, GC_C, GC_LDI);
    cp_async_commit();
    cp_async_wait<1>();            // w_i, qg_i landed (this thread's copies); the barrier publishes everyone's and S
    __syncthreads();
    // ---- X = w_i S, Y = qg_i S : warp rows [16 warp, +16), K = dk
    float X[8][4], Y[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) X[nt][e] = Y[nt][e] = 0.f;
    const int ar = warp * 16 + g;
#pragma unroll 4
    for (int kk = 0; kk < GC_DK / 8; ++kk) {
      const int kc = kk * 8 + t;
      const uint32_t wa0 = __float_as_uint(sm.w[ar * GC_LDW + kc]), wa1 = __float_as_uint(sm.w[(ar + 8) * GC_LDW + kc]);
      const uint32_t wa2 = __float_as_uint(sm.w[ar * GC_LDW + kc + 4]), wa3 = __float_as_uint(sm.w[(ar + 8) * GC_LDW + kc + 4]);
      const uint32_t qa0 = __float_as_uint(sm.q[ar * GC_LDW + kc]), qa1 = __float_as_uint(sm.q[(ar + 8) * GC_LDW + kc]);
      const uint32_t qa2 = __float_as_uint(sm.q[ar * GC_LDW + kc + 4]), qa3 = __float_as_uint(sm.q[(ar + 8) * GC_LDW + kc + 4]);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const uint32_t b0 = __float_as_uint(sm.s[kc * GC_LDS + nt * 8 + g]), b1 = __float_as_uint(sm.s[(kc + 4) * GC_LDS + nt * 8 + g]);
        mma_tf32(X[nt], wa0, wa1, wa2, wa3, b0, b1);
        mma_tf32(Y[nt], qa0, qa1, qa2, qa3, b0, b1);
      }
    }
    // ---- v_new = u_i - X  -> shared memory (B operand of the next two products)
    {
      const float* ui = u_p + static_cast<long long>(i) * GC_C * dv;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          const int r = ar + h2 * 8, c = nt * 8 + 2 * t;
          const float2 uu = *reinterpret_cast<const float2*>(ui + static_cast<long long>(r) * dv + c);
          *reinterpret_cast<float2*>(&sm.v[r * GC_LDS + c]) = make_float2(uu.x - X[nt][2 * h2], uu.y - X[nt][2 * h2 + 1]);
        }
    }
    cp_async_wait<0>();            // kd_i, intra_i
    __syncthreads();               // v_new complete; every warp is done with w, qg and the old S in shared memory
    if (i + 1 < n) {               // next chunk's first group overlaps the two products below
      stage_tile(sm.w, w_p + (i + 1) * chunk_k, GC_C, GC_DK, GC_LDW);
      stage_tile(sm.q, q_p + (i + 1) * chunk_k, GC_C, GC_DK, GC_LDW);
    }
    cp_async_commit();
    // ---- out_i = Y + intra_i v_new : K = chunk
#pragma unroll 2
    for (int kk = 0; kk < GC_C / 8; ++kk) {
      const int kc = kk * 8 + t;
      const uint32_t a0 = __float_as_uint(sm.intra[ar * GC_LDI + kc]), a1 = __float_as_uint(sm.intra[(ar + 8) * GC_LDI + kc]);
      const uint32_t a2 = __float_as_uint(sm.intra[ar * GC_LDI + kc + 4]), a3 = __float_as_uint(sm.intra[(ar + 8) * GC_LDI + kc + 4]);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const uint32_t b0 = __float_as_uint(sm.v[kc * GC_LDS + nt * 8 + g]), b1 = __float_as_uint(sm.v[(kc + 4) * GC_LDS + nt * 8 + g]);
        mma_tf32(Y[nt], a0, a1, a2, a3, b0, b1);
      }
    }
    {
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const int tok = i * GC_C + ar + h2 * 8;
        if (tok < seq) {
          __nv_bfloat16* oi = o_p + static_cast<long long>(tok) * Hv * dv;
#pragma unroll
          for (int nt = 0; nt < 8; ++nt)
            *reinterpret_cast<uint32_t*>(oi + nt * 8 + 2 * t) = pack_bf16x2(Y[nt][2 * h2], Y[nt][2 * h2 + 1]);
        }
      }
    }
    // ---- S <- exp(g_last) S + kd_i^T v_new : this warp's 32 state rows, K = chunk
    const float e = glast[static_cast<long long>(bh) * n + i];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) S[mt][nt][q4] *= e;
#pragma unroll 2
    for (int kk = 0; kk < GC_C / 8; ++kk) {
      const int kc = kk * 8 + t;
      uint32_t a[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const int m = warp * 32 + mt * 16 + g;          // A[m][k] = kd[k][m]
        a[mt][0] = __float_as_uint(sm.kd[kc * GC_LDT + m]);
        a[mt][1] = __float_as_uint(sm.kd[kc * GC_LDT + m + 8]);
        a[mt][2] = __float_as_uint(sm.kd[(kc + 4) * GC_LDT + m]);
        a[mt][3] = __float_as_uint(sm.kd[(kc + 4) * GC_LDT + m + 8]);
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const uint32_t b0 = __float_as_uint(sm.v[kc * GC_LDS + nt * 8 + g]), b1 = __float_as_uint(sm.v[(kc + 4) * GC_LDS + nt * 8 + g]);
        mma_tf32(S[0][nt], a[0][0], a[0][1], a[0][2], a[0][3], b0, b1);
        mma_tf32(S[1][nt], a[1][0], a[1][1], a[1][2], a[1][3], b0, b1);
      }
    }
    // mirror the new state for the next chunk's first products (nobody reads sm.s between the barrier above and the next one)
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2)
          *reinterpret_cast<float2*>(&sm.s[(warp * 32 + mt * 16 + g + h2 * 8) * GC_LDS + nt * 8 + 2 * t]) =
              make_float2(S[mt][nt][2 * h2], S[mt][nt][2 * h2 + 1]);
    __syncthreads();               // kd, intra, v free for the next chunk's copies; S mirror complete
  }
  float* so = state_out + (static_cast<long long>(bh) * GC_DK) * dv + col0;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2)
        *reinterpret_cast<float2*>(so + static_cast<long long>(warp * 32 + mt * 16 + g + h2 * 8) * dv + nt * 8 + 2 * t) =
            make_float2(S[mt][nt][2 * h2], S[mt][nt][2 * h2 + 1]);
}

// ------------------------------------------------------------------------------------------------------------------
// Chunked prefill: everything that is local to one chunk, in one launch per layer.
//
// One CTA per (chunk of 64 tokens, batch, value head), 256 threads:
//   1. q, k rows -> fp32 shared memory, L2-normalised (q also scaled by dk^-1/2); gc = inclusive cumulative sum of g.
//   2. k k^T and q k^T (64 x 64, K = 128) on tensor cores with the 3-term TF32 split (hi*hi + hi*lo + lo*hi, close to fp32:
//      the first matrix feeds a triangular solve), then A = beta_i (k_i.k_j) exp(gc_i - gc_j) for j < i and
//      intra = (q_i.k_j) exp(gc_i - gc_j) for j <= i.
//   3. (I + A) X = [v beta | k beta exp(gc)] by forward substitution in fp32: one thread per right-hand-side column keeps
//      its 64 unknowns in registers; the rows of A are broadcast from shared memory.  X = [u | w].
//   4. qg = q exp(gc), kd = k exp(gc_last - gc), glast = exp(gc_last).
// The reference builds the same quantities as a graph of library ops over all chunks with a 63-step loop for the solve
// (cc/src/tyr_qwen35.cpp:21-88).  Rows past the sequence end behave as g = 0, beta = 0, q = k = v = 0.
// ------------------------------------------------------------------------------------------------------------------
constexpr int GP_LDA = GC_C + 4;

struct GdrPrepSmem {
  float k[GC_C * GC_LDW];
  float q[GC_C * GC_LDW];
  float a[GC_C * GP_LDA];
  float gc[GC_C];
  float beta[GC_C];
  float eg[GC_C];        // exp(gc_i)
  __nv_bfloat16 v[GC_C * 128];   // the chunk's value rows (dv <= 128), staged with 16-byte loads
};

struct GdrPrepArgs {
  const __nv_bfloat16 *q, *k, *v;
  const float *g, *beta;               // [B, S, Hv] contiguous
  float *u, *w, *qg, *kd, *intra, *glast;
  long long q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh;
  int S, n, Hk, Hv, dv;
};

__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}

__global__ void __launch_bounds__(256, 2) gdr_chunk_prepare_kernel(GdrPrepArgs a) {
  extern __shared__ __align__(16) uint8_t gdr_smem_raw[];
  GdrPrepSmem& sm = *reinterpret_cast<GdrPrepSmem*>(gdr_smem_raw);
  const int c = blockIdx.x, bh = blockIdx.y;
  const int b = bh / a.Hv, hv = bh % a.Hv, hk = hv / (a.Hv / a.Hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row0 = c * GC_C;
  // ---- 1. stage q, k (fp32), g, beta
  for (int i = tid; i < GC_C * (GC_DK / 8); i += 256) {
    const int r = i / (GC_DK / 8), d = (i % (GC_DK / 8)) * 8;
    const int tok = row0 + r;
    uint4 uq = make_uint4(0, 0, 0, 0), uk = make_uint4(0, 0, 0, 0);
    if (tok < a.S) {
      uq = *reinterpret_cast<const uint4*>(a.q + b * a.q_sb + static_cast<long long>(tok) * a.q_ss + hk * a.q_sh + d);
      uk = *reinterpret_cast<const uint4*>(a.k + b * a.k_sb + static_cast<long long>(tok) * a.k_ss + hk * a.k_sh + d);
    }
    const uint32_t qq[4] = {uq.x, uq.y, uq.z, uq.w}, kk[4] = {uk.x, uk.y, uk.z, uk.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 fq = unpack_bf16x2(qq[e]), fk = unpack_bf16x2(kk[e]);
      sm.q[r * GC_LDW + d + 2 * e] = fq.x; sm.q[r * GC_LDW + d + 2 * e + 1] = fq.y;
      sm.k[r * GC_LDW + d + 2 * e] = fk.x; sm.k[r * GC_LDW + d + 2 * e + 1] = fk.y;
    }
  }
  for (int i = tid; i < GC_C * (a.dv / 8); i += 256) {
    const int r = i / (a.dv / 8), d = (i % (a.dv / 8)) * 8;
    const int tok = row0 + r;
    uint4 uv = make_uint4(0, 0, 0, 0);
    if (tok < a.S) uv = *reinterpret_cast<const uint4*>(a.v + b * a.v_sb + static_cast<long long>(tok) * a.v_ss + hv * a.v_sh + d);
    *reinterpret_cast<uint4*>(&sm.v[r * a.dv + d]) = uv;
  }
  if (tid < GC_C) {
    const int tok = row0 + tid;
    const long long gi = (static_cast<long long>(b) * a.S + tok) * a.Hv + hv;
    sm.gc[tid] = tok < a.S ? a.g[gi] : 0.f;
    sm.beta[tid] = tok < a.S ? a.beta[gi] : 0.f;
  }
  __syncthreads();
  // inclusive scan of g over the chunk (warp 0: two elements per lane)
  if (warp == 0) {
    float x0 = sm.gc[2 * lane], x1 = sm.gc[2 * lane + 1];
    float s = x0 + x1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += t;
    }
    const float base = s - (x0 + x1);
    sm.gc[2 * lane] = base + x0;
    sm.gc[2 * lane + 1] = base + x0 + x1;
  }
  // L2 normalisation: 4 threads per row
  {
    const int r = tid >> 2, part = tid & 3;
    float sq = 0.f, sk = 0.f;
    for (int d = part; d < GC_DK; d += 4) {            // bank (4 r + part + 4 i): the 32 lanes hit 32 banks
      const float x = sm.q[r * GC_LDW + d], y = sm.k[r * GC_LDW + d];
      sq += x * x; sk += y * y;
    }
    sq += __shfl_xor_sync(0xffffffffu, sq, 1); sq += __shfl_xor_sync(0xffffffffu, sq, 2);
    sk += __shfl_xor_sync(0xffffffffu, sk, 1); sk += __shfl_xor_sync(0xffffffffu, sk, 2);
    const float qn = rsqrtf(sq + 1e-6f) * rsqrtf(static_cast<float>(GC_DK)), kn = rsqrtf(sk + 1e-6f);
    for (int d = part; d < GC_DK; d += 4) {
      sm.q[r * GC_LDW + d] *= qn;
      sm.k[r * GC_LDW + d] *= kn;
    }
  }
  __syncthreads();
  if (tid < GC_C) sm.eg[tid] = __expf(sm.gc[tid]);
  // ---- 2. warps 0-3: k k^T strips, warps 4-7: q k^T strips (16 rows each), 3-term TF32
  {
    const int g8 = lane >> 2, t = lane & 3;
    const bool is_q = warp >= 4;
    const float* A = is_q ? sm.q : sm.k;
    const int ar = (warp & 3) * 16 + g8;
    float acc[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
#pragma unroll 2
    for (int kk = 0; kk < GC_DK / 8; ++kk) {
      const int kc = kk * 8 + t;
      const float af[4] = {A[ar * GC_LDW + kc], A[(ar + 8) * GC_LDW + kc], A[ar * GC_LDW + kc + 4], A[(ar + 8) * GC_LDW + kc + 4]};
      uint32_t ah[4], al[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        ah[e] = to_tf32(af[e]);
        al[e] = to_tf32(af[e] - __uint_as_float(ah[e]));
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const float b0f = sm.k[(nt * 8 + g8) * GC_LDW + kc], b1f = sm.k[(nt * 8 + g8) * GC_LDW + kc + 4];
        const uint32_t b0h = to_tf32(b0f), b1h = to_tf32(b1f);
        const uint32_t b0l = to_tf32(b0f - __uint_as_float(b0h)), b1l = to_tf32(b1f - __uint_as_float(b1h));
        mma_tf32(acc[nt], al[0], al[1], al[2], al[3], b0h, b1h);
        mma_tf32(acc[nt], ah[0], ah[1], ah[2], ah[3], b0l, b1l);
        mma_tf32(acc[nt], ah[0], ah[1], ah[2], ah[3], b0h, b1h);
      }
    }
    __syncthreads();          // eg ready (written above by other threads)
    float* intra_o = a.intra + (static_cast<long long>(bh) * a.n + c) * GC_C * GC_C;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const int i = ar + h2 * 8, j = nt * 8 + 2 * t;
        const float gi = sm.gc[i];
        float v0 = acc[nt][2 * h2] * __expf(gi - sm.gc[j]), v1 = acc[nt][2 * h2 + 1] * __expf(gi - sm.gc[j + 1]);
        if (is_q) {
          v0 = j <= i ? v0 : 0.f;
          v1 = j + 1 <= i ? v1 : 0.f;
          *reinterpret_cast<float2*>(intra_o + i * GC_C + j) = make_float2(v0, v1);
        } else {
          const float bi = sm.beta[i];
          sm.a[i * GP_LDA + j] = j < i ? v0 * bi : 0.f;
          sm.a[i * GP_LDA + j + 1] = j + 1 < i ? v1 * bi : 0.f;
        }
      }
  }
  __syncthreads();
  // ---- 3. forward substitution, one right-hand-side column per thread
  {
    const int col = tid;
    const int ncol = a.dv + GC_DK;
    if (col < ncol) {
      float x[GC_C];
      const bool is_v = col < a.dv;
      if (is_v) {
#pragma unroll
        for (int i = 0; i < GC_C; ++i) x[i] = __bfloat162float(sm.v[i * a.dv + col]) * sm.beta[i];
      } else {
#pragma unroll
        for (int i = 0; i < GC_C; ++i) x[i] = sm.k[i * GC_LDW + (col - a.dv)] * sm.beta[i] * sm.eg[i];
      }
#pragma unroll
      for (int i = 1; i < GC_C; ++i) {
        float acc = x[i];
#pragma unroll
        for (int j4 = 0; j4 < (i + 3) / 4; ++j4) {
          const float4 r4 = *reinterpret_cast<const float4*>(&sm.a[i * GP_LDA + 4 * j4]);     // entries at j >= i are zero
          acc -= r4.x * x[4 * j4];
          if (4 * j4 + 1 < i) acc -= r4.y * x[4 * j4 + 1];
          if (4 * j4 + 2 < i) acc -= r4.z * x[4 * j4 + 2];
          if (4 * j4 + 3 < i) acc -= r4.w * x[4 * j4 + 3];
        }
        x[i] = acc;
      }
      float* dst = is_v ? a.u + (static_cast<long long>(bh) * a.n + c) * GC_C * a.dv + col
                        : a.w + (static_cast<long long>(bh) * a.n + c) * GC_C * GC_DK + (col - a.dv);
      const int ld = is_v ? a.dv : GC_DK;
#pragma unroll
      for (int i = 0; i < GC_C; ++i) dst[static_cast<long long>(i) * ld] = x[i];
    }
  }
  // ---- 4. qg, kd, glast
  {
    const float g_last = sm.gc[GC_C - 1];
    float* qg_o = a.qg + (static_cast<long long>(bh) * a.n + c) * GC_C * GC_DK;
    float* kd_o = a.kd + (static_cast<long long>(bh) * a.n + c) * GC_C * GC_DK;
    for (int i = tid; i < GC_C * (GC_DK / 4); i += 256) {
      const int r = i / (GC_DK / 4), d = (i % (GC_DK / 4)) * 4;
      const float eq = sm.eg[r], ek = __expf(g_last - sm.gc[r]);
      const float4 fq = *reinterpret_cast<const float4*>(&sm.q[r * GC_LDW + d]);
      const float4 fk = *reinterpret_cast<const float4*>(&sm.k[r * GC_LDW + d]);
      *reinterpret_cast<float4*>(qg_o + r * GC_DK + d) = make_float4(fq.x * eq, fq.y * eq, fq.z * eq, fq.w * eq);
      *reinterpret_cast<float4*>(kd_o + r * GC_DK + d) = make_float4(fk.x * ek, fk.y * ek, fk.z * ek, fk.w * ek);
    }
    if (tid == 0) a.glast[static_cast<long long>(bh) * a.n + c] = __expf(g_last);
  }
}

}  // namespace tyr

// Causal depthwise conv1d (kernel taps K <= 4, zero history) + bias + SiLU on channels-last activations:
//   y[b, s, c] = silu(bias[c] + sum_j w[c, j] * x[b, s - (K - 1) + j, c]).
// One thread per (32 tokens, 8 channels): its taps and a sliding window of K rows stay in registers, so every input row is
// loaded once and a warp's accesses are 512 contiguous bytes.  The reference transposes to channels-first
// and calls the library's grouped convolution (Tyr/Model/Qwen35/Model.lean:642-700).
namespace tyr {
constexpr int CONV_TOK = 32;      // tokens per thread: the taps and the sliding window stay in registers
template <int K>
__global__ void __launch_bounds__(256) causal_conv1d_silu_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                                                 const float* __restrict__ bias, __nv_bfloat16* __restrict__ y,
                                                                 long long total, int S, int C, long long x_sb, long long x_ss) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c8 = C >> 3;
  const int c = static_cast<int>(i % c8) * 8;
  const long long bt = i / c8;
  const int nblk = (S + CONV_TOK - 1) / CONV_TOK;
  const int s0 = static_cast<int>(bt % nblk) * CONV_TOK;
  const long long b = bt / nblk;
  float wt[8][K], bs[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    bs[e] = bias ? bias[c + e] : 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) wt[e][j] = w[(c + e) * K + j];
  }
  float win[K][8];                                   // win[j] = x[s - (K - 1) + j]
  const __nv_bfloat16* xb = x + b * x_sb + c;
  auto load_row = [&](int t, float (&dst)[8]) {
    if (t < 0 || t >= S) {
#pragma unroll
      for (int e = 0; e < 8; ++e) dst[e] = 0.f;
      return;
    }
    const uint4 u = *reinterpret_cast<const uint4*>(xb + static_cast<long long>(t) * x_ss);
    const uint32_t uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf16x2(uu[e]);
      dst[2 * e] = f.x;
      dst[2 * e + 1] = f.y;
    }
  };
#pragma unroll
  for (int j = 0; j < K - 1; ++j) load_row(s0 - (K - 1) + j, win[j]);
  for (int s = s0; s < min(S, s0 + CONV_TOK); ++s) {
    load_row(s, win[K - 1]);
    uint4 o;
    uint32_t* oo = reinterpret_cast<uint32_t*>(&o);
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      acc[e] = bs[e];
#pragma unroll
      for (int j = 0; j < K; ++j) acc[e] += win[j][e] * wt[e][j];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float a0 = acc[2 * e], a1 = acc[2 * e + 1];
      oo[e] = pack_bf16x2(a0 / (1.f + __expf(-a0)), a1 / (1.f + __expf(-a1)));
    }
    *reinterpret_cast<uint4*>(y + (b * S + s) * C + c) = o;
#pragma unroll
    for (int j = 0; j < K - 1; ++j)
#pragma unroll
      for (int e = 0; e < 8; ++e) win[j][e] = win[j + 1][e];
  }
}
}  // namespace tyr

// x: bf16 [B, S, C] with (batch, token) element strides and contiguous channels; w: fp32 [C, K]; bias: fp32 [C] or null;
// y: bf16 [B, S, C] contiguous.  C must be a multiple of 8.
extern "C" TYR_EXPORT int tyr_causal_conv1d_silu(const void* x, const float* w, const float* bias, void* y, int B, int S, int C,
                                                 int K, long long x_sb, long long x_ss, void* stream) {
  if (B <= 0 || S <= 0 || C <= 0 || (C & 7) || K <= 0 || K > 4 || (x_sb & 7) || (x_ss & 7)) return -1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) return -2;
  const long long total = static_cast<long long>(B) * ((S + tyr::CONV_TOK - 1) / tyr::CONV_TOK) * (C >> 3);
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  auto* xx = reinterpret_cast<const __nv_bfloat16*>(x);
  auto* yy = reinterpret_cast<__nv_bfloat16*>(y);
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
  switch (K) {
    case 1: tyr::causal_conv1d_silu_kernel<1><<<blocks, 256, 0, cs>>>(xx, w, bias, yy, total, S, C, x_sb, x_ss); break;
    case 2: tyr::causal_conv1d_silu_kernel<2><<<blocks, 256, 0, cs>>>(xx, w, bias, yy, total, S, C, x_sb, x_ss); break;
    case 3: tyr::causal_conv1d_silu_kernel<3><<<blocks, 256, 0, cs>>>(xx, w, bias, yy, total, S, C, x_sb, x_ss); break;
    case 4: tyr::causal_conv1d_silu_kernel<4><<<blocks, 256, 0, cs>>>(xx, w, bias, yy, total, S, C, x_sb, x_ss); break;
    default: return -3;
  }
  return static_cast<int>(cudaGetLastError());
}

// Chunk-local quantities of the gated delta rule (chunk 64, dk 128, dv 64 or 128).  q, k: bf16 [B, S, Hk, 128] and
// v: bf16 [B, S, Hv, dv] given by (batch, token, head) element strides; g, beta: fp32 [B, S, Hv] contiguous.  Outputs (fp32,
// n = ceil(S / 64) chunks): u [B*Hv, n, 64, dv], w / qg / kd [B*Hv, n, 64, 128], intra [B*Hv, n, 64, 64], glast [B*Hv, n].
extern "C" TYR_EXPORT int tyr_gdr_chunk_prepare(const void* q, const void* k, const void* v, const float* g,
                                                const float* beta, float* u, float* w, float* qg, float* kd,
                                                float* intra, float* glast, const long long* strides, int B, int S,
                                                int Hk, int Hv, int dk, int dv, void* stream) {
  using namespace tyr;
  if (B <= 0 || S <= 0 || Hk <= 0 || Hv <= 0 || Hv % Hk || dk != GC_DK || (dv != 64 && dv != 128)) return -1;
  for (int i = 0; i < 9; ++i)
    if (strides[i] & 7) return -3;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) return -4;
  GdrPrepArgs a;
  a.q = reinterpret_cast<const __nv_bfloat16*>(q);
  a.k = reinterpret_cast<const __nv_bfloat16*>(k);
  a.v = reinterpret_cast<const __nv_bfloat16*>(v);
  a.g = g; a.beta = beta; a.u = u; a.w = w; a.qg = qg; a.kd = kd; a.intra = intra; a.glast = glast;
  a.q_sb = strides[0]; a.q_ss = strides[1]; a.q_sh = strides[2];
  a.k_sb = strides[3]; a.k_ss = strides[4]; a.k_sh = strides[5];
  a.v_sb = strides[6]; a.v_ss = strides[7]; a.v_sh = strides[8];
  a.S = S; a.n = (S + GC_C - 1) / GC_C; a.Hk = Hk; a.Hv = Hv; a.dv = dv;
  constexpr size_t smem = sizeof(GdrPrepSmem);
  static bool configured_dev[64] = {false};     // the attribute is per device
  int cfg_dev = 0;
  if (cudaGetDevice(&cfg_dev) != cudaSuccess || cfg_dev < 0 || cfg_dev >= 64) cfg_dev = 0;
  bool& configured = configured_dev[cfg_dev];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gdr_chunk_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return 1000 + (int)e;
    configured = true;
  }
  gdr_chunk_prepare_kernel<<<dim3(a.n, B * Hv), 256, smem, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return static_cast<int>(cudaGetLastError());
}

// Sequential chunk pass of the gated delta rule (chunk 64, dk 128, dv a multiple of 64), all tensors fp32 and contiguous:
// u [BH, n, 64, dv], w / qg / kd [BH, n, 64, 128], intra [BH, n, 64, 64], glast [BH, n] (= exp of the chunk's last cumulative
// log decay), state_in [BH, 128, dv] (nullable = zeros), state_out [BH, 128, dv]; out: bf16 [B, S, Hv, dv] with BH = B * Hv and
// n = ceil(S / 64).
extern "C" TYR_EXPORT int tyr_gdr_chunk_scan(const float* u, const float* w, const float* qg, const float* kd,
                                             const float* intra, const float* glast, const float* state_in,
                                             float* state_out, void* out, int BH, int n, int dk, int dv, int chunk, int S,
                                             int Hv, void* stream) {
  using namespace tyr;
  if (BH <= 0 || n <= 0 || dk != GC_DK || chunk != GC_C || dv <= 0 || dv % GC_DVS || Hv <= 0 || BH % Hv || S <= 0 || S > n * GC_C) return -1;
  if ((reinterpret_cast<uintptr_t>(u) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(qg) |
       reinterpret_cast<uintptr_t>(kd) | reinterpret_cast<uintptr_t>(intra) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(state_out) | reinterpret_cast<uintptr_t>(state_in)) & 15)
    return -2;
  constexpr size_t smem = sizeof(GdrChunkSmem);
  static bool configured_dev[64] = {false};     // the attribute is per device
  int cfg_dev = 0;
  if (cudaGetDevice(&cfg_dev) != cudaSuccess || cfg_dev < 0 || cfg_dev >= 64) cfg_dev = 0;
  bool& configured = configured_dev[cfg_dev];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gdr_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return 1000 + (int)e;
    configured = true;
  }
  gdr_chunk_scan_kernel<<<dim3(dv / GC_DVS, BH), 128, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
      u, w, qg, kd, intra, glast, state_in, state_out, reinterpret_cast<__nv_bfloat16*>(out), n, dv, S, Hv);
  return static_cast<int>(cudaGetLastError());
}

extern "C" TYR_EXPORT int tyr_gdr_decode_norm(const void* q, const void* k, const void* v, const float* g, const float* beta,
                                              float* state, void* out, int B, int Hk, int Hv, int dk, int dv,
                                              long long q_bstride, long long v_bstride, const void* z, long long z_bstride,
                                              const void* norm_w, float norm_eps, void* stream);

// Conv + SiLU (state shifted in place) and the per-head gates of one decode token; see gdn_conv_gates_kernel.
extern "C" TYR_EXPORT int tyr_gdn_conv_gates(const void* mixed, const void* b_in, const void* a_in, long long ld_m, long long ld_b,
                                             long long ld_a, void* conv_state,
                                             const void* conv_w, const void* conv_b, const float* dt_bias, const float* a_log,
                                             void* conv_out, float* g, float* beta, int B, int cd, int K, int Hv, void* stream) {
  using namespace tyr;
  if (B <= 0 || cd <= 0 || K < 1 || K > 8 || Hv <= 0) return -1;
  const long long n = static_cast<long long>(B) * cd + static_cast<long long>(B) * Hv;
  launch_dependent(gdn_conv_gates_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
      (const __nv_bfloat16*)mixed, (const __nv_bfloat16*)b_in, (const __nv_bfloat16*)a_in, ld_m, ld_b, ld_a, (__nv_bfloat16*)conv_state,
      (const __nv_bfloat16*)conv_w, (const __nv_bfloat16*)conv_b, dt_bias, a_log, (__nv_bfloat16*)conv_out, g, beta, B, cd, K, Hv);
  return static_cast<int>(cudaGetLastError());
}

// q, k: bf16 [B, Hk, dk] (rows may be strided by q_bstride elements between batches); v: bf16 [B, Hv, dv]
// (v_bstride); g, beta: fp32 [B, Hv]; state: fp32 [B, Hv, dk, dv] updated in place; out: bf16 [B, Hv, dv].
extern "C" TYR_EXPORT int tyr_gdr_decode(const void* q, const void* k, const void* v, const float* g, const float* beta,
                                         float* state, void* out, int B, int Hk, int Hv, int dk, int dv,
                                         long long q_bstride, long long v_bstride, void* stream) {
  return tyr_gdr_decode_norm(q, k, v, g, beta, state, out, B, Hk, Hv, dk, dv, q_bstride, v_bstride, nullptr, 0, nullptr, 0.f,
                             stream);
}

// dv == 128, dk 64 or 128, v / z rows 8-byte aligned (strides multiples of 4 elements): the shared-memory tile form of the
// step (gdr_decode_tile_kernel); `z` / `norm_w` may be null (no gated RMSNorm).  `err`: the device error record.
extern "C" TYR_EXPORT int tyr_gdr_decode_tile(const void* q, const void* k, const void* v, const float* g, const float* beta,
                                              float* state, void* out, int B, int Hk, int Hv, int dk,
                                              long long q_bstride, long long v_bstride, const void* z, long long z_bstride,
                                              const void* norm_w, float norm_eps, int* err, void* stream) {
  using namespace tyr;
  if (B <= 0 || Hk <= 0 || Hv <= 0 || Hv % Hk != 0 || (dk != 64 && dk != 128)) return -1;
  if (z != nullptr && norm_w == nullptr) return -3;
  if ((v_bstride & 3) || (z != nullptr && (z_bstride & 3))) return -4;
  if ((reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(z) | reinterpret_cast<uintptr_t>(out)) & 7) return -4;
  if (reinterpret_cast<uintptr_t>(state) & 15) return -4;
  const size_t smem = static_cast<size_t>(dk) * 128 * 4;
  static bool configured[64][2] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  const int which = dk == 128 ? 1 : 0;
  if (!configured[dev][which]) {
    cudaError_t e = dk == 128 ? cudaFuncSetAttribute(gdr_decode_tile_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                              : cudaFuncSetAttribute(gdr_decode_tile_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return 1000 + static_cast<int>(e);
    configured[dev][which] = true;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  auto* qq = reinterpret_cast<const __nv_bfloat16*>(q);
  auto* kk = reinterpret_cast<const __nv_bfloat16*>(k);
  auto* vv = reinterpret_cast<const __nv_bfloat16*>(v);
  auto* zz = reinterpret_cast<const __nv_bfloat16*>(z);
  auto* nw = reinterpret_cast<const __nv_bfloat16*>(norm_w);
  auto* oo = reinterpret_cast<__nv_bfloat16*>(out);
  cudaError_t e;
  if (dk == 128)
    e = launch_dependent(gdr_decode_tile_kernel<128>, dim3(B * Hv), dim3(256), smem, st, qq, kk, vv, g, beta, state, oo, Hk, Hv,
                         q_bstride, v_bstride, zz, z_bstride, nw, norm_eps, err);
  else
    e = launch_dependent(gdr_decode_tile_kernel<64>, dim3(B * Hv), dim3(256), smem, st, qq, kk, vv, g, beta, state, oo, Hk, Hv,
                         q_bstride, v_bstride, zz, z_bstride, nw, norm_eps, err);
  return static_cast<int>(e);
}

// The same step with the layer's gated RMSNorm in the epilogue when `z` (bf16 [B, Hv, dv], batch stride z_bstride) and
// `norm_w` (bf16 [dv]) are given; that form needs dv == 128.
extern "C" TYR_EXPORT int tyr_gdr_decode_norm(const void* q, const void* k, const void* v, const float* g, const float* beta,
                                              float* state, void* out, int B, int Hk, int Hv, int dk, int dv,
                                              long long q_bstride, long long v_bstride, const void* z, long long z_bstride,
                                              const void* norm_w, float norm_eps, void* stream) {
  using namespace tyr;
  if (B <= 0 || Hk <= 0 || Hv <= 0 || Hv % Hk != 0 || dv <= 0) return -1;
  if (z != nullptr && (dv != 128 || norm_w == nullptr)) return -3;
  auto* zz = reinterpret_cast<const __nv_bfloat16*>(z);
  auto* nw = reinterpret_cast<const __nv_bfloat16*>(norm_w);
  dim3 grid(B * Hv, (dv + 127) / 128);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  auto* qq = reinterpret_cast<const __nv_bfloat16*>(q);
  auto* kk = reinterpret_cast<const __nv_bfloat16*>(k);
  auto* vv = reinterpret_cast<const __nv_bfloat16*>(v);
  auto* oo = reinterpret_cast<__nv_bfloat16*>(out);
  if (dk == 128)
    launch_dependent(gdr_decode_kernel<128>, dim3(grid), dim3(512), 0, st, qq, kk, vv, g, beta, state, oo, Hk, Hv, dv, q_bstride, v_bstride, zz, z_bstride,
                                                 nw, norm_eps);
  else if (dk == 64)
    launch_dependent(gdr_decode_kernel<64>, dim3(grid), dim3(512), 0, st, qq, kk, vv, g, beta, state, oo, Hk, Hv, dv, q_bstride, v_bstride, zz, z_bstride,
                                                nw, norm_eps);
  else
    return -2;
  return static_cast<int>(cudaGetLastError());
}
