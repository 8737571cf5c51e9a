// Adaptive-LayerNorm pieces of the Flux DiT blocks, fused so that each activation row is read
// once and written once:
//  * layernorm_modulate:  y = (1 + scale[b]) * LayerNorm(x) + shift[b]   (no affine weights)
//  * gate_residual:       out = x + gate[b] * y
//  * flux_qk_post:        q, k <- RoPE(RMSNorm(q, k) * weight) per head, straight from the fused projection's output into the
//                         packed [B, S_total, 3, H, 128] buffer the attention kernel reads (in place when source and destination
//                         coincide; text and image streams land at their row offsets of one joint buffer, so no concatenation)
// Rows are [batch, seq, D] bf16; scale / shift / gate are per-batch vectors addressed with an
// element stride so that the chunks of one [batch, n_mods, D] modulation tensor are used in place
// (Tyr/Model/Flux/Modulation.lean:84-109, DoubleStreamBlock.lean:143-215 of the reference).
#include "common.cuh"

namespace tyr {

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// one warp per row; the second pass re-reads the row from L1/L2
__global__ void __launch_bounds__(256)
layernorm_modulate_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ scale,
                          const __nv_bfloat16* __restrict__ shift, __nv_bfloat16* __restrict__ y,
                          long long rows, int seq, int D, long long mod_bstride, float eps) {
  pdl_entry();
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int nvec = D >> 3;
  for (long long row = blockIdx.x * static_cast<long long>(warps) + (threadIdx.x >> 5); row < rows;
       row += static_cast<long long>(gridDim.x) * warps) {
    const __nv_bfloat16* xr = x + row * D;
    float sum = 0.f, sq = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      float f[8];
      ld8(xr + v * 8, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) { sum += f[j]; sq += f[j] * f[j]; }
    }
    sum = warp_sum(sum); sq = warp_sum(sq);
    const float mean = sum / D;
    const float rstd = rsqrtf(fmaxf(sq / D - mean * mean, 0.f) + eps);
    const long long b = row / seq;
    const __nv_bfloat16* sc = scale ? scale + b * mod_bstride : nullptr;
    const __nv_bfloat16* sh = shift ? shift + b * mod_bstride : nullptr;
    for (int v = lane; v < nvec; v += 32) {
      float f[8], s[8], t[8];
      ld8(xr + v * 8, f);
      if (sc) ld8(sc + v * 8, s);
      if (sh) ld8(sh + v * 8, t);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float n = (f[j] - mean) * rstd;
        if (sc) n *= 1.f + s[j];
        if (sh) n += t[j];
        f[j] = n;
      }
      st8(y + row * D + v * 8, f);
    }
  }
}

__global__ void __launch_bounds__(256)
gate_residual_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ yv,
                     const __nv_bfloat16* __restrict__ gate, __nv_bfloat16* __restrict__ out,
                     long long rows, int seq, int D, long long mod_bstride) {
  pdl_entry();
  const int nvec = D >> 3;
  const long long total = rows * nvec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / nvec;
    const int v = static_cast<int>(i % nvec);
    float a[8], b[8], g[8];
    ld8(x + row * D + v * 8, a);
    ld8(yv + row * D + v * 8, b);
    ld8(gate + (row / seq) * mod_bstride + v * 8, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] += g[j] * b[j];
    st8(out + row * D + v * 8, a);
  }
}

struct FluxQkPostArgs {
  const __nv_bfloat16* src;      // [B, S, >= 3 * H * 128]: q at column 0, k at H * 128, v at 2 * H * 128
  long long src_sb, src_st;      // element strides of batch and row
  __nv_bfloat16* dst;            // same column layout; row s of the source goes to row dst_row0 + s
  long long dst_sb, dst_st;
  const __nv_bfloat16* wq;       // [128] RMSNorm weights
  const __nv_bfloat16* wk;
  const float* cosv;             // [B or 1, S, 64]
  const float* sinv;
  long long cs_sb;               // batch stride of cos / sin (0: shared by the batch)
  int B, S, H, dst_row0, copy_v;
  float eps;
};

// One warp per (batch, row, head): lane l owns elements 4l .. 4l+3 of the 128-wide head, i.e. the rotation pairs 2l and 2l+1.
// fp32 throughout; one rounding to bf16 at the end (the unfused sequence rounds after the norm as well).
__global__ void __launch_bounds__(256) flux_qk_post_kernel(FluxQkPostArgs a) {
  pdl_entry();
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(a.B) * a.S * a.H;
  const float2 wq0 = unpack_bf16x2(reinterpret_cast<const uint32_t*>(a.wq)[2 * lane]);
  const float2 wq1 = unpack_bf16x2(reinterpret_cast<const uint32_t*>(a.wq)[2 * lane + 1]);
  const float2 wk0 = unpack_bf16x2(reinterpret_cast<const uint32_t*>(a.wk)[2 * lane]);
  const float2 wk1 = unpack_bf16x2(reinterpret_cast<const uint32_t*>(a.wk)[2 * lane + 1]);
  for (long long w = blockIdx.x * 8LL + (threadIdx.x >> 5); w < total; w += gridDim.x * 8LL) {
    const int h = static_cast<int>(w % a.H);
    const long long bs = w / a.H;
    const int srow = static_cast<int>(bs % a.S);
    const int b = static_cast<int>(bs / a.S);
    const __nv_bfloat16* src = a.src + b * a.src_sb + static_cast<long long>(srow) * a.src_st + h * 128 + lane * 4;
    __nv_bfloat16* dst = a.dst + b * a.dst_sb + static_cast<long long>(a.dst_row0 + srow) * a.dst_st + h * 128 + lane * 4;
    const int hd = a.H * 128;
    const uint2 uq = *reinterpret_cast<const uint2*>(src);
    const uint2 uk = *reinterpret_cast<const uint2*>(src + hd);
    const float2 cs = *reinterpret_cast<const float2*>(a.cosv + b * a.cs_sb + static_cast<long long>(srow) * 64 + lane * 2);
    const float2 sn = *reinterpret_cast<const float2*>(a.sinv + b * a.cs_sb + static_cast<long long>(srow) * 64 + lane * 2);
    float2 q0 = unpack_bf16x2(uq.x), q1 = unpack_bf16x2(uq.y), k0 = unpack_bf16x2(uk.x), k1 = unpack_bf16x2(uk.y);
    float sq = q0.x * q0.x + q0.y * q0.y + q1.x * q1.x + q1.y * q1.y;
    float sk = k0.x * k0.x + k0.y * k0.y + k1.x * k1.x + k1.y * k1.y;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sq += __shfl_xor_sync(0xffffffffu, sq, o);
      sk += __shfl_xor_sync(0xffffffffu, sk, o);
    }
    const float rq = rsqrtf(sq * (1.f / 128.f) + a.eps), rk = rsqrtf(sk * (1.f / 128.f) + a.eps);
    q0.x *= rq * wq0.x; q0.y *= rq * wq0.y; q1.x *= rq * wq1.x; q1.y *= rq * wq1.y;
    k0.x *= rk * wk0.x; k0.y *= rk * wk0.y; k1.x *= rk * wk1.x; k1.y *= rk * wk1.y;
    uint2 oq, ok;
    oq.x = pack_bf16x2(cs.x * q0.x - sn.x * q0.y, sn.x * q0.x + cs.x * q0.y);
    oq.y = pack_bf16x2(cs.y * q1.x - sn.y * q1.y, sn.y * q1.x + cs.y * q1.y);
    ok.x = pack_bf16x2(cs.x * k0.x - sn.x * k0.y, sn.x * k0.x + cs.x * k0.y);
    ok.y = pack_bf16x2(cs.y * k1.x - sn.y * k1.y, sn.y * k1.x + cs.y * k1.y);
    *reinterpret_cast<uint2*>(dst) = oq;
    *reinterpret_cast<uint2*>(dst + hd) = ok;
    if (a.copy_v) *reinterpret_cast<uint2*>(dst + 2 * hd) = *reinterpret_cast<const uint2*>(src + 2 * hd);
  }
}

}  // namespace tyr

// Returns 0 on success, -1 on a bad shape, stride or alignment.
extern "C" TYR_EXPORT int tyr_flux_qk_post(const void* src, long long src_sb, long long src_st, void* dst, long long dst_sb,
                                           long long dst_st, const void* wq, const void* wk, const float* cosv, const float* sinv,
                                           long long cs_sb, int B, int S, int H, int D, int dst_row0, int copy_v, float eps,
                                           void* stream) {
  using namespace tyr;
  if (D != 128 || B <= 0 || S <= 0 || H <= 0 || dst_row0 < 0) return -1;
  if ((src_sb & 3) || (src_st & 3) || (dst_sb & 3) || (dst_st & 3) || (cs_sb & 1)) return -1;
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(wq) |
       reinterpret_cast<uintptr_t>(wk) | reinterpret_cast<uintptr_t>(cosv) | reinterpret_cast<uintptr_t>(sinv)) & 7)
    return -1;
  FluxQkPostArgs a;
  a.src = (const __nv_bfloat16*)src; a.src_sb = src_sb; a.src_st = src_st;
  a.dst = (__nv_bfloat16*)dst; a.dst_sb = dst_sb; a.dst_st = dst_st;
  a.wq = (const __nv_bfloat16*)wq; a.wk = (const __nv_bfloat16*)wk;
  a.cosv = cosv; a.sinv = sinv; a.cs_sb = cs_sb;
  a.B = B; a.S = S; a.H = H; a.dst_row0 = dst_row0; a.copy_v = copy_v; a.eps = eps;
  long long blocks = (static_cast<long long>(B) * S * H + 7) / 8;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  launch_dependent(flux_qk_post_kernel, dim3(static_cast<int>(blocks)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), a);
  return static_cast<int>(cudaGetLastError());
}

extern "C" TYR_EXPORT int tyr_layernorm_modulate(const void* x, const void* scale, const void* shift, void* y,
                                                 long long rows, int seq, int D, long long mod_bstride, float eps,
                                                 void* stream) {
  using namespace tyr;
  if (rows <= 0 || seq <= 0 || (D & 7) || (mod_bstride & 7)) return -1;
  long long blocks = (rows + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  launch_dependent(layernorm_modulate_kernel, dim3(static_cast<int>(blocks)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)scale, (const __nv_bfloat16*)shift, (__nv_bfloat16*)y, rows, seq, D,
      mod_bstride, eps);
  return static_cast<int>(cudaGetLastError());
}

extern "C" TYR_EXPORT int tyr_gate_residual(const void* x, const void* y, const void* gate, void* out, long long rows,
                                            int seq, int D, long long mod_bstride, void* stream) {
  using namespace tyr;
  if (rows <= 0 || seq <= 0 || (D & 7) || (mod_bstride & 7)) return -1;
  long long blocks = (rows * (D >> 3) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  launch_dependent(gate_residual_kernel, dim3(static_cast<int>(blocks)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)y, (const __nv_bfloat16*)gate, (__nv_bfloat16*)out, rows, seq, D,
      mod_bstride);
  return static_cast<int>(cudaGetLastError());
}
