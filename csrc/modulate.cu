// Adaptive-LayerNorm pieces of the Flux DiT blocks, fused so that each activation row is read
// once and written once:
//  * layernorm_modulate:  y = (1 + scale[b]) * LayerNorm(x) + shift[b]   (no affine weights)
//  * gate_residual:       out = x + gate[b] * y
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

}  // namespace tyr

extern "C" TYR_EXPORT int tyr_layernorm_modulate(const void* x, const void* scale, const void* shift, void* y,
                                                 long long rows, int seq, int D, long long mod_bstride, float eps,
                                                 void* stream) {
  using namespace tyr;
  if (rows <= 0 || seq <= 0 || (D & 7) || (mod_bstride & 7)) return -1;
  long long blocks = (rows + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  layernorm_modulate_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
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
  gate_residual_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)y, (const __nv_bfloat16*)gate, (__nv_bfloat16*)out, rows, seq, D,
      mod_bstride);
  return static_cast<int>(cudaGetLastError());
}
