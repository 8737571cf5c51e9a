// Fused optimizer kernels (single-GPU forms; the multi-GPU forms that pull peer gradient
// shards over NVLink live in comm_fused.cu and share the update math below).
//
//  * adamw_step: bias-corrected AdamW with decoupled weight decay on fp32 master weights, fp32
//    moments, bf16 or fp32 gradients, and the bf16 working copy refreshed in the same pass.
//    Reference math: Tyr/Optim/DistAdam.lean:109-158 (about 15 elementwise kernels there).
//  * muon_momentum: m = mu*m + (1-mu)*g ; u = (1-mu)*g + mu*m (Nesterov blend) written as bf16
//    into the Newton-Schulz input, plus per-matrix sum of squares for the Frobenius normalise
//    (Tyr/Optim/NorMuon.lean:196-203, 232-246; cc/src/tyr_polar.cpp:283-293).
//  * scale_rows_by_inv_norm: X <- X / (||X||_F + 1e-7) per matrix of a stacked batch.
//  * muon_apply: p <- p*(1 - lr*wd) - lr * O (O = bf16 orthogonalised update), master + bf16.
#include "common.cuh"

namespace tyr {

__device__ __forceinline__ float4 ld_grad4(const void* g, long long i, int g_is_bf16) {
  if (g_is_bf16) {
    uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(g) + i);
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
    return make_float4(a.x, a.y, b.x, b.y);
  }
  return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(g) + i);
}

struct AdamArgs {
  float* p;                // fp32 master
  __nv_bfloat16* p_bf16;   // nullable
  const void* g;
  float* m;
  float* v;
  long long n;
  float lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale;
  int g_is_bf16;
};

__device__ __forceinline__ void adam_elem(float& p, float g, float& m, float& v, const AdamArgs& a) {
  g *= a.grad_scale;
  m = a.beta1 * m + (1.f - a.beta1) * g;
  v = a.beta2 * v + (1.f - a.beta2) * g * g;
  const float mh = m / a.bc1;
  const float vh = v / a.bc2;
  p = p * (1.f - a.lr * a.wd) - a.lr * mh / (sqrtf(vh) + a.eps);
}

__global__ void __launch_bounds__(256) adamw_kernel(AdamArgs a) {
  pdl_entry();
  const long long n4 = a.n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 p = reinterpret_cast<float4*>(a.p)[i];
    float4 m = reinterpret_cast<float4*>(a.m)[i];
    float4 v = reinterpret_cast<float4*>(a.v)[i];
    float4 g = ld_grad4(a.g, i * 4, a.g_is_bf16);
    adam_elem(p.x, g.x, m.x, v.x, a);
    adam_elem(p.y, g.y, m.y, v.y, a);
    adam_elem(p.z, g.z, m.z, v.z, a);
    adam_elem(p.w, g.w, m.w, v.w, a);
    reinterpret_cast<float4*>(a.p)[i] = p;
    reinterpret_cast<float4*>(a.m)[i] = m;
    reinterpret_cast<float4*>(a.v)[i] = v;
    if (a.p_bf16) {
      uint2 u;
      u.x = pack_bf16x2(p.x, p.y);
      u.y = pack_bf16x2(p.z, p.w);
      reinterpret_cast<uint2*>(a.p_bf16)[i] = u;
    }
  }
  // tail (n not a multiple of 4)
  const long long tail0 = n4 << 2;
  if (blockIdx.x == 0 && threadIdx.x < a.n - tail0) {
    const long long i = tail0 + threadIdx.x;
    float p = a.p[i], m = a.m[i], v = a.v[i];
    float g = a.g_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.g)[i])
                          : reinterpret_cast<const float*>(a.g)[i];
    adam_elem(p, g, m, v, a);
    a.p[i] = p; a.m[i] = m; a.v[i] = v;
    if (a.p_bf16) a.p_bf16[i] = __float2bfloat16(p);
  }
}

struct MuonMomArgs {
  const void* g;           // [B, per] gradient (bf16 or fp32)
  float* mom;              // [B, per] fp32 momentum buffer
  __nv_bfloat16* u;        // [B, per] bf16 Nesterov-blended update (Newton-Schulz input)
  float* sumsq;            // [B] (must be zero on entry)
  long long per;           // elements per matrix (multiple of 4)
  int B;
  float mu, grad_scale;
  int g_is_bf16;
};

__global__ void __launch_bounds__(256) muon_momentum_kernel(MuonMomArgs a) {
  pdl_entry();
  // grid.y = matrix index, grid.x = chunk of the matrix
  const int b = blockIdx.y;
  const long long base = static_cast<long long>(b) * a.per;
  const long long n4 = a.per >> 2;
  float ss = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 g = ld_grad4(a.g, base + i * 4, a.g_is_bf16);
    float4 m = *reinterpret_cast<float4*>(a.mom + base + i * 4);
    g.x *= a.grad_scale; g.y *= a.grad_scale; g.z *= a.grad_scale; g.w *= a.grad_scale;
    const float om = 1.f - a.mu;
    m.x = a.mu * m.x + om * g.x; m.y = a.mu * m.y + om * g.y;
    m.z = a.mu * m.z + om * g.z; m.w = a.mu * m.w + om * g.w;
    *reinterpret_cast<float4*>(a.mom + base + i * 4) = m;
    float4 u = make_float4(om * g.x + a.mu * m.x, om * g.y + a.mu * m.y, om * g.z + a.mu * m.z,
                           om * g.w + a.mu * m.w);
    uint2 w;
    w.x = pack_bf16x2(u.x, u.y);
    w.y = pack_bf16x2(u.z, u.w);
    *reinterpret_cast<uint2*>(a.u + base + i * 4) = w;
    // norm of the values Newton-Schulz will actually see (bf16-rounded)
    float2 r0 = unpack_bf16x2(w.x), r1 = unpack_bf16x2(w.y);
    ss += r0.x * r0.x + r0.y * r0.y + r1.x * r1.x + r1.y * r1.y;
  }
  __shared__ float red[8];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
    atomicAdd(a.sumsq + b, t);
  }
}

__global__ void __launch_bounds__(256)
scale_by_inv_norm_kernel(__nv_bfloat16* x, const float* sumsq, long long per, float eps) {
  pdl_entry();
  const int b = blockIdx.y;
  const float inv = 1.f / (sqrtf(sumsq[b]) + eps);
  const long long base = static_cast<long long>(b) * per;
  const long long n8 = per >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint4 u = *reinterpret_cast<uint4*>(x + base + i * 8);
    float2 a = unpack_bf16x2(u.x), bb = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    u.x = pack_bf16x2(a.x * inv, a.y * inv);
    u.y = pack_bf16x2(bb.x * inv, bb.y * inv);
    u.z = pack_bf16x2(c.x * inv, c.y * inv);
    u.w = pack_bf16x2(d.x * inv, d.y * inv);
    *reinterpret_cast<uint4*>(x + base + i * 8) = u;
  }
}

__global__ void __launch_bounds__(256)
muon_apply_kernel(float* p, __nv_bfloat16* p_bf16, const __nv_bfloat16* o, long long n, float lr,
                  float wd) {
  pdl_entry();
  const long long n4 = n >> 2;
  const float decay = 1.f - lr * wd;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 w = reinterpret_cast<float4*>(p)[i];
    uint2 u = reinterpret_cast<const uint2*>(o)[i];
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
    // the reference scales the bf16 orthogonalised update by lr in bf16, then casts back
    // (Tyr/Optim/NorMuon.lean:260-263)
    w.x = w.x * decay - __bfloat162float(__float2bfloat16(a.x * lr));
    w.y = w.y * decay - __bfloat162float(__float2bfloat16(a.y * lr));
    w.z = w.z * decay - __bfloat162float(__float2bfloat16(b.x * lr));
    w.w = w.w * decay - __bfloat162float(__float2bfloat16(b.y * lr));
    reinterpret_cast<float4*>(p)[i] = w;
    if (p_bf16) {
      uint2 q;
      q.x = pack_bf16x2(w.x, w.y);
      q.y = pack_bf16x2(w.z, w.w);
      reinterpret_cast<uint2*>(p_bf16)[i] = q;
    }
  }
}

static int grid_1d(long long work_items) {
  long long b = (work_items + 255) / 256;
  const long long cap = 148LL * 8;
  return static_cast<int>(b < cap ? (b < 1 ? 1 : b) : cap);
}

}  // namespace tyr

using namespace tyr;

extern "C" TYR_EXPORT int tyr_adamw_step(float* p, void* p_bf16, const void* g, float* m, float* v,
                                         long long n, float lr, float beta1, float beta2, float eps,
                                         float wd, float bc1, float bc2, float grad_scale,
                                         int g_is_bf16, void* stream) {
  if (n <= 0) return -1;
  AdamArgs a{p, (__nv_bfloat16*)p_bf16, g, m, v, n, lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale,
             g_is_bf16};
  launch_dependent(adamw_kernel, dim3(grid_1d(n / 4 + 1)), dim3(256), 0, (cudaStream_t)stream, a);
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_muon_momentum(const void* g, float* mom, void* u, float* sumsq,
                                            long long per, int B, float mu, float grad_scale,
                                            int g_is_bf16, void* stream) {
  if (per <= 0 || (per & 3) || B <= 0 || B > 65535) return -1;
  MuonMomArgs a{g, mom, (__nv_bfloat16*)u, sumsq, per, B, mu, grad_scale, g_is_bf16};
  int gx = static_cast<int>((per / 4 + 255) / 256);
  int cap = (148 * 8 + B - 1) / B;
  if (cap < 1) cap = 1;
  if (gx > cap) gx = cap;
  launch_dependent(muon_momentum_kernel, dim3(gx, B), dim3(256), 0, (cudaStream_t)stream, a);
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_scale_by_inv_norm(void* x, const float* sumsq, long long per, int B,
                                                float eps, void* stream) {
  if (per <= 0 || (per & 7) || B <= 0 || B > 65535) return -1;
  int gx = static_cast<int>((per / 8 + 255) / 256);
  int cap = (148 * 8 + B - 1) / B;
  if (cap < 1) cap = 1;
  if (gx > cap) gx = cap;
  launch_dependent(scale_by_inv_norm_kernel, dim3(gx, B), dim3(256), 0, (cudaStream_t)stream, (__nv_bfloat16*)x, sumsq,
                                                                         per, eps);
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_muon_apply(float* p, void* p_bf16, const void* o, long long n,
                                         float lr, float wd, void* stream) {
  if (n <= 0 || (n & 3)) return -1;
  launch_dependent(muon_apply_kernel, dim3(grid_1d(n / 4)), dim3(256), 0, (cudaStream_t)stream,
      p, (__nv_bfloat16*)p_bf16, (const __nv_bfloat16*)o, n, lr, wd);
  return (int)cudaGetLastError();
}
