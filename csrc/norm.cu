// RMSNorm family (memory-bound, one warp per row, fp32 accumulation).
//
//  * lincomb_rmsnorm: out = sum_i s_i * t_i (up to 4 bf16 inputs, fp32 device scalars) and
//    normed = out * rsqrt(mean(out^2) + eps) in ONE pass over the inputs.  This is the residual
//    stream update of the modded-nanogpt block (x = lam_x*x + lam_0*x0, x += lam*attn, ...)
//    fused with the pre-norm that follows it; the reference issues one broadcast-multiply, one
//    add and 5-7 norm kernels for the same thing (Examples/NanoChat/ModdedGPT.lean:449-452,
//    586-611; Tyr/Typed/Neural.lean:38-43).
//  * its backward: grads of every input and of every scalar from (d_out, d_normed).
//  * rmsnorm_weighted: y = x * rstd * w with w either plain, "(1 + w)" zero-centred (Qwen3.5) or
//    absent, optional SiLU(z) gate (GatedDeltaNet output norm) and optional residual add
//    (cc/src/tyr.cpp:3766-3772, Tyr/Model/Qwen35/Model.lean RMSNorm variants).
#include "common.cuh"

namespace tyr {

struct LincombArgs {
  const __nv_bfloat16* t[4];
  const float* scal;   // device pointer to n_in floats (nullptr = all ones)
  int n_in;
  int rows, D;
  float eps;
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z),
         d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

template <int NIN>
__global__ void __launch_bounds__(256)
lincomb_rmsnorm_fwd_kernel(LincombArgs a, __nv_bfloat16* __restrict__ out,
                           __nv_bfloat16* __restrict__ normed) {
  pdl_entry();
  const int warps = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  float s[NIN];
#pragma unroll
  for (int i = 0; i < NIN; ++i) s[i] = a.scal ? a.scal[i] : 1.f;
  const int nvec = a.D >> 3;
  for (long long row = blockIdx.x * warps + (threadIdx.x >> 5); row < a.rows;
       row += static_cast<long long>(gridDim.x) * warps) {
    const long long base = row * a.D;
    float ss = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
      for (int i = 0; i < NIN; ++i) {
        float f[8];
        load8(a.t[i] + base + v * 8, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += s[i] * f[j];
      }
      if (out) {
        store8(out + base + v * 8, acc);
        // normalise the value that is actually stored (bf16-rounded) so that the backward,
        // which only sees the stored tensor, recomputes the same statistics
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = __bfloat162float(__float2bfloat16(acc[j]));
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += acc[j] * acc[j];
    }
    if (normed == nullptr) continue;
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / a.D + a.eps);
    for (int v = lane; v < nvec; v += 32) {
      float acc[8];
      if (out) {
        load8(out + base + v * 8, acc);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
        for (int i = 0; i < NIN; ++i) {
          float f[8];
          load8(a.t[i] + base + v * 8, f);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += s[i] * f[j];
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] *= rstd;
      store8(normed + base + v * 8, acc);
    }
  }
}

struct LincombBwdArgs {
  const __nv_bfloat16* t[4];      // forward inputs (needed for the scalar gradients)
  __nv_bfloat16* dt[4];           // gradient outputs (nullable)
  const float* scal;
  float* dscal;                   // fp32[n_in], accumulated with atomics (nullable)
  const __nv_bfloat16* out;       // forward combined output (the tensor that was normalised)
  const __nv_bfloat16* d_out;     // nullable
  const __nv_bfloat16* d_normed;  // nullable
  int n_in, rows, D;
  float eps;
};

template <int NIN>
__global__ void __launch_bounds__(256)
lincomb_rmsnorm_bwd_kernel(LincombBwdArgs a) {
  pdl_entry();
  const int warps = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int wid = threadIdx.x >> 5;
  float s[NIN], ds[NIN];
#pragma unroll
  for (int i = 0; i < NIN; ++i) {
    s[i] = a.scal ? a.scal[i] : 1.f;
    ds[i] = 0.f;
  }
  const int nvec = a.D >> 3;
  for (long long row = blockIdx.x * warps + wid; row < a.rows;
       row += static_cast<long long>(gridDim.x) * warps) {
    const long long base = row * a.D;
    float rstd = 0.f, coef = 0.f;
    if (a.d_normed) {
      float ss = 0.f, dot = 0.f;
      for (int v = lane; v < nvec; v += 32) {
        float o[8], dn[8];
        load8(a.out + base + v * 8, o);
        load8(a.d_normed + base + v * 8, dn);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          ss += o[j] * o[j];
          dot += o[j] * dn[j];
        }
      }
      ss = warp_sum(ss);
      dot = warp_sum(dot);
      rstd = rsqrtf(ss / a.D + a.eps);
      coef = rstd * rstd * rstd * dot / a.D;
    }
    for (int v = lane; v < nvec; v += 32) {
      float g[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = 0.f;
      if (a.d_out) load8(a.d_out + base + v * 8, g);
      if (a.d_normed) {
        float o[8], dn[8];
        load8(a.out + base + v * 8, o);
        load8(a.d_normed + base + v * 8, dn);
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] += rstd * dn[j] - coef * o[j];
      }
#pragma unroll
      for (int i = 0; i < NIN; ++i) {
        if (a.dscal) {
          float f[8];
          load8(a.t[i] + base + v * 8, f);
#pragma unroll
          for (int j = 0; j < 8; ++j) ds[i] += g[j] * f[j];
        }
        if (a.dt[i]) {
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = s[i] * g[j];
          store8(a.dt[i] + base + v * 8, o);
        }
      }
    }
  }
  if (a.dscal) {
    __shared__ float red[4][8];
#pragma unroll
    for (int i = 0; i < NIN; ++i) {
      float v = warp_sum(ds[i]);
      if (lane == 0) red[i][wid] = v;
    }
    __syncthreads();
    if (threadIdx.x < NIN) {
      float v = 0.f;
      for (int w = 0; w < warps; ++w) v += red[threadIdx.x][w];
      atomicAdd(a.dscal + threadIdx.x, v);
    }
  }
}

// y = x * rstd * weight-ish (+ optional gate), used by the inference model families.
struct RmsWArgs {
  const __nv_bfloat16* x;
  const __nv_bfloat16* w;       // [D] (nullable)
  const __nv_bfloat16* gate;    // [rows, D] (nullable): y *= silu(gate)
  const __nv_bfloat16* resid;   // [rows, D] (nullable): x := x + resid before the norm
  __nv_bfloat16* resid_out;     // receives x + resid (nullable)
  __nv_bfloat16* y;
  int rows, D;
  float eps;
  int one_plus_w;               // weight = 1 + w
};

__global__ void __launch_bounds__(256) rmsnorm_weighted_kernel(RmsWArgs a) {
  pdl_entry();
  const int warps = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = a.D >> 3;
  for (long long row = blockIdx.x * warps + (threadIdx.x >> 5); row < a.rows;
       row += static_cast<long long>(gridDim.x) * warps) {
    const long long base = row * a.D;
    float ss = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      float f[8];
      load8(a.x + base + v * 8, f);
      if (a.resid) {
        float r[8];
        load8(a.resid + base + v * 8, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += r[j];
        if (a.resid_out) {
          store8(a.resid_out + base + v * 8, f);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(__float2bfloat16(f[j]));
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / a.D + a.eps);
    for (int v = lane; v < nvec; v += 32) {
      float f[8];
      if (a.resid && a.resid_out) {
        load8(a.resid_out + base + v * 8, f);
      } else {
        load8(a.x + base + v * 8, f);
        if (a.resid) {
          float r[8];
          load8(a.resid + base + v * 8, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] += r[j];
        }
      }
      float w[8];
      if (a.w) {
        load8(a.w + v * 8, w);
        if (a.one_plus_w) {
#pragma unroll
          for (int j = 0; j < 8; ++j) w[j] += 1.f;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) w[j] = 1.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * w[j];
      if (a.gate) {
        float g[8];
        load8(a.gate + base + v * 8, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] *= g[j] / (1.f + __expf(-g[j]));
      }
      store8(a.y + base + v * 8, f);
    }
  }
}

// Decode-sized inputs (a few dozen rows of a few thousand channels): one CTA per row, the row stays in registers between
// the sum of squares and the scaled write, so every operand is read once and the kernel is one load latency deep instead
// of two loops of eight dependent iterations per warp (8 - 9 us per launch with one warp per row, measured in a decode step).
constexpr int kRowVecs = 4;     // 16-byte vectors per thread: D <= 256 * 4 * 8

__global__ void __launch_bounds__(256) rmsnorm_weighted_row_kernel(RmsWArgs a) {
  pdl_entry();
  __shared__ float red[8];
  const int tid = threadIdx.x;
  const int nvec = a.D >> 3;
  const long long base = static_cast<long long>(blockIdx.x) * a.D;
  float f[kRowVecs][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kRowVecs; ++j) {
    const int v = tid + j * 256;
    if (v < nvec) {
      load8(a.x + base + v * 8, f[j]);
      if (a.resid) {
        float r[8];
        load8(a.resid + base + v * 8, r);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[j][e] += r[e];
        if (a.resid_out) {
          store8(a.resid_out + base + v * 8, f[j]);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[j][e] = __bfloat162float(__float2bfloat16(f[j][e]));
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += f[j][e] * f[j][e];
    }
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += (i < (blockDim.x >> 5)) ? red[i] : 0.f;
  const float rstd = rsqrtf(tot / a.D + a.eps);
#pragma unroll
  for (int j = 0; j < kRowVecs; ++j) {
    const int v = tid + j * 256;
    if (v < nvec) {
      float w[8];
      if (a.w) {
        load8(a.w + v * 8, w);
        if (a.one_plus_w) {
#pragma unroll
          for (int e = 0; e < 8; ++e) w[e] += 1.f;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) w[e] = 1.f;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) f[j][e] = f[j][e] * rstd * w[e];
      if (a.gate) {
        float g[8];
        load8(a.gate + base + v * 8, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[j][e] *= g[e] / (1.f + __expf(-g[e]));
      }
      store8(a.y + base + v * 8, f[j]);
    }
  }
}

static int grid_for_rows(long long rows, int warps_per_block) {
  long long blocks = (rows + warps_per_block - 1) / warps_per_block;
  const long long cap = 148LL * 16;
  return static_cast<int>(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

}  // namespace tyr

using namespace tyr;

extern "C" TYR_EXPORT int tyr_lincomb_rmsnorm_fwd(const void* t0, const void* t1, const void* t2,
                                                  const void* t3, const float* scal, int n_in,
                                                  int rows, int D, void* out, void* normed,
                                                  float eps, void* stream) {
  if (n_in < 1 || n_in > 4 || (D & 7) || rows <= 0) return -1;
  LincombArgs a;
  a.t[0] = (const __nv_bfloat16*)t0; a.t[1] = (const __nv_bfloat16*)t1;
  a.t[2] = (const __nv_bfloat16*)t2; a.t[3] = (const __nv_bfloat16*)t3;
  a.scal = scal; a.n_in = n_in; a.rows = rows; a.D = D; a.eps = eps;
  const int grid = grid_for_rows(rows, 8);
  cudaStream_t st = (cudaStream_t)stream;
  auto o = (__nv_bfloat16*)out;
  auto n = (__nv_bfloat16*)normed;
  switch (n_in) {
    case 1: launch_dependent(lincomb_rmsnorm_fwd_kernel<1>, dim3(grid), dim3(256), 0, st, a, o, n); break;
    case 2: launch_dependent(lincomb_rmsnorm_fwd_kernel<2>, dim3(grid), dim3(256), 0, st, a, o, n); break;
    case 3: launch_dependent(lincomb_rmsnorm_fwd_kernel<3>, dim3(grid), dim3(256), 0, st, a, o, n); break;
    default: launch_dependent(lincomb_rmsnorm_fwd_kernel<4>, dim3(grid), dim3(256), 0, st, a, o, n); break;
  }
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_lincomb_rmsnorm_bwd(const void* const* t, void* const* dt,
                                                  const float* scal, float* dscal,
                                                  const void* out, const void* d_out,
                                                  const void* d_normed, int n_in, int rows, int D,
                                                  float eps, void* stream) {
  if (n_in < 1 || n_in > 4 || (D & 7) || rows <= 0) return -1;
  LincombBwdArgs a;
  for (int i = 0; i < 4; ++i) {
    a.t[i] = i < n_in ? (const __nv_bfloat16*)t[i] : nullptr;
    a.dt[i] = i < n_in ? (__nv_bfloat16*)dt[i] : nullptr;
  }
  a.scal = scal; a.dscal = dscal;
  a.out = (const __nv_bfloat16*)out;
  a.d_out = (const __nv_bfloat16*)d_out;
  a.d_normed = (const __nv_bfloat16*)d_normed;
  a.n_in = n_in; a.rows = rows; a.D = D; a.eps = eps;
  const int grid = grid_for_rows(rows, 8);
  cudaStream_t st = (cudaStream_t)stream;
  switch (n_in) {
    case 1: launch_dependent(lincomb_rmsnorm_bwd_kernel<1>, dim3(grid), dim3(256), 0, st, a); break;
    case 2: launch_dependent(lincomb_rmsnorm_bwd_kernel<2>, dim3(grid), dim3(256), 0, st, a); break;
    case 3: launch_dependent(lincomb_rmsnorm_bwd_kernel<3>, dim3(grid), dim3(256), 0, st, a); break;
    default: launch_dependent(lincomb_rmsnorm_bwd_kernel<4>, dim3(grid), dim3(256), 0, st, a); break;
  }
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_rmsnorm_weighted(const void* x, const void* w, const void* gate,
                                               const void* resid, void* resid_out, void* y,
                                               int rows, int D, float eps, int one_plus_w,
                                               void* stream) {
  if ((D & 7) || rows <= 0) return -1;
  RmsWArgs a;
  a.x = (const __nv_bfloat16*)x; a.w = (const __nv_bfloat16*)w;
  a.gate = (const __nv_bfloat16*)gate; a.resid = (const __nv_bfloat16*)resid;
  a.resid_out = (__nv_bfloat16*)resid_out; a.y = (__nv_bfloat16*)y;
  a.rows = rows; a.D = D; a.eps = eps; a.one_plus_w = one_plus_w;
  if (rows <= 2048 && D >= 1024 && D <= 256 * kRowVecs * 8)
    return (int)launch_dependent(rmsnorm_weighted_row_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)stream, a);
  return (int)launch_dependent(rmsnorm_weighted_kernel, dim3(grid_for_rows(rows, 8)), dim3(256), 0, (cudaStream_t)stream, a);
}
