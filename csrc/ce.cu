// Soft-capped cross-entropy over a chunk of bf16 logits, forward and gradient in one kernel.
//
//   z = cap * tanh(l / cap)                 (cap <= 0 disables the soft cap)
//   loss_row = logsumexp(z) - z[target]
//   dl = gscale * (softmax(z) - onehot) * (1 - tanh^2(l / cap))      written IN PLACE over l
//
// The caller produces the logits chunk by chunk (rows x vocab) with the GEMM, runs this kernel,
// and immediately feeds `dl` to the two gradient GEMMs, so the full [tokens, vocab] fp32 logits
// tensor the reference materialises (linear -> softcap ops -> cross_entropy with a host-side
// label check, cc/src/tyr.cpp:2769-2773, 971-993, 2063-2072) never exists.
// Out-of-range targets contribute zero loss / zero gradient and are counted in `bad_count`
// (no host synchronisation).  target == ignore_index is skipped silently.
#include "common.cuh"

namespace tyr {

struct CeArgs {
  __nv_bfloat16* logits;     // [rows, ld] in: logits, out: gradient
  const long long* targets;  // [rows]
  float* loss_rows;          // [rows]
  int* bad_count;            // nullable
  int rows, V;
  long long ld;
  float cap, gscale;
  const float* gscale_dev;   // optional device multiplier applied on top of gscale
  long long ignore_index;
  int write_grad;
};

__device__ __forceinline__ float softcap(float l, float cap, float inv_cap) {
  return cap > 0.f ? cap * tanhf(l * inv_cap) : l;
}

__global__ void __launch_bounds__(512) softcap_ce_kernel(CeArgs a) {
  pdl_entry();
  __shared__ float red_m[16], red_s[16];
  __shared__ float sh_m, sh_lse;
  const int tid = threadIdx.x;
  const int lane = tid & 31, wid = tid >> 5, nw = blockDim.x >> 5;
  const float inv_cap = a.cap > 0.f ? 1.f / a.cap : 0.f;
  for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
    __nv_bfloat16* l = a.logits + static_cast<long long>(row) * a.ld;
    // pass 1: online max / sum
    float m = -INFINITY, s = 0.f;
    for (int v = tid * 8; v < a.V; v += blockDim.x * 8) {
      uint4 u = *reinterpret_cast<const uint4*>(l + v);
      float2 p[4] = {unpack_bf16x2(u.x), unpack_bf16x2(u.y), unpack_bf16x2(u.z), unpack_bf16x2(u.w)};
      float z[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        z[2 * j] = softcap(p[j].x, a.cap, inv_cap);
        z[2 * j + 1] = softcap(p[j].y, a.cap, inv_cap);
      }
      float mx = m;
#pragma unroll
      for (int j = 0; j < 8; ++j) mx = fmaxf(mx, z[j]);
      float acc = s * __expf(m - mx);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += __expf(z[j] - mx);
      m = mx;
      s = acc;
    }
    // warp then block combine of (m, s)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float m2 = __shfl_xor_sync(0xffffffffu, m, o);
      float s2 = __shfl_xor_sync(0xffffffffu, s, o);
      float mx = fmaxf(m, m2);
      s = (m == -INFINITY ? 0.f : s * __expf(m - mx)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mx));
      m = mx;
    }
    if (lane == 0) {
      red_m[wid] = m;
      red_s[wid] = s;
    }
    __syncthreads();
    if (wid == 0) {
      float mm = lane < nw ? red_m[lane] : -INFINITY;
      float sv = lane < nw ? red_s[lane] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        float m2 = __shfl_xor_sync(0xffffffffu, mm, o);
        float s2 = __shfl_xor_sync(0xffffffffu, sv, o);
        float mx = fmaxf(mm, m2);
        sv = (mm == -INFINITY ? 0.f : sv * __expf(mm - mx)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mx));
        mm = mx;
      }
      if (lane == 0) {
        sh_m = mm;
        sh_lse = mm + __logf(sv);
      }
    }
    __syncthreads();
    const float lse = sh_lse;
    const long long t = a.targets[row];
    const bool ignored = (t == a.ignore_index);
    const bool valid = !ignored && t >= 0 && t < a.V;
    if (tid == 0) {
      float loss = 0.f;
      if (valid) loss = lse - softcap(__bfloat162float(l[t]), a.cap, inv_cap);
      else if (!ignored && a.bad_count) atomicAdd(a.bad_count, 1);
      a.loss_rows[row] = loss;
    }
    if (a.write_grad) {
      __syncthreads();  // l[t] read above must precede the in-place overwrite
      const float g = valid ? a.gscale * (a.gscale_dev ? *a.gscale_dev : 1.f) : 0.f;
      for (int v = tid * 8; v < a.V; v += blockDim.x * 8) {
        uint4 u = *reinterpret_cast<const uint4*>(l + v);
        float2 p[4] = {unpack_bf16x2(u.x), unpack_bf16x2(u.y), unpack_bf16x2(u.z), unpack_bf16x2(u.w)};
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float lv = (j & 1) ? p[j >> 1].y : p[j >> 1].x;
          float z, dz = 1.f;
          if (a.cap > 0.f) {
            const float th = tanhf(lv * inv_cap);
            z = a.cap * th;
            dz = 1.f - th * th;
          } else {
            z = lv;
          }
          float pr = __expf(z - lse);
          if (v + j == t) pr -= 1.f;
          o[j] = g * pr * dz;
        }
        uint4 w;
        w.x = pack_bf16x2(o[0], o[1]); w.y = pack_bf16x2(o[2], o[3]);
        w.z = pack_bf16x2(o[4], o[5]); w.w = pack_bf16x2(o[6], o[7]);
        *reinterpret_cast<uint4*>(l + v) = w;
      }
    }
    __syncthreads();
  }
}

}  // namespace tyr

using namespace tyr;

extern "C" TYR_EXPORT int tyr_softcap_ce(void* logits, const long long* targets, float* loss_rows,
                                         int* bad_count, int rows, int V, long long ld, float cap,
                                         float gscale, const float* gscale_dev,
                                         long long ignore_index, int write_grad, void* stream) {
  if ((V & 7) || (ld & 7) || rows <= 0) return -1;
  CeArgs a{(__nv_bfloat16*)logits, targets, loss_rows, bad_count, rows, V, ld, cap, gscale,
           gscale_dev, ignore_index, write_grad};
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  launch_dependent(softcap_ce_kernel, dim3(grid), dim3(512), 0, (cudaStream_t)stream, a);
  return (int)cudaGetLastError();
}
