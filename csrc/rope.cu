// Rotary embedding fused with per-head RMSNorm and the value-embedding blend.
//
// qkv_post (NanoChat order: RoPE first, then QK-norm; Examples/NanoChat/ModdedGPT.lean:301-327):
//   q' = rmsnorm(rope(q)), k' = rmsnorm(rope(k)), v' = (1-m) v + m ve
// on a packed [rows, 3, H, D] projection output, one warp per (row, head).  The rotation is the
// half-split form of cc/src/tyr.cpp:2823-2856: [x1, x2] -> [x1 c - x2 s, x1 s + x2 c] with
// cos/sin tables of shape [T, D/2] (position = row % T).
//
// rope_norm (generic, inference families): optional per-head RMSNorm with weight BEFORE the
// rotation (Laguna / Qwen order), partial rotary dimension, explicit position ids.
#include "common.cuh"

namespace tyr {

struct QkvPostArgs {
  const __nv_bfloat16* qkv;   // [rows, 3*H*D]
  const __nv_bfloat16* ve;    // [rows, H*D] or nullptr
  const float* mix;           // device scalar in (0,1) or nullptr
  const float* cosT;          // [T, D/2]
  const float* sinT;
  __nv_bfloat16* out;         // [rows, 3*H*D]
  int rows, T, H, D;
  float eps;
};

// D == 128 fast path: lane l owns x1[2l..2l+1] and x2[2l..2l+1].
__global__ void __launch_bounds__(256) qkv_post_fwd_kernel(QkvPostArgs a) {
  pdl_entry();
  const int lane = threadIdx.x & 31;
  const long long unit0 = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long units = static_cast<long long>(a.rows) * 3 * a.H;
  const long long stride = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const int half = a.D >> 1;
  const float mix = a.mix ? *a.mix : 0.f;
  for (long long u = unit0; u < units; u += stride) {
    const long long row = u / (3 * a.H);
    const int rem = static_cast<int>(u % (3 * a.H));
    const int which = rem / a.H;
    const int head = rem % a.H;
    const long long off = row * (3LL * a.H * a.D) + static_cast<long long>(which) * a.H * a.D +
                          static_cast<long long>(head) * a.D;
    const __nv_bfloat16* x = a.qkv + off;
    __nv_bfloat16* y = a.out + off;
    if (which == 2) {
      const __nv_bfloat16* ve = a.ve ? a.ve + row * (static_cast<long long>(a.H) * a.D) + head * a.D : nullptr;
      for (int i = lane * 2; i < a.D; i += 64) {
        float2 v = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + i));
        if (ve) {
          float2 e = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(ve + i));
          v.x = (1.f - mix) * v.x + mix * e.x;
          v.y = (1.f - mix) * v.y + mix * e.y;
        }
        *reinterpret_cast<uint32_t*>(y + i) = pack_bf16x2(v.x, v.y);
      }
      continue;
    }
    const int pos = static_cast<int>(row % a.T);
    const float* c = a.cosT + static_cast<long long>(pos) * half;
    const float* s = a.sinT + static_cast<long long>(pos) * half;
    float ss = 0.f;
    // two passes over <= D/64 register pairs; D <= 256 keeps this at 4 pairs per lane
    float r1[4][2], r2[4][2];
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int i = lane * 2 + n * 64;
      if (i >= half) continue;
      float2 x1 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + i));
      float2 x2 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + half + i));
      float2 cc = *reinterpret_cast<const float2*>(c + i);
      float2 sn = *reinterpret_cast<const float2*>(s + i);
      r1[n][0] = x1.x * cc.x - x2.x * sn.x;
      r1[n][1] = x1.y * cc.y - x2.y * sn.y;
      r2[n][0] = x1.x * sn.x + x2.x * cc.x;
      r2[n][1] = x1.y * sn.y + x2.y * cc.y;
      ss += r1[n][0] * r1[n][0] + r1[n][1] * r1[n][1] + r2[n][0] * r2[n][0] + r2[n][1] * r2[n][1];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / a.D + a.eps);
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int i = lane * 2 + n * 64;
      if (i >= half) continue;
      *reinterpret_cast<uint32_t*>(y + i) = pack_bf16x2(r1[n][0] * rstd, r1[n][1] * rstd);
      *reinterpret_cast<uint32_t*>(y + half + i) = pack_bf16x2(r2[n][0] * rstd, r2[n][1] * rstd);
    }
  }
}

struct QkvPostBwdArgs {
  const __nv_bfloat16* qkv;   // forward input
  const __nv_bfloat16* ve;
  const float* mix;
  const float* cosT;
  const float* sinT;
  const __nv_bfloat16* dy;    // [rows, 3*H*D] gradient of the forward output
  __nv_bfloat16* dqkv;        // [rows, 3*H*D]
  __nv_bfloat16* dve;         // [rows, H*D] or nullptr
  float* dmix;                // fp32 scalar, atomically accumulated (nullable)
  int rows, T, H, D;
  float eps;
};

__global__ void __launch_bounds__(256) qkv_post_bwd_kernel(QkvPostBwdArgs a) {
  pdl_entry();
  const int lane = threadIdx.x & 31;
  const int wid = threadIdx.x >> 5;
  const long long unit0 = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + wid;
  const long long units = static_cast<long long>(a.rows) * 3 * a.H;
  const long long stride = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const int half = a.D >> 1;
  const float mix = a.mix ? *a.mix : 0.f;
  float dmix_acc = 0.f;
  for (long long u = unit0; u < units; u += stride) {
    const long long row = u / (3 * a.H);
    const int rem = static_cast<int>(u % (3 * a.H));
    const int which = rem / a.H;
    const int head = rem % a.H;
    const long long off = row * (3LL * a.H * a.D) + static_cast<long long>(which) * a.H * a.D +
                          static_cast<long long>(head) * a.D;
    const __nv_bfloat16* x = a.qkv + off;
    const __nv_bfloat16* dy = a.dy + off;
    __nv_bfloat16* dx = a.dqkv + off;
    if (which == 2) {
      const long long voff = row * (static_cast<long long>(a.H) * a.D) + head * a.D;
      for (int i = lane * 2; i < a.D; i += 64) {
        float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dy + i));
        if (a.ve) {
          float2 v = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + i));
          float2 e = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(a.ve + voff + i));
          dmix_acc += g.x * (e.x - v.x) + g.y * (e.y - v.y);
          if (a.dve) *reinterpret_cast<uint32_t*>(a.dve + voff + i) = pack_bf16x2(mix * g.x, mix * g.y);
          g.x *= (1.f - mix);
          g.y *= (1.f - mix);
        }
        *reinterpret_cast<uint32_t*>(dx + i) = pack_bf16x2(g.x, g.y);
      }
      continue;
    }
    const int pos = static_cast<int>(row % a.T);
    const float* c = a.cosT + static_cast<long long>(pos) * half;
    const float* s = a.sinT + static_cast<long long>(pos) * half;
    float r1[4][2], r2[4][2], g1[4][2], g2[4][2];
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int i = lane * 2 + n * 64;
      if (i >= half) continue;
      float2 x1 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + i));
      float2 x2 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + half + i));
      float2 cc = *reinterpret_cast<const float2*>(c + i);
      float2 sn = *reinterpret_cast<const float2*>(s + i);
      float2 d1 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dy + i));
      float2 d2 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dy + half + i));
      r1[n][0] = x1.x * cc.x - x2.x * sn.x;
      r1[n][1] = x1.y * cc.y - x2.y * sn.y;
      r2[n][0] = x1.x * sn.x + x2.x * cc.x;
      r2[n][1] = x1.y * sn.y + x2.y * cc.y;
      g1[n][0] = d1.x; g1[n][1] = d1.y; g2[n][0] = d2.x; g2[n][1] = d2.y;
      ss += r1[n][0] * r1[n][0] + r1[n][1] * r1[n][1] + r2[n][0] * r2[n][0] + r2[n][1] * r2[n][1];
      dot += r1[n][0] * d1.x + r1[n][1] * d1.y + r2[n][0] * d2.x + r2[n][1] * d2.y;
    }
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    const float rstd = rsqrtf(ss / a.D + a.eps);
    const float coef = rstd * rstd * rstd * dot / a.D;
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int i = lane * 2 + n * 64;
      if (i >= half) continue;
      float2 cc = *reinterpret_cast<const float2*>(c + i);
      float2 sn = *reinterpret_cast<const float2*>(s + i);
      // gradient w.r.t. the rotated vector
      const float a10 = rstd * g1[n][0] - coef * r1[n][0];
      const float a11 = rstd * g1[n][1] - coef * r1[n][1];
      const float a20 = rstd * g2[n][0] - coef * r2[n][0];
      const float a21 = rstd * g2[n][1] - coef * r2[n][1];
      // transpose of the rotation
      *reinterpret_cast<uint32_t*>(dx + i) =
          pack_bf16x2(a10 * cc.x + a20 * sn.x, a11 * cc.y + a21 * sn.y);
      *reinterpret_cast<uint32_t*>(dx + half + i) =
          pack_bf16x2(-a10 * sn.x + a20 * cc.x, -a11 * sn.y + a21 * cc.y);
    }
  }
  if (a.dmix) {
    __shared__ float red[8];
    float v = warp_sum(dmix_acc);
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
      if (t != 0.f) atomicAdd(a.dmix, t);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// D == 128 fast path: 8 lanes per (row, head), 16-byte loads/stores; a warp covers 4 heads and a
// block walks the (row, head-group) units.  x1/x2 halves of a head are 128 B each, so every group
// of 8 lanes reads two fully coalesced 128-byte segments.
// ---------------------------------------------------------------------------------------------
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
__device__ __forceinline__ void ldf8(const float* p, float (&f)[8]) {
  float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ float group8_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}

__global__ void __launch_bounds__(256) qkv_post_fwd_d128_kernel(QkvPostArgs a) {
  pdl_entry();
  const int lane = threadIdx.x & 31;
  const int sub = lane >> 3;          // head within the group of 4
  const int ch = (lane & 7) * 8;      // channel offset inside a 64-wide half
  const int groups = (3 * a.H + 3) / 4;   // 4 (which, head) slots per warp step
  const long long units = static_cast<long long>(a.rows) * groups;
  const long long stride = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const float mix = a.mix ? *a.mix : 0.f;
  const int HD = a.H * 128;
  for (long long u = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); u < units;
       u += stride) {
    const long long row = u / groups;
    const int slot = static_cast<int>(u % groups) * 4 + sub;   // index into [3*H]
    const bool live = slot < 3 * a.H;
    const int which = live ? slot / a.H : 0;
    const int head = live ? slot % a.H : 0;
    const long long off = row * (3LL * HD) + static_cast<long long>(which) * HD + head * 128;
    float x1[8], x2[8];
    if (live) {
      ld8(a.qkv + off + ch, x1);
      ld8(a.qkv + off + 64 + ch, x2);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) x1[j] = x2[j] = 0.f;
    }
    if (which == 2) {
      if (live) {
        if (a.ve) {
          float e1[8], e2[8];
          const long long voff = row * HD + head * 128;
          ld8(a.ve + voff + ch, e1);
          ld8(a.ve + voff + 64 + ch, e2);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            x1[j] = (1.f - mix) * x1[j] + mix * e1[j];
            x2[j] = (1.f - mix) * x2[j] + mix * e2[j];
          }
        }
        st8(a.out + off + ch, x1);
        st8(a.out + off + 64 + ch, x2);
      }
      // the q/k lanes of this warp still run the shuffles below; v lanes join them with zeros
    }
    const int pos = static_cast<int>(row % a.T);
    float c[8], sn[8], r1[8], r2[8];
    ldf8(a.cosT + static_cast<long long>(pos) * 64 + ch, c);
    ldf8(a.sinT + static_cast<long long>(pos) * 64 + ch, sn);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      r1[j] = x1[j] * c[j] - x2[j] * sn[j];
      r2[j] = x1[j] * sn[j] + x2[j] * c[j];
      ss += r1[j] * r1[j] + r2[j] * r2[j];
    }
    ss = group8_sum(ss);
    if (live && which != 2) {
      const float rstd = rsqrtf(ss * (1.f / 128.f) + a.eps);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        r1[j] *= rstd;
        r2[j] *= rstd;
      }
      st8(a.out + off + ch, r1);
      st8(a.out + off + 64 + ch, r2);
    }
  }
}

__global__ void __launch_bounds__(256) qkv_post_bwd_d128_kernel(QkvPostBwdArgs a) {
  pdl_entry();
  const int lane = threadIdx.x & 31;
  const int wid = threadIdx.x >> 5;
  const int sub = lane >> 3;
  const int ch = (lane & 7) * 8;
  const int groups = (3 * a.H + 3) / 4;
  const long long units = static_cast<long long>(a.rows) * groups;
  const long long stride = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const float mix = a.mix ? *a.mix : 0.f;
  const int HD = a.H * 128;
  float dmix_acc = 0.f;
  for (long long u = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + wid; u < units; u += stride) {
    const long long row = u / groups;
    const int slot = static_cast<int>(u % groups) * 4 + sub;
    const bool live = slot < 3 * a.H;
    const int which = live ? slot / a.H : 0;
    const int head = live ? slot % a.H : 0;
    const long long off = row * (3LL * HD) + static_cast<long long>(which) * HD + head * 128;
    float x1[8], x2[8], g1[8], g2[8];
    if (live) {
      ld8(a.qkv + off + ch, x1);
      ld8(a.qkv + off + 64 + ch, x2);
      ld8(a.dy + off + ch, g1);
      ld8(a.dy + off + 64 + ch, g2);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) x1[j] = x2[j] = g1[j] = g2[j] = 0.f;
    }
    if (live && which == 2) {
      if (a.ve) {
        float e1[8], e2[8];
        const long long voff = row * HD + head * 128;
        ld8(a.ve + voff + ch, e1);
        ld8(a.ve + voff + 64 + ch, e2);
        float d1[8], d2[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dmix_acc += g1[j] * (e1[j] - x1[j]) + g2[j] * (e2[j] - x2[j]);
          d1[j] = mix * g1[j];
          d2[j] = mix * g2[j];
          g1[j] *= (1.f - mix);
          g2[j] *= (1.f - mix);
        }
        if (a.dve) {
          st8(a.dve + voff + ch, d1);
          st8(a.dve + voff + 64 + ch, d2);
        }
      }
      st8(a.dqkv + off + ch, g1);
      st8(a.dqkv + off + 64 + ch, g2);
    }
    const int pos = static_cast<int>(row % a.T);
    float c[8], sn[8], r1[8], r2[8];
    ldf8(a.cosT + static_cast<long long>(pos) * 64 + ch, c);
    ldf8(a.sinT + static_cast<long long>(pos) * 64 + ch, sn);
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      r1[j] = x1[j] * c[j] - x2[j] * sn[j];
      r2[j] = x1[j] * sn[j] + x2[j] * c[j];
      ss += r1[j] * r1[j] + r2[j] * r2[j];
      dot += r1[j] * g1[j] + r2[j] * g2[j];
    }
    ss = group8_sum(ss);
    dot = group8_sum(dot);
    if (live && which != 2) {
      const float rstd = rsqrtf(ss * (1.f / 128.f) + a.eps);
      const float coef = rstd * rstd * rstd * dot * (1.f / 128.f);
      float o1[8], o2[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float a1 = rstd * g1[j] - coef * r1[j];
        const float a2 = rstd * g2[j] - coef * r2[j];
        o1[j] = a1 * c[j] + a2 * sn[j];
        o2[j] = -a1 * sn[j] + a2 * c[j];
      }
      st8(a.dqkv + off + ch, o1);
      st8(a.dqkv + off + 64 + ch, o2);
    }
  }
  if (a.dmix) {
    __shared__ float red[8];
    float v = warp_sum(dmix_acc);
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
      if (t != 0.f) atomicAdd(a.dmix, t);
    }
  }
}

// Generic rope for the inference families: x [rows, H, D] (row stride given), optional RMSNorm
// with weight over the head BEFORE rotation, rotary applied to the first `rot` channels of each
// head (half-split inside that span), position ids explicit (nullptr = row % T).
struct RopeNormArgs {
  const __nv_bfloat16* x;
  __nv_bfloat16* y;
  const __nv_bfloat16* w;      // [D] norm weight (nullable = no norm)
  const float* cosT;           // [P, rot/2]
  const float* sinT;
  const int* pos;              // [rows] (nullable)
  long long row_stride;        // elements between rows of x
  long long y_row_stride;      // elements between rows of y
  int rows, T, H, D, rot;
  float eps;
  int one_plus_w;
};

__global__ void __launch_bounds__(256) rope_norm_kernel(RopeNormArgs a) {
  pdl_entry();
  const int lane = threadIdx.x & 31;
  const long long unit0 = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long units = static_cast<long long>(a.rows) * a.H;
  const long long stride = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const int hr = a.rot >> 1;
  for (long long u = unit0; u < units; u += stride) {
    const long long row = u / a.H;
    const int head = static_cast<int>(u % a.H);
    const __nv_bfloat16* x = a.x + row * a.row_stride + static_cast<long long>(head) * a.D;
    __nv_bfloat16* y = a.y + row * a.y_row_stride + static_cast<long long>(head) * a.D;
    float rstd = 1.f;
    if (a.w) {
      float ss = 0.f;
      for (int i = lane; i < a.D; i += 32) {
        float v = __bfloat162float(x[i]);
        ss += v * v;
      }
      ss = warp_sum(ss);
      rstd = rsqrtf(ss / a.D + a.eps);
    }
    int pos = a.pos ? a.pos[row] : static_cast<int>(row % a.T);
    if (!TYR_INDEX_OK(pos, a.T, 21)) pos = 0;      // checked builds record a position outside the tables and rotate by position 0
    const float* c = a.cosT + static_cast<long long>(pos) * hr;
    const float* s = a.sinT + static_cast<long long>(pos) * hr;
    auto nrm = [&](int i) -> float {
      float v = __bfloat162float(x[i]);
      if (a.w) {
        float w = __bfloat162float(a.w[i]);
        if (a.one_plus_w) w += 1.f;
        // normalised value is rounded to bf16 before the weight multiply, as the HF models do
        v = __bfloat162float(__float2bfloat16(v * rstd)) * w;
        v = __bfloat162float(__float2bfloat16(v));
      }
      return v;
    };
    for (int i = lane; i < hr; i += 32) {
      const float x1 = nrm(i), x2 = nrm(i + hr);
      y[i] = __float2bfloat16(x1 * c[i] - x2 * s[i]);
      y[i + hr] = __float2bfloat16(x1 * s[i] + x2 * c[i]);
    }
    for (int i = a.rot + lane; i < a.D; i += 32) y[i] = __float2bfloat16(nrm(i));
  }
}

static int grid_for_units(long long units, int warps) {
  long long blocks = (units + warps - 1) / warps;
  const long long cap = 148LL * 32;
  return static_cast<int>(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

}  // namespace tyr

using namespace tyr;

extern "C" TYR_EXPORT int tyr_qkv_post_fwd(const void* qkv, const void* ve, const float* mix,
                                           const float* cosT, const float* sinT, void* out,
                                           int rows, int T, int H, int D, float eps, void* stream) {
  if (D % 128 != 0 && D != 64) return -1;
  if (D > 512) return -2;
  QkvPostArgs a{(const __nv_bfloat16*)qkv, (const __nv_bfloat16*)ve, mix, cosT, sinT,
                (__nv_bfloat16*)out, rows, T, H, D, eps};
  if (D == 128) {
    const long long units = static_cast<long long>(rows) * ((3 * H + 3) / 4);
    launch_dependent(qkv_post_fwd_d128_kernel, dim3(grid_for_units(units, 8)), dim3(256), 0, (cudaStream_t)stream, a);
    return (int)cudaGetLastError();
  }
  launch_dependent(qkv_post_fwd_kernel, dim3(grid_for_units(3LL * rows * H, 8)), dim3(256), 0, (cudaStream_t)stream, a);
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_qkv_post_bwd(const void* qkv, const void* ve, const float* mix,
                                           const float* cosT, const float* sinT, const void* dy,
                                           void* dqkv, void* dve, float* dmix, int rows, int T,
                                           int H, int D, float eps, void* stream) {
  if (D % 128 != 0 && D != 64) return -1;
  if (D > 512) return -2;
  QkvPostBwdArgs a{(const __nv_bfloat16*)qkv, (const __nv_bfloat16*)ve, mix, cosT, sinT,
                   (const __nv_bfloat16*)dy, (__nv_bfloat16*)dqkv, (__nv_bfloat16*)dve, dmix,
                   rows, T, H, D, eps};
  if (D == 128) {
    const long long units = static_cast<long long>(rows) * ((3 * H + 3) / 4);
    launch_dependent(qkv_post_bwd_d128_kernel, dim3(grid_for_units(units, 8)), dim3(256), 0, (cudaStream_t)stream, a);
    return (int)cudaGetLastError();
  }
  launch_dependent(qkv_post_bwd_kernel, dim3(grid_for_units(3LL * rows * H, 8)), dim3(256), 0, (cudaStream_t)stream, a);
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_rope_norm(const void* x, void* y, const void* w, const float* cosT,
                                        const float* sinT, const int* pos, long long row_stride,
                                        long long y_row_stride, int rows, int T, int H, int D, int rot, float eps,
                                        int one_plus_w, void* stream) {
  if (rot > D || (rot & 1)) return -1;
  RopeNormArgs a{(const __nv_bfloat16*)x, (__nv_bfloat16*)y, (const __nv_bfloat16*)w, cosT, sinT,
                 pos, row_stride, y_row_stride, rows, T, H, D, rot, eps, one_plus_w};
  return (int)launch_dependent(rope_norm_kernel, dim3(grid_for_units(1LL * rows * H, 8)), dim3(256), 0, (cudaStream_t)stream, a);
}

TYR_DEFINE_BOUNDS_STATUS(rope)
