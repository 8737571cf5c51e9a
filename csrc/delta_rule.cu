// Gated delta rule, single-token recurrent step (Qwen3.5 GatedDeltaNet decode).
//
// Per (batch, value head) the state S is [dk, dv] fp32.  One step is
//   S <- exp(g) * S;  kv = S^T k;  delta = beta * (v - kv);  S <- S + k delta^T;  out = S^T q
// with q, k L2-normalised over dk and q scaled by dk^-1/2.  The step is bound by one read and one
// write of S (2 * dk * dv * 4 bytes); the kernel below does exactly that: each thread owns one
// state column, keeps its dk values in registers between the two reductions, and the CTA's accesses
// to a state row are contiguous.  Semantics follow cc/src/tyr_qwen35.cpp:121-170 of the reference.
#include "common.cuh"

namespace tyr {

template <int DK>
__global__ void __launch_bounds__(128)
gdr_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                  const __nv_bfloat16* __restrict__ v, const float* __restrict__ g,
                  const float* __restrict__ beta, float* __restrict__ state, __nv_bfloat16* __restrict__ out,
                  int Hk, int Hv, int dv, long long q_bstride, long long v_bstride) {
  __shared__ float sq[DK], sk[DK];
  __shared__ float red[2][4];
  const int bh = blockIdx.x;
  const int b = bh / Hv, hv = bh % Hv;
  const int hk = hv / (Hv / Hk);
  const int tid = threadIdx.x;
  const __nv_bfloat16* qp = q + b * q_bstride + static_cast<long long>(hk) * DK;
  const __nv_bfloat16* kp = k + b * q_bstride + static_cast<long long>(hk) * DK;
  // L2 norms of q and k (DK <= 128 * ceil: each thread takes DK/128 elements)
  float qs = 0.f, ks = 0.f;
  for (int i = tid; i < DK; i += 128) {
    const float a = __bfloat162float(qp[i]), c = __bfloat162float(kp[i]);
    sq[i] = a; sk[i] = c;
    qs += a * a; ks += c * c;
  }
  qs = warp_sum(qs); ks = warp_sum(ks);
  if ((tid & 31) == 0) { red[0][tid >> 5] = qs; red[1][tid >> 5] = ks; }
  __syncthreads();
  qs = red[0][0] + red[0][1] + red[0][2] + red[0][3];
  ks = red[1][0] + red[1][1] + red[1][2] + red[1][3];
  const float qn = rsqrtf(qs + 1e-6f) * rsqrtf(static_cast<float>(DK));
  const float kn = rsqrtf(ks + 1e-6f);
  const float decay = __expf(g[bh]);
  const float bt = beta[bh];
  float* S = state + static_cast<long long>(bh) * DK * dv;
  for (int col = blockIdx.y * 128 + tid; col < dv; col += gridDim.y * 128) {
    float s[DK];
    float kv = 0.f;
#pragma unroll
    for (int r = 0; r < DK; ++r) {
      s[r] = S[static_cast<long long>(r) * dv + col] * decay;
      kv += s[r] * sk[r];
    }
    kv *= kn;
    const float vt = __bfloat162float(v[b * v_bstride + static_cast<long long>(hv) * dv + col]);
    const float delta = (vt - kv) * bt * kn;       // k enters normalised: k_hat = kn * k
    float o = 0.f;
#pragma unroll
    for (int r = 0; r < DK; ++r) {
      s[r] += sk[r] * delta;
      o += s[r] * sq[r];
      S[static_cast<long long>(r) * dv + col] = s[r];
    }
    out[(static_cast<long long>(bh)) * dv + col] = __float2bfloat16(o * qn);
  }
}

}  // namespace tyr

// q, k: bf16 [B, Hk, dk] (rows may be strided by q_bstride elements between batches); v: bf16 [B, Hv, dv]
// (v_bstride); g, beta: fp32 [B, Hv]; state: fp32 [B, Hv, dk, dv] updated in place; out: bf16 [B, Hv, dv].
extern "C" TYR_EXPORT int tyr_gdr_decode(const void* q, const void* k, const void* v, const float* g, const float* beta,
                                         float* state, void* out, int B, int Hk, int Hv, int dk, int dv,
                                         long long q_bstride, long long v_bstride, void* stream) {
  using namespace tyr;
  if (B <= 0 || Hk <= 0 || Hv <= 0 || Hv % Hk != 0 || dv <= 0) return -1;
  dim3 grid(B * Hv, (dv + 127) / 128);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  auto* qq = reinterpret_cast<const __nv_bfloat16*>(q);
  auto* kk = reinterpret_cast<const __nv_bfloat16*>(k);
  auto* vv = reinterpret_cast<const __nv_bfloat16*>(v);
  auto* oo = reinterpret_cast<__nv_bfloat16*>(out);
  if (dk == 128)
    gdr_decode_kernel<128><<<grid, 128, 0, st>>>(qq, kk, vv, g, beta, state, oo, Hk, Hv, dv, q_bstride, v_bstride);
  else if (dk == 64)
    gdr_decode_kernel<64><<<grid, 128, 0, st>>>(qq, kk, vv, g, beta, state, oo, Hk, Hv, dv, q_bstride, v_bstride);
  else
    return -2;
  return static_cast<int>(cudaGetLastError());
}
