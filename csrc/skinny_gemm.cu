// y[M, N] = x[M, K] @ W[N, K]^T (+ bias) for decode-sized M (1..32 rows): a weight-streaming kernel.  The product is bound
// by reading W once from HBM, so a CTA owns 16 weight rows and its 8 warps split K; every lane streams 16 bytes of two
// weight rows per step straight into mma.sync m16n8k16 A fragments (W rows are the M dimension of the tile, the tokens the
// N dimension; the reduction over K is order-free, so a lane's 8 consecutive channels serve as the fragment's k-slots and
// the activations are loaded with the same addressing).  Tokens beyond M load nothing.  Warp partials meet in shared memory.
//
// The reference sends these products to the library GEMM (cc/src/tyr.cpp:1003-1036).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace tyr {

constexpr int kSkWarps = 8;

struct SkinnyArgs {
  const __nv_bfloat16* x;      // [M, K], row stride ldx
  const __nv_bfloat16* w;      // [N, K], row stride ldw
  const __nv_bfloat16* w2;     // gated form only: the second matrix [N, K]; y = silu(x w^T) * (x w2^T)
  const __nv_bfloat16* bias;   // [N] or null
  __nv_bfloat16* y;            // [M, N], row stride ldy
  float* ws;                   // [M, N] fp32, zero on entry and exit; used when the reduction is split over gridDim.y CTAs
  long long ldx, ldw, ldy;
  int M, N, K;
};

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr long long kSkPrefetchBytes = 32LL << 20;   // L2 prefetch issued by one launch before its input is ready

template <int TILES, bool GATED>                   // token tiles of 8: M <= 8 * TILES; GATED: two matrices, SwiGLU epilogue
__global__ void __launch_bounds__(kSkWarps * 32) skinny_gemm_kernel(SkinnyArgs a) {
  __shared__ float part[GATED ? 2 : 1][kSkWarps][TILES][16][8];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * 16;
  // The weights are constants: while the kernel that produces `x` still runs (this one may already be resident, see
  // launch_dependent), pull the head of every weight row of this CTA into the L2.  The whole grid asks for at most
  // kSkPrefetchBytes, so what it brings in is still there when the loop below reads it.
  pdl_trigger();
  if (tid < (GATED ? 32 : 16) && (a.ldw & 7) == 0) {
    const int r = row0 + (tid & 15);
    const int chunks = a.K >> 5;
    const int c0 = static_cast<int>(static_cast<long long>(chunks) * blockIdx.y / gridDim.y);
    const int c1 = static_cast<int>(static_cast<long long>(chunks) * (blockIdx.y + 1) / gridDim.y);
    long long per_row = kSkPrefetchBytes / (static_cast<long long>(gridDim.x) * gridDim.y * (GATED ? 32 : 16));
    per_row = min(per_row & ~127LL, static_cast<long long>(c1 - c0) * 64);
    if (r < a.N && per_row >= 128)
      bulk_prefetch_l2((tid < 16 ? a.w : a.w2) + static_cast<long long>(r) * a.ldw + 32LL * c0, static_cast<uint32_t>(per_row));
  }
  pdl_wait();
  int r_lo = row0 + g, r_hi = row0 + g + 8;
  r_lo = r_lo < a.N ? r_lo : a.N - 1;            // clamped rows are not written
  r_hi = r_hi < a.N ? r_hi : a.N - 1;
  const __nv_bfloat16* w_lo = a.w + r_lo * a.ldw + 8 * t;
  const __nv_bfloat16* w_hi = a.w + r_hi * a.ldw + 8 * t;
  const __nv_bfloat16* v_lo = GATED ? a.w2 + r_lo * a.ldw + 8 * t : nullptr;
  const __nv_bfloat16* v_hi = GATED ? a.w2 + r_hi * a.ldw + 8 * t : nullptr;
  const __nv_bfloat16* xr[TILES];
  bool live[TILES];
#pragma unroll
  for (int i = 0; i < TILES; ++i) {
    const int tok = 8 * i + g;
    live[i] = tok < a.M;
    xr[i] = a.x + (live[i] ? tok : 0) * a.ldx + 8 * t;
  }
  float acc[TILES][4], acc2[TILES][4];
#pragma unroll
  for (int i = 0; i < TILES; ++i) {
    acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    acc2[i][0] = acc2[i][1] = acc2[i][2] = acc2[i][3] = 0.f;
  }

  const int chunks = a.K >> 5;                   // 32 channels per warp step
  const int c_lo = static_cast<int>(static_cast<long long>(chunks) * blockIdx.y / gridDim.y);
  const int c_hi = static_cast<int>(static_cast<long long>(chunks) * (blockIdx.y + 1) / gridDim.y);
#pragma unroll 4
  for (int c = c_lo + warp; c < c_hi; c += kSkWarps) {
    const uint4 lo = __ldcs(reinterpret_cast<const uint4*>(w_lo + 32 * c));    // streamed once: do not keep in cache
    const uint4 hi = __ldcs(reinterpret_cast<const uint4*>(w_hi + 32 * c));
    uint4 lo2 = make_uint4(0u, 0u, 0u, 0u), hi2 = lo2;
    if (GATED) {
      lo2 = __ldcs(reinterpret_cast<const uint4*>(v_lo + 32 * c));
      hi2 = __ldcs(reinterpret_cast<const uint4*>(v_hi + 32 * c));
    }
#pragma unroll
    for (int i = 0; i < TILES; ++i) {
      const uint4 xv = live[i] ? __ldg(reinterpret_cast<const uint4*>(xr[i] + 32 * c)) : make_uint4(0u, 0u, 0u, 0u);
      mma_16816(acc[i], lo.x, hi.x, lo.y, hi.y, xv.x, xv.y);
      mma_16816(acc[i], lo.z, hi.z, lo.w, hi.w, xv.z, xv.w);
      if (GATED) {
        mma_16816(acc2[i], lo2.x, hi2.x, lo2.y, hi2.y, xv.x, xv.y);
        mma_16816(acc2[i], lo2.z, hi2.z, lo2.w, hi2.w, xv.z, xv.w);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < TILES; ++i) {
    part[0][warp][i][g][2 * t] = acc[i][0];
    part[0][warp][i][g][2 * t + 1] = acc[i][1];
    part[0][warp][i][g + 8][2 * t] = acc[i][2];
    part[0][warp][i][g + 8][2 * t + 1] = acc[i][3];
    if (GATED) {
      part[1][warp][i][g][2 * t] = acc2[i][0];
      part[1][warp][i][g][2 * t + 1] = acc2[i][1];
      part[1][warp][i][g + 8][2 * t] = acc2[i][2];
      part[1][warp][i][g + 8][2 * t + 1] = acc2[i][3];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < TILES * 8 * 16; idx += kSkWarps * 32) {
    const int tok = idx >> 4, r = idx & 15;        // consecutive threads write consecutive output columns
    const int row = row0 + r;
    if (tok < a.M && row < a.N) {
      float s = 0.f;
#pragma unroll
      for (int wp = 0; wp < kSkWarps; ++wp) s += part[0][wp][tok >> 3][r][tok & 7];
      if (GATED) {
        float u = 0.f;
#pragma unroll
        for (int wp = 0; wp < kSkWarps; ++wp) u += part[1][wp][tok >> 3][r][tok & 7];
        a.y[tok * a.ldy + row] = __float2bfloat16(s / (1.f + __expf(-s)) * u);
      } else if (gridDim.y == 1) {
        if (a.bias) s += __bfloat162float(a.bias[row]);
        a.y[tok * a.ldy + row] = __float2bfloat16(s);
      } else {
        atomicAdd(a.ws + static_cast<long long>(tok) * a.N + row, s);
      }
    }
  }
}

// Second pass of a split reduction: round the fp32 sums (+ bias) and leave the workspace zeroed for the next call.
__global__ void __launch_bounds__(256) skinny_finish_kernel(SkinnyArgs a) {
  pdl_entry();
  const long long n = static_cast<long long>(a.M) * a.N;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * 256) {
    const int tok = static_cast<int>(i / a.N), row = static_cast<int>(i - static_cast<long long>(tok) * a.N);
    float s = a.ws[i];
    a.ws[i] = 0.f;
    if (a.bias) s += __bfloat162float(a.bias[row]);
    a.y[tok * a.ldy + row] = __float2bfloat16(s);
  }
}

}  // namespace tyr

// The kernels above read the activations through the L1: the eight CTAs of an SM walk the same rows of x.  A kernel with a
// large shared-memory footprint earlier in the stream leaves the SMs split in favour of shared memory, and a kernel that
// states no preference inherits that split.  Ask for just the shared memory that the resident CTAs need (registers and
// threads bound their number); the rest is L1.
template <int TILES, bool GATED>
static void skinny_set_carveout() {
  const int per_cta = (GATED ? 2 : 1) * tyr::kSkWarps * TILES * 16 * 8 * 4 + 1024;
  int ctas = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas, tyr::skinny_gemm_kernel<TILES, GATED>, tyr::kSkWarps * 32, 0) != cudaSuccess ||
      ctas < 1)
    return;
  int pct = (ctas * per_cta * 100 + 227 * 1024 - 1) / (227 * 1024);
  if (pct > 100) pct = 100;
  cudaFuncSetAttribute(tyr::skinny_gemm_kernel<TILES, GATED>, cudaFuncAttributePreferredSharedMemoryCarveout, pct);
}
static void skinny_prefer_l1() {
  static bool done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (done[dev]) return;
  done[dev] = true;
  const char* v = getenv("TYR_SKINNY_CARVEOUT");
  if (v != nullptr && v[0] == '0') return;
  skinny_set_carveout<1, false>();
  skinny_set_carveout<2, false>();
  skinny_set_carveout<4, false>();
  skinny_set_carveout<1, true>();
  skinny_set_carveout<2, true>();
  skinny_set_carveout<4, true>();
}

// Number of CTAs the reduction should be split over for this shape (1 = no workspace needed): enough CTAs to cover the
// SMs about three times, at least 1024 channels per split.
extern "C" TYR_EXPORT int tyr_skinny_gemm_splits(int N, int K) {
  const int row_ctas = (N + 15) / 16;
  int splits = (3 * 148 + row_ctas - 1) / row_ctas;
  const int max_by_k = K / 1024 > 0 ? K / 1024 : 1;
  if (splits > max_by_k) splits = max_by_k;
  if (splits > 8) splits = 8;
  return splits < 1 ? 1 : splits;
}

extern "C" TYR_EXPORT int tyr_skinny_gemm_bf16(const void* x, const void* w, const void* bias, void* y, void* ws, long long ldx,
                                               long long ldw, long long ldy, int M, int N, int K, void* stream) {
  using namespace tyr;
  if (M < 1 || M > 32 || N < 1 || K < 32 || (K & 31)) return -1;
  if ((ldx | ldw) & 7) return -2;                                    // 16-byte loads
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return -3;
  SkinnyArgs a{(const __nv_bfloat16*)x, (const __nv_bfloat16*)w, nullptr, (const __nv_bfloat16*)bias, (__nv_bfloat16*)y, (float*)ws, ldx, ldw, ldy, M, N, K};
  const int splits = ws != nullptr ? tyr_skinny_gemm_splits(N, K) : 1;
  const dim3 grid((N + 15) / 16, splits);
  skinny_prefer_l1();
  if (M <= 8) launch_dependent(skinny_gemm_kernel<1, false>, dim3(grid), dim3(kSkWarps * 32), 0, (cudaStream_t)stream, a);
  else if (M <= 16) launch_dependent(skinny_gemm_kernel<2, false>, dim3(grid), dim3(kSkWarps * 32), 0, (cudaStream_t)stream, a);
  else launch_dependent(skinny_gemm_kernel<4, false>, dim3(grid), dim3(kSkWarps * 32), 0, (cudaStream_t)stream, a);
  if (splits > 1) {
    long long blocks = (static_cast<long long>(M) * N + 255) / 256;
    if (blocks > 592) blocks = 592;
    launch_dependent(skinny_finish_kernel, dim3((int)blocks), dim3(256), 0, (cudaStream_t)stream, a);
  }
  return (int)cudaGetLastError();
}

// y[M, N] = silu(x wg^T) * (x wu^T): the gate and up projections of a SwiGLU MLP for decode-sized M in one pass over both
// matrices (same row stride ldw), no intermediate tensors.
extern "C" TYR_EXPORT int tyr_skinny_swiglu_bf16(const void* x, const void* wg, const void* wu, void* y, long long ldx,
                                                 long long ldw, long long ldy, int M, int N, int K, void* stream) {
  using namespace tyr;
  if (M < 1 || M > 32 || N < 1 || K < 32 || (K & 31)) return -1;
  if ((ldx | ldw) & 7) return -2;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(wg) | reinterpret_cast<uintptr_t>(wu)) & 15) return -3;
  SkinnyArgs a{(const __nv_bfloat16*)x, (const __nv_bfloat16*)wg, (const __nv_bfloat16*)wu, nullptr, (__nv_bfloat16*)y, nullptr, ldx, ldw, ldy, M, N, K};
  const dim3 grid((N + 15) / 16, 1);
  skinny_prefer_l1();
  if (M <= 8) launch_dependent(skinny_gemm_kernel<1, true>, dim3(grid), dim3(kSkWarps * 32), 0, (cudaStream_t)stream, a);
  else if (M <= 16) launch_dependent(skinny_gemm_kernel<2, true>, dim3(grid), dim3(kSkWarps * 32), 0, (cudaStream_t)stream, a);
  else launch_dependent(skinny_gemm_kernel<4, true>, dim3(grid), dim3(kSkWarps * 32), 0, (cudaStream_t)stream, a);
  return (int)cudaGetLastError();
}
