// Embedding-table gradient: grad[id] += sum of the dy rows whose token is `id`, accumulated into an fp32 table.
//
// The token stream is Zipf-distributed: a handful of ids own thousands of rows each, and a plain scatter-add (one fp32
// atomic per element and occurrence, what `index_add_` does) serialises on those table rows.  Here the rows arrive SORTED
// by id (one sort per step serves the token table and every value-embedding table).  A CTA takes a run of consecutive
// sorted positions, keeps the running sum of equal ids in registers and touches the table once per id and run: the
// atomics drop from one per occurrence to one per (id, run), and dy is read exactly once, 16 bytes per thread and row.
//
// The reference differentiates `embedding` through autograd's dense scatter (Examples/NanoChat/ModdedGPT.lean:563-567,
// cc/src/tyr.cpp embedding op).
#include "common.cuh"

namespace tyr {

constexpr int kEmbedRun = 64;   // sorted positions per CTA

// dy [N, d] bf16 (row stride ld), order[p] = row of dy at sorted position p, sorted_ids[p] ascending, grad fp32 [V, d].
// blockDim.x * 8 >= d is not required: threads stride over the columns in 8-element vectors.
__global__ void __launch_bounds__(256)
embed_grad_sorted_kernel(const __nv_bfloat16* __restrict__ dy, const long long* __restrict__ order,
                         const long long* __restrict__ sorted_ids, float* __restrict__ grad, int N, int d, long long ld,
                         int V) {
  pdl_entry();
  __shared__ long long s_row[kEmbedRun];
  __shared__ long long s_id[kEmbedRun];
  const int p0 = blockIdx.x * kEmbedRun;
  const int n = min(kEmbedRun, N - p0);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    s_row[i] = order[p0 + i];
    s_id[i] = sorted_ids[p0 + i];
  }
  __syncthreads();
  for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    long long cur = s_id[0];
    for (int i = 0; i < n; ++i) {
      const long long id = s_id[i];
      if (id != cur) {
        if (cur >= 0 && cur < V) {
          float* g = grad + cur * d + c;
#pragma unroll
          for (int q = 0; q < 2; ++q)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(g + q * 4), "f"(acc[q * 4]), "f"(acc[q * 4 + 1]),
                         "f"(acc[q * 4 + 2]), "f"(acc[q * 4 + 3])
                         : "memory");
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        cur = id;
      }
      const long long r = s_row[i];
      if (r < 0 || r >= N) continue;
      const uint4 u = *reinterpret_cast<const uint4*>(dy + r * ld + c);
      const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
      acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
      acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
    }
    if (cur >= 0 && cur < V) {
      float* g = grad + cur * d + c;
#pragma unroll
      for (int q = 0; q < 2; ++q)
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(g + q * 4), "f"(acc[q * 4]), "f"(acc[q * 4 + 1]),
                     "f"(acc[q * 4 + 2]), "f"(acc[q * 4 + 3])
                     : "memory");
    }
  }
}

}  // namespace tyr

// Returns 0 on success, -1 on a bad shape / alignment.
extern "C" TYR_EXPORT int tyr_embed_grad_sorted(const void* dy, const long long* order, const long long* sorted_ids, float* grad,
                                                int N, int d, long long ld, int V, void* stream) {
  if (N <= 0 || d <= 0 || (d & 7) || (ld & 7) || V <= 0) return -1;
  if ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(grad)) & 15) return -1;
  const int blocks = (N + tyr::kEmbedRun - 1) / tyr::kEmbedRun;
  const int threads = d / 8 >= 256 ? 256 : ((d / 8 + 31) / 32) * 32;
  tyr::launch_dependent(tyr::embed_grad_sorted_kernel, dim3(blocks), dim3(threads), 0, reinterpret_cast<cudaStream_t>(stream),
      reinterpret_cast<const __nv_bfloat16*>(dy), order, sorted_ids, grad, N, d, ld, V);
  return static_cast<int>(cudaGetLastError());
}
