// Expert-parallel dispatch / combine over peer memory (one NVLink domain, symmetric heap).
//
// Experts are split over the ranks (expert e lives on rank e / E_local).  Both directions are PULLS with
// plain peer loads, so every row crosses NVLink exactly once and nobody writes into memory it does not own:
//
//   source rank:  route -> expert-major sort of its (token, slot) pairs -> rows gathered into the symmetric
//                 buffer `xs`, offsets[E + 1] published                                   | flag barrier 1
//   owner rank:   ep_layout: reads every source's offsets for its experts, lays the incoming rows out
//                 expert-major / source-minor, publishes dest_base[e_local][src]
//                 ep_pull:   copies the segments from the sources' xs into its local row buffer
//                 expert FFN on the local rows (grouped tcgen05 GEMM or the FP4 GEMV), result y in
//                 symmetric memory                                                           | flag barrier 2
//   source rank:  ep_combine: out[t] = sum_slots w * y_owner[dest_base_owner[e][me] + q] (+ add), reading
//                 the owners' y rows directly.
//
// The reference keeps all experts on one GPU (Tyr/Model/Laguna/MoE.lean:271-356); this is the multi-GPU
// counterpart of that dispatch.  No kernel here waits on another rank: ordering comes from the flag
// barriers between the launches (bounded waits, csrc/comm_fused.cu).
#include "common.cuh"

namespace tyr {

constexpr int kEpMaxRanks = 8;

struct EpPeers {
  const void* p[kEpMaxRanks];
};

// One block.  seg = e_local * world + src.
//   seg_rows[seg]     rows arriving from src for expert e_local
//   seg_src_row[seg]  first row of that segment inside src's xs
//   dest_base[seg]    first row of that segment in the local row buffer (published to the sources)
//   meta[0] = total rows, meta[1..] expert offsets [E_local + 1], then tile prefix [E_local + 1]
__global__ void ep_layout_kernel(EpPeers src_offsets, int world, int my_rank, int E_local, int* seg_rows, int* seg_src_row,
                                 int* dest_base, int* expert_offsets, int* expert_tiles, int* total_rows, int capacity,
                                 int* err) {
  extern __shared__ int sh[];           // [E_local * world] counts then scan
  const int nseg = E_local * world;
  for (int s = threadIdx.x; s < nseg; s += blockDim.x) {
    const int e = s / world, src = s % world;
    const int* off = reinterpret_cast<const int*>(src_offsets.p[src]);
    const int ge = my_rank * E_local + e;
    const int a = off[ge], b = off[ge + 1];
    sh[s] = b - a;
    seg_rows[s] = b - a;
    seg_src_row[s] = a;
  }
  __syncthreads();
  if (threadIdx.x == 0) {               // nseg <= 8 * 512: a serial scan is a few microseconds
    int run = 0, tiles = 0;
    for (int e = 0; e < E_local; ++e) {
      expert_offsets[e] = run;
      expert_tiles[e] = tiles;
      const int start = run;
      for (int src = 0; src < world; ++src) {
        dest_base[e * world + src] = run;
        run += sh[e * world + src];
      }
      tiles += (run - start + 127) >> 7;
    }
    expert_offsets[E_local] = run;
    expert_tiles[E_local] = tiles;
    total_rows[0] = run;
    if (run > capacity) report_error(err, ERR_BOUNDS, run);
  }
}

// grid = (row blocks, E_local * world).  Copies one segment (rows of h bf16) from the source's xs.
__global__ void __launch_bounds__(256)
ep_pull_kernel(EpPeers xs, const int* seg_rows, const int* seg_src_row, const int* dest_base, __nv_bfloat16* rows_out,
               int* row_expert, int world, int h, int capacity) {
  const int seg = blockIdx.y;
  const int n = seg_rows[seg];
  if (n == 0) return;
  const int e = seg / world, src = seg % world;
  const int dst0 = dest_base[seg];
  if (dst0 + n > capacity) return;      // overflow was reported by the layout kernel
  const __nv_bfloat16* from = reinterpret_cast<const __nv_bfloat16*>(xs.p[src]) + static_cast<long long>(seg_src_row[seg]) * h;
  __nv_bfloat16* to = rows_out + static_cast<long long>(dst0) * h;
  const long long nvec = static_cast<long long>(n) * h / 8;
  const uint4* f4 = reinterpret_cast<const uint4*>(from);
  uint4* t4 = reinterpret_cast<uint4*>(to);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < nvec; v += 4 * stride) {
    uint4 b[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (v + j * stride < nvec) b[j] = f4[v + j * stride];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (v + j * stride < nvec) t4[v + j * stride] = b[j];
  }
  if (row_expert)
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < n; r += gridDim.x * blockDim.x) row_expert[dst0 + r] = e;
}

// out[t] = sum_s w[t,s] * y_owner[dest_base_owner[e_local][me] + (pos - offsets[e])] (+ add[t])
// A row index outside [0, capacity) (the owner received more rows than its buffers hold: ep_layout recorded the overflow
// and ep_pull skipped the segment) contributes nothing and records ERR_BOUNDS; the owner's y is never read past its end.
__global__ void __launch_bounds__(256)
ep_combine_kernel(EpPeers y, EpPeers dest_base, const int* ids, const float* weights, const int* pair_pos, const int* offsets,
                  const __nv_bfloat16* add, __nv_bfloat16* out, int T, int k, int h, int E_local, int world, int my_rank,
                  int capacity, int* err) {
  const int vec = h >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < static_cast<long long>(T) * vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int tok = static_cast<int>(i / vec), c = static_cast<int>(i % vec);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < k; ++s) {
      const int pair = tok * k + s;
      const int e = ids[pair];
      const int owner = e / E_local, el = e - owner * E_local;
      const int q = pair_pos[pair] - offsets[e];
      const int row = reinterpret_cast<const int*>(dest_base.p[owner])[el * world + my_rank] + q;
      if (e < 0 || owner >= world || row < 0 || row >= capacity) {
        if (c == 0) report_error(err, ERR_BOUNDS, row);
        continue;
      }
      const float w = weights[pair];
      const uint4 u = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(y.p[owner]) +
                                                     static_cast<long long>(row) * h)[c];
      const float2 a0 = unpack_bf16x2(u.x), a1 = unpack_bf16x2(u.y), a2 = unpack_bf16x2(u.z), a3 = unpack_bf16x2(u.w);
      acc[0] += w * a0.x; acc[1] += w * a0.y; acc[2] += w * a1.x; acc[3] += w * a1.y;
      acc[4] += w * a2.x; acc[5] += w * a2.y; acc[6] += w * a3.x; acc[7] += w * a3.y;
    }
    if (add) {
      const uint4 u = reinterpret_cast<const uint4*>(add + static_cast<long long>(tok) * h)[c];
      const float2 a0 = unpack_bf16x2(u.x), a1 = unpack_bf16x2(u.y), a2 = unpack_bf16x2(u.z), a3 = unpack_bf16x2(u.w);
      acc[0] += a0.x; acc[1] += a0.y; acc[2] += a1.x; acc[3] += a1.y;
      acc[4] += a2.x; acc[5] += a2.y; acc[6] += a3.x; acc[7] += a3.y;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + static_cast<long long>(tok) * h)[c] = o;
  }
}

static EpPeers make_ep_peers(void* const* ptrs, int world) {
  EpPeers p{};
  for (int i = 0; i < world; ++i) p.p[i] = ptrs[i];
  return p;
}

}  // namespace tyr

using namespace tyr;

// Owner side: layout + pull.  `src_offsets[r]` / `xs[r]`: rank r's published offsets[E + 1] and sorted rows.
// Outputs (local): seg tables [E_local * world] x3 (dest_base must live in symmetric memory), expert_offsets and
// expert_tiles [E_local + 1], total_rows [1], rows_out [capacity, h], row_expert [capacity] (nullable).
extern "C" TYR_EXPORT int tyr_ep_pull(void* const* src_offsets, void* const* xs, int world, int my_rank, int E_local, int h,
                                      int* seg_rows, int* seg_src_row, int* dest_base, int* expert_offsets, int* expert_tiles,
                                      int* total_rows, void* rows_out, int* row_expert, int capacity, int max_seg_rows,
                                      int* err, void* stream) {
  if (world < 1 || world > kEpMaxRanks || E_local <= 0 || (h & 7) || capacity <= 0) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  const int nseg = E_local * world;
  if (nseg * (int)sizeof(int) > 48 * 1024) return -2;
  ep_layout_kernel<<<1, 256, nseg * sizeof(int), st>>>(make_ep_peers(src_offsets, world), world, my_rank, E_local, seg_rows,
                                                      seg_src_row, dest_base, expert_offsets, expert_tiles, total_rows,
                                                      capacity, err);
  long long bx = (static_cast<long long>(max_seg_rows) * h / 8 + 1023) / 1024;
  if (bx < 1) bx = 1;
  if (bx > 64) bx = 64;
  ep_pull_kernel<<<dim3((unsigned)bx, nseg), 256, 0, st>>>(make_ep_peers(xs, world), seg_rows, seg_src_row, dest_base,
                                                          (__nv_bfloat16*)rows_out, row_expert, world, h, capacity);
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_ep_combine(void* const* y, void* const* dest_base, const int* ids, const float* weights,
                                         const int* pair_pos, const int* offsets, const void* add, void* out, int T, int k,
                                         int h, int E_local, int world, int my_rank, int capacity, int* err, void* stream) {
  if (world < 1 || world > kEpMaxRanks || T <= 0 || (h & 7) || capacity <= 0) return -1;
  long long blocks = (static_cast<long long>(T) * (h / 8) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  ep_combine_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(make_ep_peers(y, world), make_ep_peers(dest_base, world), ids,
                                                                  weights, pair_pos, offsets, (const __nv_bfloat16*)add,
                                                                  (__nv_bfloat16*)out, T, k, h, E_local, world, my_rank,
                                                                  capacity, err);
  return (int)cudaGetLastError();
}
