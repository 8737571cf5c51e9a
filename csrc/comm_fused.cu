// Fused compute + collective kernels over NVLink peer memory (plain P2P loads/stores on
// IPC-mapped buffers; no NCCL call, no multicast loads).
//
// Data-parallel optimizer step.  Every rank holds complete local gradients in a symmetric
// buffer (same layout on every rank, mapped into every peer).  The reference does, per tensor,
// a blocking NCCL reduce_scatter, ~15 elementwise kernels and two or three all_gathers
// (Tyr/Optim/DistAdam.lean:185-267, Tyr/Optim/NorMuon.lean:346-425).  Here each of these is ONE
// kernel per parameter group:
//
//  * dp_adam_shard: the owner of a row shard pulls that shard of the gradient from all W peers
//    (16-byte P2P loads), averages in fp32, applies bias-corrected AdamW to its fp32 master shard
//    and moment shards (state is truly sharded), and pushes the refreshed bf16 parameters into
//    the working copy of EVERY rank (P2P stores) - reduce-scatter + update + all-gather.
//  * dp_muon_gather: the owner of a whole matrix (block-cyclic ownership, as the reference) pulls
//    and averages its gradient from all peers and applies momentum + Nesterov, emitting the bf16
//    Newton-Schulz input and its squared norm.
//  * dp_muon_apply_push: after the owner's Newton-Schulz GEMMs, applies the update to the fp32
//    master and pushes bf16 parameters to all ranks.
//  * signal / wait_all: a flag barrier in symmetric memory (st.release.sys / ld.acquire.sys).
//    Waits are bounded: on timeout the kernel records ERR_PEER_FLAG_TIMEOUT and returns.
//
// The tensor-parallel fusions (GEMM -> reduce-scatter epilogue, all-gather prologue) are modes of the GEMM kernel in
// gemm_tcgen05.cu; the expert-parallel dispatch / combine kernels live in ep_fused.cu.
#include "common.cuh"

namespace tyr {

constexpr int kMaxRanks = 8;

struct PeerPtrs {
  void* p[kMaxRanks];
};

__device__ __forceinline__ void st_release_sys(unsigned long long* addr, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(addr), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* addr) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(addr) : "memory");
  return v;
}
// Peer data is written by the other ranks while this kernel may already be resident (it waits for their flags itself), so
// the load must go through the coherent path: no `.nc`.  It bypasses L1 allocation because every value is read once.
__device__ __forceinline__ float4 ld_peer_f4(const float* p) {
  float4 v;
  asm volatile("ld.global.L1::no_allocate.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}

// Each rank writes `value` into slot [my_rank] of every peer's flag array.
__global__ void signal_kernel(PeerPtrs flags, int world, int my_rank, int slot_base,
                              unsigned long long value) {
  const int r = threadIdx.x;
  if (r < world) {
    __threadfence_system();
    unsigned long long* f = reinterpret_cast<unsigned long long*>(flags.p[r]) + slot_base + my_rank;
    st_release_sys(f, value);
  }
}

// Waits until every slot [slot_base + r] of the LOCAL flag array is >= value.
__global__ void wait_all_kernel(const unsigned long long* local_flags, int world, int slot_base,
                                unsigned long long value, int* err, long long budget_cycles) {
  const int r = threadIdx.x;
  if (r < world) {
    const unsigned long long* f = local_flags + slot_base + r;
    long long start = clock64();
    while (ld_acquire_sys(f) < value) {
      if (clock64() - start > budget_cycles) {
        report_error(err, ERR_PEER_FLAG_TIMEOUT, slot_base + r);
        break;
      }
      __nanosleep(200);
    }
  }
}

__device__ __forceinline__ bool wait_flags_in_kernel(const unsigned long long* local_flags, int world,
                                                     int slot_base, unsigned long long value,
                                                     int* err) {
  // executed by one thread of the CTA
  for (int r = 0; r < world; ++r) {
    const unsigned long long* f = local_flags + slot_base + r;
    long long start = clock64();
    while (ld_acquire_sys(f) < value) {
      if (clock64() - start > kWaitBudgetCycles * 4) {
        report_error(err, ERR_PEER_FLAG_TIMEOUT, slot_base + r);
        return false;
      }
      __nanosleep(200);
    }
  }
  return true;
}

struct DpAdamArgs {
  PeerPtrs grads;          // fp32 gradient buffers of all ranks (same offsets everywhere)
  PeerPtrs work;           // bf16 working-parameter buffers of all ranks
  long long grad_off;      // element offset of this tensor's shard start in the gradient buffers
  long long work_off;      // element offset of the shard start in the working buffers
  float* master;           // local fp32 master shard
  float* m;
  float* v;
  long long n;             // shard elements (multiple of 4)
  int world;
  float lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale;
  const unsigned long long* wait_flags;   // nullable: wait for all ranks' gradients first
  int wait_slot;
  unsigned long long wait_value;
  int* err;
};

__global__ void __launch_bounds__(256) dp_adam_shard_kernel(DpAdamArgs a) {
  if (a.wait_flags) {
    __shared__ int ok_s;
    if (threadIdx.x == 0)
      ok_s = wait_flags_in_kernel(a.wait_flags, a.world, a.wait_slot, a.wait_value, a.err) ? 1 : 0;
    __syncthreads();
    if (!ok_s) return;
  }
  const long long n4 = a.n >> 2;
  const float inv_w = a.grad_scale / a.world;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  // Four independent 16-byte elements per thread and iteration: all of their peer loads are issued before the first
  // result is used, so several NVLink round trips are in flight per thread (one element at a time reached about half of
  // the link bandwidth).
  constexpr int U = 4;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < n4; i0 += stride * U) {
    float4 g[U];
#pragma unroll
    for (int u = 0; u < U; ++u) g[u] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) {
      if (r < a.world) {
        const float* src = reinterpret_cast<const float*>(a.grads.p[r]) + a.grad_off;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * stride;
          if (i < n4) {
            const float4 t = ld_peer_f4(src + i * 4);
            g[u].x += t.x; g[u].y += t.y; g[u].z += t.z; g[u].w += t.w;
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= n4) break;
      float4 p = reinterpret_cast<float4*>(a.master)[i];
      float4 m = reinterpret_cast<float4*>(a.m)[i];
      float4 v = reinterpret_cast<float4*>(a.v)[i];
      float gg[4] = {g[u].x * inv_w, g[u].y * inv_w, g[u].z * inv_w, g[u].w * inv_w};
      float pp[4] = {p.x, p.y, p.z, p.w}, mm[4] = {m.x, m.y, m.z, m.w}, vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gg[j];
        vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gg[j] * gg[j];
        pp[j] = pp[j] * (1.f - a.lr * a.wd) - a.lr * (mm[j] / a.bc1) / (sqrtf(vv[j] / a.bc2) + a.eps);
      }
      reinterpret_cast<float4*>(a.master)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
      reinterpret_cast<float4*>(a.m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
      reinterpret_cast<float4*>(a.v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
      uint2 w;
      w.x = pack_bf16x2(pp[0], pp[1]);
      w.y = pack_bf16x2(pp[2], pp[3]);
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < a.world)
          reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.work.p[r]) + a.work_off)[i] = w;
    }
  }
}

struct DpMuonGatherArgs {
  PeerPtrs grads;
  const long long* grad_offs;   // [B_own] element offset of each owned matrix in the gradient buffers
  float* mom;                   // [B_own, per] local momentum of owned matrices
  __nv_bfloat16* u;             // [B_own, per]
  float* sumsq;                 // [B_own] zero on entry
  long long per;
  int B_own, world;
  float mu, grad_scale;
  const unsigned long long* wait_flags;
  int wait_slot;
  unsigned long long wait_value;
  int* err;
};

__global__ void __launch_bounds__(256) dp_muon_gather_kernel(DpMuonGatherArgs a) {
  if (a.wait_flags) {
    __shared__ int ok_s;
    if (threadIdx.x == 0)
      ok_s = wait_flags_in_kernel(a.wait_flags, a.world, a.wait_slot, a.wait_value, a.err) ? 1 : 0;
    __syncthreads();
    if (!ok_s) return;
  }
  const int b = blockIdx.y;
  const long long goff = a.grad_offs[b];
  const long long base = static_cast<long long>(b) * a.per;
  const long long n4 = a.per >> 2;
  const float inv_w = a.grad_scale / a.world;
  const float om = 1.f - a.mu;
  float ss = 0.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  constexpr int U = 4;          // see dp_adam_shard_kernel
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < n4; i0 += stride * U) {
    float4 gs[U];
#pragma unroll
    for (int u = 0; u < U; ++u) gs[u] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) {
      if (r < a.world) {
        const float* src = reinterpret_cast<const float*>(a.grads.p[r]) + goff;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * stride;
          if (i < n4) {
            const float4 t = ld_peer_f4(src + i * 4);
            gs[u].x += t.x; gs[u].y += t.y; gs[u].z += t.z; gs[u].w += t.w;
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= n4) break;
      float4 g = gs[u];
      g.x *= inv_w; g.y *= inv_w; g.z *= inv_w; g.w *= inv_w;
      float4 m = *reinterpret_cast<float4*>(a.mom + base + i * 4);
      m.x = a.mu * m.x + om * g.x; m.y = a.mu * m.y + om * g.y;
      m.z = a.mu * m.z + om * g.z; m.w = a.mu * m.w + om * g.w;
      *reinterpret_cast<float4*>(a.mom + base + i * 4) = m;
      uint2 w;
      w.x = pack_bf16x2(om * g.x + a.mu * m.x, om * g.y + a.mu * m.y);
      w.y = pack_bf16x2(om * g.z + a.mu * m.z, om * g.w + a.mu * m.w);
      *reinterpret_cast<uint2*>(a.u + base + i * 4) = w;
      float2 r0 = unpack_bf16x2(w.x), r1 = unpack_bf16x2(w.y);
      ss += r0.x * r0.x + r0.y * r0.y + r1.x * r1.x + r1.y * r1.y;
    }
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

struct DpMuonApplyArgs {
  PeerPtrs work;
  const long long* work_offs;   // [B_own]
  float* master;                // [B_own, per]
  const __nv_bfloat16* o;       // [B_own, per] orthogonalised update
  long long per;
  int B_own, world;
  float lr, wd;
};

__global__ void __launch_bounds__(256) dp_muon_apply_push_kernel(DpMuonApplyArgs a) {
  const int b = blockIdx.y;
  const long long woff = a.work_offs[b];
  const long long base = static_cast<long long>(b) * a.per;
  const long long n4 = a.per >> 2;
  const float decay = 1.f - a.lr * a.wd;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 w = *reinterpret_cast<float4*>(a.master + base + i * 4);
    uint2 u = *reinterpret_cast<const uint2*>(a.o + base + i * 4);
    float2 x = unpack_bf16x2(u.x), y = unpack_bf16x2(u.y);
    w.x = w.x * decay - __bfloat162float(__float2bfloat16(x.x * a.lr));
    w.y = w.y * decay - __bfloat162float(__float2bfloat16(x.y * a.lr));
    w.z = w.z * decay - __bfloat162float(__float2bfloat16(y.x * a.lr));
    w.w = w.w * decay - __bfloat162float(__float2bfloat16(y.y * a.lr));
    *reinterpret_cast<float4*>(a.master + base + i * 4) = w;
    uint2 q;
    q.x = pack_bf16x2(w.x, w.y);
    q.y = pack_bf16x2(w.z, w.w);
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < a.world)
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.work.p[r]) + woff + i * 4) = q;
  }
}

// Generic peer reduce: out[i] = scale * sum_r src_r[off + i]  (fp32), used for small tensors and
// for the all-reduce flavour of the public API.
__global__ void __launch_bounds__(256)
peer_sum_kernel(PeerPtrs src, long long off, float* out, long long n, int world, float scale) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float s = 0.f;
    for (int r = 0; r < world; ++r) s += reinterpret_cast<const float*>(src.p[r])[off + i];
    out[i] = s * scale;
  }
}

// The same sum with 16-byte peer loads, four per thread in flight (off and n multiples of 4 elements, 16-byte aligned bases).
__global__ void __launch_bounds__(256)
peer_sum_v4_kernel(PeerPtrs src, long long off, float* out, long long n4, int world, float scale) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < n4; i0 += 4 * stride) {
    float4 acc[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const float* base = reinterpret_cast<const float*>(src.p[r]) + off;
      float4 t[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * stride < n4) t[u] = ld_peer_f4(base + (i0 + u * stride) * 4);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * stride < n4) { acc[u].x += t[u].x; acc[u].y += t[u].y; acc[u].z += t[u].z; acc[u].w += t[u].w; }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i0 + u * stride < n4)
        reinterpret_cast<float4*>(out)[i0 + u * stride] =
            make_float4(acc[u].x * scale, acc[u].y * scale, acc[u].z * scale, acc[u].w * scale);
  }
}

// All-gather flavour: out[r * m + i] = src_r[off + i] for every rank r (m a multiple of 4 elements): every rank pulls the
// other ranks' pieces with plain peer loads.
__global__ void __launch_bounds__(256)
peer_gather_kernel(PeerPtrs src, long long off, float* out, long long m4, int world) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long total = m4 * world;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < total; i0 += 4 * stride) {
    float4 t[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * stride;
      if (i < total) {
        const int r = static_cast<int>(i / m4);
        t[u] = ld_peer_f4(reinterpret_cast<const float*>(src.p[r]) + off + (i - r * m4) * 4);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * stride;
      if (i < total) reinterpret_cast<float4*>(out)[i] = t[u];
    }
  }
}

}  // namespace tyr

using namespace tyr;

// ----------------------------------------------------------------------------------------
// symmetric memory: allocation + CUDA IPC export/import
// ----------------------------------------------------------------------------------------
extern "C" TYR_EXPORT int tyr_symm_alloc(void** out, long long bytes) {
  cudaError_t e = cudaMalloc(out, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(*out, 0, (size_t)bytes);
  return (int)e;
}
extern "C" TYR_EXPORT int tyr_symm_free(void* p) { return (int)cudaFree(p); }
extern "C" TYR_EXPORT int tyr_ipc_export(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
extern "C" TYR_EXPORT int tyr_ipc_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
extern "C" TYR_EXPORT int tyr_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

// Signal + wait in one launch with the sequence number in device memory (`*seq` holds the number of barriers completed on
// this slot), so the launch has no host-dependent argument and can be replayed from a CUDA graph: every rank publishes
// seq + 1 to all peers, waits (bounded) until all peers published it, then advances the counter.
__global__ void barrier_dev_kernel(PeerPtrs flags, const unsigned long long* local_flags, int world, int my_rank,
                                   int slot_base, unsigned long long* seq, int* err) {
  const int r = threadIdx.x;
  const unsigned long long value = *seq + 1;
  if (r < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<unsigned long long*>(flags.p[r]) + slot_base + my_rank, value);
    const unsigned long long* f = local_flags + slot_base + r;
    const long long start = clock64();
    while (ld_acquire_sys(f) < value) {
      if (clock64() - start > kWaitBudgetCycles * 4) {
        report_error(err, ERR_PEER_FLAG_TIMEOUT, slot_base + r);
        break;
      }
      __nanosleep(100);
    }
  }
  __syncwarp();
  if (r == 0) *seq = value;
}

static PeerPtrs make_peers(void* const* ptrs, int world) {
  PeerPtrs pp;
  for (int i = 0; i < kMaxRanks; ++i) pp.p[i] = i < world ? ptrs[i] : nullptr;
  return pp;
}

extern "C" TYR_EXPORT int tyr_signal(void* const* flag_ptrs, int world, int my_rank, int slot_base,
                                     unsigned long long value, void* stream) {
  if (world < 1 || world > kMaxRanks) return -1;
  signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(make_peers(flag_ptrs, world), world, my_rank,
                                                    slot_base, value);
  return (int)cudaGetLastError();
}
extern "C" TYR_EXPORT int tyr_barrier_dev(void* const* flag_ptrs, const void* local_flags, int world, int my_rank, int slot_base,
                                          void* seq, int* err, void* stream) {
  if (world < 1 || world > kMaxRanks) return -1;
  barrier_dev_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(make_peers(flag_ptrs, world), (const unsigned long long*)local_flags,
                                                         world, my_rank, slot_base, (unsigned long long*)seq, err);
  return (int)cudaGetLastError();
}
extern "C" TYR_EXPORT int tyr_wait_all(const void* local_flags, int world, int slot_base,
                                       unsigned long long value, int* err, void* stream) {
  if (world < 1 || world > kMaxRanks) return -1;
  wait_all_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((const unsigned long long*)local_flags, world,
                                                      slot_base, value, err, kWaitBudgetCycles * 4);
  return (int)cudaGetLastError();
}

// Same wait with a caller-chosen cycle budget (health checks and tests use a short one): on expiry the
// kernel records ERR_PEER_FLAG_TIMEOUT with the slot in the error record and returns; the context stays usable.
extern "C" TYR_EXPORT int tyr_wait_all_budget(const void* local_flags, int world, int slot_base, unsigned long long value,
                                              int* err, long long budget_cycles, void* stream) {
  if (world < 1 || world > kMaxRanks || budget_cycles <= 0) return -1;
  wait_all_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((const unsigned long long*)local_flags, world,
                                                      slot_base, value, err, budget_cycles);
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_dp_adam_shard(void* const* grad_ptrs, void* const* work_ptrs, int world,
                                            long long grad_off, long long work_off, float* master,
                                            float* m, float* v, long long n, float lr, float beta1,
                                            float beta2, float eps, float wd, float bc1, float bc2,
                                            float grad_scale, const void* wait_flags, int wait_slot,
                                            unsigned long long wait_value, int* err, int ctas,
                                            void* stream) {
  if (world < 1 || world > kMaxRanks || n <= 0 || (n & 3) || (grad_off & 3) || (work_off & 3)) return -1;
  DpAdamArgs a;
  a.grads = make_peers(grad_ptrs, world);
  a.work = make_peers(work_ptrs, world);
  a.grad_off = grad_off; a.work_off = work_off;
  a.master = master; a.m = m; a.v = v; a.n = n; a.world = world;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.wd = wd; a.bc1 = bc1; a.bc2 = bc2;
  a.grad_scale = grad_scale;
  a.wait_flags = (const unsigned long long*)wait_flags; a.wait_slot = wait_slot; a.wait_value = wait_value;
  a.err = err;
  long long blocks = (n / 4 + 255) / 256;
  const int cap = ctas > 0 ? ctas : 148 * 4;
  if (blocks > cap) blocks = cap;
  dp_adam_shard_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_dp_muon_gather(void* const* grad_ptrs, int world, const long long* grad_offs,
                                             float* mom, void* u, float* sumsq, long long per, int B_own,
                                             float mu, float grad_scale, const void* wait_flags,
                                             int wait_slot, unsigned long long wait_value, int* err,
                                             int ctas, void* stream) {
  if (world < 1 || world > kMaxRanks || per <= 0 || (per & 3) || B_own <= 0) return -1;
  DpMuonGatherArgs a;
  a.grads = make_peers(grad_ptrs, world);
  a.grad_offs = grad_offs; a.mom = mom; a.u = (__nv_bfloat16*)u; a.sumsq = sumsq; a.per = per;
  a.B_own = B_own; a.world = world; a.mu = mu; a.grad_scale = grad_scale;
  a.wait_flags = (const unsigned long long*)wait_flags; a.wait_slot = wait_slot; a.wait_value = wait_value;
  a.err = err;
  const int cap = ctas > 0 ? ctas : 148 * 4;
  int gx = (int)((per / 4 + 255) / 256);
  int per_b = (cap + B_own - 1) / B_own;
  if (per_b < 1) per_b = 1;
  if (gx > per_b) gx = per_b;
  dp_muon_gather_kernel<<<dim3(gx, B_own), 256, 0, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_dp_muon_apply_push(void* const* work_ptrs, int world, const long long* work_offs,
                                                 float* master, const void* o, long long per, int B_own,
                                                 float lr, float wd, int ctas, void* stream) {
  if (world < 1 || world > kMaxRanks || per <= 0 || (per & 3) || B_own <= 0) return -1;
  DpMuonApplyArgs a;
  a.work = make_peers(work_ptrs, world);
  a.work_offs = work_offs; a.master = master; a.o = (const __nv_bfloat16*)o; a.per = per;
  a.B_own = B_own; a.world = world; a.lr = lr; a.wd = wd;
  const int cap = ctas > 0 ? ctas : 148 * 4;
  int gx = (int)((per / 4 + 255) / 256);
  int per_b = (cap + B_own - 1) / B_own;
  if (per_b < 1) per_b = 1;
  if (gx > per_b) gx = per_b;
  dp_muon_apply_push_kernel<<<dim3(gx, B_own), 256, 0, (cudaStream_t)stream>>>(a);
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_peer_sum(void* const* src_ptrs, int world, long long off, float* out,
                                       long long n, float scale, void* stream) {
  if (world < 1 || world > kMaxRanks || n <= 0) return -1;
  bool vec = (off & 3) == 0 && (n & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  for (int r = 0; r < world && vec; ++r) vec = (reinterpret_cast<uintptr_t>(src_ptrs[r]) & 15) == 0;
  if (vec) {
    long long blocks = (n / 4 + 1023) / 1024;
    if (blocks > 148 * 4) blocks = 148 * 4;
    if (blocks < 1) blocks = 1;
    peer_sum_v4_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(make_peers(src_ptrs, world), off, out, n / 4, world,
                                                                       scale);
    return (int)cudaGetLastError();
  }
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  peer_sum_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(make_peers(src_ptrs, world), off, out, n,
                                                                 world, scale);
  return (int)cudaGetLastError();
}

// out[r * m + i] = src_r[off + i], i < m, for every rank r.  off, m multiples of 4 elements; bases 16-byte aligned.
extern "C" TYR_EXPORT int tyr_peer_gather(void* const* src_ptrs, int world, long long off, float* out, long long m,
                                          void* stream) {
  if (world < 1 || world > kMaxRanks || m <= 0 || (m & 3) || (off & 3) || (reinterpret_cast<uintptr_t>(out) & 15)) return -1;
  for (int r = 0; r < world; ++r)
    if (reinterpret_cast<uintptr_t>(src_ptrs[r]) & 15) return -1;
  long long blocks = (m / 4 * world + 1023) / 1024;
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (blocks < 1) blocks = 1;
  peer_gather_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(make_peers(src_ptrs, world), off, out, m / 4, world);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Second half of the fused GEMM -> reduce-scatter: the GEMM epilogues of all ranks have stored their
// bf16 partial tiles into this rank's slot buffer [world][n]; sum the slots in fp32 (plus an optional
// residual) and round once.
// ---------------------------------------------------------------------------------------------
namespace tyr {
__global__ void __launch_bounds__(256)
slot_sum_bf16_kernel(const __nv_bfloat16* __restrict__ slots, int world, long long n, const __nv_bfloat16* __restrict__ add,
                     __nv_bfloat16* __restrict__ out) {
  pdl_entry();
  const long long nvec = n >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {
      const uint4 u = *reinterpret_cast<const uint4*>(slots + r * n + i * 8);
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
    if (add) {
      const uint4 u = *reinterpret_cast<const uint4*>(add + i * 8);
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + i * 8) = o;
  }
}
}  // namespace tyr

extern "C" TYR_EXPORT int tyr_slot_sum_bf16(const void* slots, int world, long long n, const void* add, void* out,
                                            void* stream) {
  if (world < 1 || world > tyr::kMaxRanks || n <= 0 || (n & 7)) return -1;
  long long blocks = (n / 8 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  tyr::launch_dependent(tyr::slot_sum_bf16_kernel, dim3((int)blocks), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)slots, world, n,
                                                                          (const __nv_bfloat16*)add, (__nv_bfloat16*)out);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// One-shot all-reduce for the small activations of tensor-parallel decode: every rank has published
// its bf16 partial [n] in symmetric memory; each rank reads all of them over NVLink (plain peer
// loads, 16 B per thread), sums in fp32 (plus an optional residual) and rounds once.
// ---------------------------------------------------------------------------------------------
namespace tyr {
__global__ void __launch_bounds__(256)
peer_sum_bf16_kernel(PeerPtrs src, int world, long long n, const __nv_bfloat16* __restrict__ add, __nv_bfloat16* __restrict__ out) {
  pdl_entry();
  const long long nvec = n >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    uint4 u[kMaxRanks];
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < world) u[r] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(src.p[r]) + i * 8);
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < world) {
        const float2 a = unpack_bf16x2(u[r].x), b = unpack_bf16x2(u[r].y), c = unpack_bf16x2(u[r].z), d = unpack_bf16x2(u[r].w);
        acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
      }
    if (add) {
      const uint4 v = *reinterpret_cast<const uint4*>(add + i * 8);
      const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + i * 8) = o;
  }
}
}  // namespace tyr

// ---------------------------------------------------------------------------------------------
// Decode-sized all-reduce of a tensor-parallel sub-layer, with everything that follows it, in one launch:
//   flag barrier (this rank's partial is published, every peer's partial is waited for, bounded)
//   -> x = sum over ranks of the bf16 partials [M, N] (peer loads) + residual
//   -> out_resid = bf16(x);  out_norm = RMSNorm(out_resid) * (w or 1 + w)   (the next sub-layer's input)
// One CTA per row; the row stays in registers between the sum and the norm.  The barrier's sequence number lives in device
// memory (the same counter as tyr_barrier_dev uses for the slot), advanced by the last CTA to finish, so the launch can be
// replayed from a CUDA graph.  Replaces a barrier launch, a peer-sum launch and a norm launch.
// ---------------------------------------------------------------------------------------------
namespace tyr {
struct TpArNormArgs {
  PeerPtrs part;
  PeerPtrs flags;
  const unsigned long long* local_flags;
  unsigned long long* seq;
  int* done;
  const __nv_bfloat16* resid;
  const __nv_bfloat16* norm_w;
  __nv_bfloat16* out_resid;
  __nv_bfloat16* out_norm;
  int world, my_rank, slot_base, M, N, one_plus_w;
  float eps;
  int* err;
};

constexpr int kArVecs = 4;      // 16-byte vectors per thread: N <= 256 * 4 * 8 = 8192

__global__ void __launch_bounds__(256) tp_allreduce_norm_kernel(TpArNormArgs a) {
  pdl_entry();
  __shared__ float red[8];
  const int tid = threadIdx.x;
  const unsigned long long value = *a.seq + 1;
  if (blockIdx.x == 0 && tid < a.world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<unsigned long long*>(a.flags.p[tid]) + a.slot_base + a.my_rank, value);
  }
  if (tid < a.world) {
    const unsigned long long* f = a.local_flags + a.slot_base + tid;
    const long long start = clock64();
    while (ld_acquire_sys(f) < value) {
      if (clock64() - start > kWaitBudgetCycles * 4) {
        report_error(a.err, ERR_PEER_FLAG_TIMEOUT, a.slot_base + tid);
        break;
      }
      __nanosleep(40);
    }
  }
  __syncthreads();
  const int row = blockIdx.x;
  const int nvec = a.N >> 3;
  float x[kArVecs][8];
  float sq = 0.f;
#pragma unroll
  for (int j = 0; j < kArVecs; ++j) {
    const int v = tid + j * 256;
    if (v < nvec) {
      const long long off = static_cast<long long>(row) * a.N + v * 8;
      uint4 u[kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < a.world) {
          const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(a.part.p[r]) + off;
          asm volatile("ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(u[r].x), "=r"(u[r].y), "=r"(u[r].z), "=r"(u[r].w)
                       : "l"(p));
        }
#pragma unroll
      for (int e = 0; e < 8; ++e) x[j][e] = 0.f;
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < a.world) {
          const float2 p0 = unpack_bf16x2(u[r].x), p1 = unpack_bf16x2(u[r].y), p2 = unpack_bf16x2(u[r].z), p3 = unpack_bf16x2(u[r].w);
          x[j][0] += p0.x; x[j][1] += p0.y; x[j][2] += p1.x; x[j][3] += p1.y;
          x[j][4] += p2.x; x[j][5] += p2.y; x[j][6] += p3.x; x[j][7] += p3.y;
        }
      if (a.resid) {
        const uint4 rv = *reinterpret_cast<const uint4*>(a.resid + off);
        const float2 p0 = unpack_bf16x2(rv.x), p1 = unpack_bf16x2(rv.y), p2 = unpack_bf16x2(rv.z), p3 = unpack_bf16x2(rv.w);
        x[j][0] += p0.x; x[j][1] += p0.y; x[j][2] += p1.x; x[j][3] += p1.y;
        x[j][4] += p2.x; x[j][5] += p2.y; x[j][6] += p3.x; x[j][7] += p3.y;
      }
      uint4 o;
      o.x = pack_bf16x2(x[j][0], x[j][1]); o.y = pack_bf16x2(x[j][2], x[j][3]);
      o.z = pack_bf16x2(x[j][4], x[j][5]); o.w = pack_bf16x2(x[j][6], x[j][7]);
      *reinterpret_cast<uint4*>(a.out_resid + off) = o;
      // the norm sees the rounded residual stream, like a separate norm kernel would
      const float2 q0 = unpack_bf16x2(o.x), q1 = unpack_bf16x2(o.y), q2 = unpack_bf16x2(o.z), q3 = unpack_bf16x2(o.w);
      x[j][0] = q0.x; x[j][1] = q0.y; x[j][2] = q1.x; x[j][3] = q1.y; x[j][4] = q2.x; x[j][5] = q2.y; x[j][6] = q3.x; x[j][7] = q3.y;
#pragma unroll
      for (int e = 0; e < 8; ++e) sq += x[j][e] * x[j][e];
    }
  }
  if (a.out_norm != nullptr) {
    sq = warp_sum(sq);
    if ((tid & 31) == 0) red[tid >> 5] = sq;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float rstd = rsqrtf(tot / static_cast<float>(a.N) + a.eps);
#pragma unroll
    for (int j = 0; j < kArVecs; ++j) {
      const int v = tid + j * 256;
      if (v < nvec) {
        const uint4 wv = *reinterpret_cast<const uint4*>(a.norm_w + v * 8);
        const float2 w0 = unpack_bf16x2(wv.x), w1 = unpack_bf16x2(wv.y), w2 = unpack_bf16x2(wv.z), w3 = unpack_bf16x2(wv.w);
        const float wf[8] = {w0.x, w0.y, w1.x, w1.y, w2.x, w2.y, w3.x, w3.y};
        float y[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = x[j][e] * rstd * (a.one_plus_w ? 1.f + wf[e] : wf[e]);
        uint4 o;
        o.x = pack_bf16x2(y[0], y[1]); o.y = pack_bf16x2(y[2], y[3]); o.z = pack_bf16x2(y[4], y[5]); o.w = pack_bf16x2(y[6], y[7]);
        *reinterpret_cast<uint4*>(a.out_norm + static_cast<long long>(row) * a.N + v * 8) = o;
      }
    }
  }
  // the last CTA to get here advances the barrier's sequence number (every CTA has read it by then)
  __syncthreads();
  if (tid == 0) {
    if (atomicAdd(a.done, 1) == static_cast<int>(gridDim.x) - 1) {
      *a.done = 0;
      __threadfence();
      *a.seq = value;
    }
  }
}
}  // namespace tyr

// part_ptrs / flag_ptrs: per-rank base pointers of the bf16 partial [M, N] and of the flag array; `seq` is the slot's device
// counter, `done` a zeroed int.  resid, norm_w, out_norm may be null.  N % 8 == 0, N <= 8192, 16-byte aligned pointers.
extern "C" TYR_EXPORT int tyr_tp_allreduce_norm(void* const* part_ptrs, void* const* flag_ptrs, const void* local_flags, int world,
                                                int my_rank, int slot_base, void* seq, int* done, const void* resid,
                                                const void* norm_w, void* out_resid, void* out_norm, int M, int N, int one_plus_w,
                                                float eps, int* err, void* stream) {
  using namespace tyr;
  if (world < 1 || world > kMaxRanks || M <= 0 || N <= 0 || (N & 7) || N > 256 * kArVecs * 8) return -1;
  if (out_resid == nullptr || seq == nullptr || done == nullptr || (out_norm != nullptr && norm_w == nullptr)) return -1;
  uintptr_t al = reinterpret_cast<uintptr_t>(resid) | reinterpret_cast<uintptr_t>(norm_w) | reinterpret_cast<uintptr_t>(out_resid) |
                 reinterpret_cast<uintptr_t>(out_norm);
  for (int r = 0; r < world; ++r) al |= reinterpret_cast<uintptr_t>(part_ptrs[r]);
  if (al & 15) return -2;
  TpArNormArgs a;
  a.part = make_peers(part_ptrs, world);
  a.flags = make_peers(flag_ptrs, world);
  a.local_flags = (const unsigned long long*)local_flags;
  a.seq = (unsigned long long*)seq; a.done = done;
  a.resid = (const __nv_bfloat16*)resid; a.norm_w = (const __nv_bfloat16*)norm_w;
  a.out_resid = (__nv_bfloat16*)out_resid; a.out_norm = (__nv_bfloat16*)out_norm;
  a.world = world; a.my_rank = my_rank; a.slot_base = slot_base; a.M = M; a.N = N; a.one_plus_w = one_plus_w; a.eps = eps; a.err = err;
  launch_dependent(tp_allreduce_norm_kernel, dim3(M), dim3(256), 0, (cudaStream_t)stream, a);
  return (int)cudaGetLastError();
}

// Column gather of a vocabulary-parallel product: every rank holds y_r [M, Nl] bf16 at the same offset of its heap;
// out[m, r * Nl + c] = y_r[m, c] on every rank, read with 16-byte peer loads (Nl % 8 == 0).  The caller orders it after a flag
// barrier.  Replaces an NCCL all-gather plus a concatenation.
namespace tyr {
__global__ void __launch_bounds__(256)
peer_gather_cols_bf16_kernel(PeerPtrs src, int world, int M, int Nl, __nv_bfloat16* __restrict__ out) {
  pdl_entry();
  const int vpr = Nl >> 3;                                    // vectors per source row
  const long long total = static_cast<long long>(world) * M * vpr;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < total; i0 += 4 * stride) {
    uint4 t[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * stride;
      if (i < total) {
        const int r = static_cast<int>(i / (static_cast<long long>(M) * vpr));
        const long long j = i - static_cast<long long>(r) * M * vpr;
        const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(src.p[r]) + j * 8;
        asm volatile("ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(t[u].x), "=r"(t[u].y), "=r"(t[u].z), "=r"(t[u].w)
                     : "l"(p));
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * stride;
      if (i < total) {
        const int r = static_cast<int>(i / (static_cast<long long>(M) * vpr));
        const long long j = i - static_cast<long long>(r) * M * vpr;
        const int m = static_cast<int>(j / vpr), c = static_cast<int>(j - static_cast<long long>(m) * vpr);
        *reinterpret_cast<uint4*>(out + (static_cast<long long>(m) * world + r) * Nl + c * 8) = t[u];
      }
    }
  }
}
}  // namespace tyr

extern "C" TYR_EXPORT int tyr_peer_gather_cols_bf16(void* const* src_ptrs, int world, int M, int Nl, void* out, void* stream) {
  if (world < 1 || world > tyr::kMaxRanks || M <= 0 || Nl <= 0 || (Nl & 7) || (reinterpret_cast<uintptr_t>(out) & 15)) return -1;
  for (int r = 0; r < world; ++r)
    if (reinterpret_cast<uintptr_t>(src_ptrs[r]) & 15) return -1;
  long long blocks = (static_cast<long long>(world) * M * (Nl >> 3) + 1023) / 1024;
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (blocks < 1) blocks = 1;
  tyr::launch_dependent(tyr::peer_gather_cols_bf16_kernel, dim3((int)blocks), dim3(256), 0, (cudaStream_t)stream, make_peers(src_ptrs, world), world, M, Nl,
                                                                                   (__nv_bfloat16*)out);
  return (int)cudaGetLastError();
}

extern "C" TYR_EXPORT int tyr_peer_sum_bf16(void* const* src_ptrs, int world, long long n, const void* add, void* out,
                                            void* stream) {
  if (world < 1 || world > tyr::kMaxRanks || n <= 0 || (n & 7)) return -1;
  long long blocks = (n / 8 + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  tyr::launch_dependent(tyr::peer_sum_bf16_kernel, dim3((int)blocks), dim3(256), 0, (cudaStream_t)stream, make_peers(src_ptrs, world), world, n,
                                                                          (const __nv_bfloat16*)add, (__nv_bfloat16*)out);
  return (int)cudaGetLastError();
}
