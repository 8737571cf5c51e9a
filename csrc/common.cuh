// Shared device-side helpers for every sm_100a kernel in this library:
// PTX wrappers (mbarrier, TMA, tcgen05/TMEM), bounded waits and the error-word convention.
//
// Error-word convention: every kernel that can wait on something (an mbarrier, a peer flag)
// receives `int* err` pointing at a 4-int device record {code, block, detail, iterations}.
// A wait that exceeds its cycle budget stores a non-zero code there and the kernel unwinds
// through its normal teardown path (TMEM is freed, outstanding copies are drained with a
// bounded wait).  Host wrappers read the record after synchronising and raise.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda.h>
#include <stdint.h>
#include <stdlib.h>

#define TYR_EXPORT __attribute__((visibility("default")))

namespace tyr {

enum ErrCode : int {
  ERR_NONE = 0,
  ERR_MBAR_TIMEOUT = 1,
  ERR_PEER_FLAG_TIMEOUT = 2,
  ERR_BOUNDS = 3,
  ERR_TMEM = 4,
};

// ~1.0 s at 1.9 GHz; bounded so a lost arrival never hangs the GPU.
constexpr long long kWaitBudgetCycles = 2000000000LL;

__device__ __forceinline__ void report_error(int* err, int code, int detail) {
  if (err != nullptr) {
    if (atomicCAS(err, 0, code) == 0) {
      err[1] = blockIdx.x;
      err[2] = detail;
    }
  }
}

// Checked builds (-DTYR_BOUNDS_CHECK, library libtyr_kernels_checked.so): data-dependent indices (token ids, positions,
// expert ids, pair maps) are tested before use.  A violation is written once into a per-translation-unit record
// {ERR_BOUNDS, tag, index, limit} that `tyr_bounds_status_<unit>` copies out and clears, and the access is skipped or
// clamped; nothing traps.  Release builds compile the test away.
#ifdef TYR_BOUNDS_CHECK
static __device__ int g_bounds_record[4];
__device__ __forceinline__ bool index_ok(long long i, long long n, int tag) {
  if (i >= 0 && i < n) return true;
  if (atomicCAS(&g_bounds_record[0], 0, static_cast<int>(ERR_BOUNDS)) == 0) {
    g_bounds_record[1] = tag;
    g_bounds_record[2] = static_cast<int>(i);
    g_bounds_record[3] = static_cast<int>(n);
  }
  return false;
}
#define TYR_INDEX_OK(i, n, tag) ::tyr::index_ok((i), (n), (tag))
#define TYR_DEFINE_BOUNDS_STATUS(unit)                                                                   \
  extern "C" TYR_EXPORT int tyr_bounds_status_##unit(int* out4) {                                        \
    int zero[4] = {0, 0, 0, 0};                                                                          \
    cudaError_t e = cudaMemcpyFromSymbol(out4, ::tyr::g_bounds_record, sizeof(zero));                    \
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(::tyr::g_bounds_record, zero, sizeof(zero));            \
    return static_cast<int>(e);                                                                          \
  }
#else
#define TYR_INDEX_OK(i, n, tag) true
#define TYR_DEFINE_BOUNDS_STATUS(unit)
#endif

// ---- programmatic dependent launch ---------------------------------------------------------------------------------
// A kernel launched through `launch_dependent` may become resident while the kernel before it in the stream still
// runs: its CTAs take the slots that the earlier kernel's CTAs leave, so launch latency and the kernel's own set-up
// (barrier init, TMEM allocation, descriptor prefetch) overlap the earlier kernel's tail.  Contract for such a kernel:
// `pdl_trigger()` first (lets ITS successor do the same), then set-up that touches no global memory another kernel
// writes, then `pdl_wait()` before the first access to such memory; `pdl_wait` returns when every earlier kernel of the
// stream has completed and its writes are visible.  Both instructions do nothing in a kernel launched the plain way.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_entry() {
  pdl_trigger();
  pdl_wait();
}

// TYR_PDL=0 turns the launch attribute off (every kernel then starts after its predecessor has finished).
inline bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("TYR_PDL");
    return v == nullptr || v[0] != '0';
  }();
  return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait.  Returns true when the phase completed, false on timeout (error recorded).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err, int tag) {
  const uint32_t addr = smem_u32(bar);
  long long start = 0;
  uint32_t spins = 0;
  while (true) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
    ++spins;
    if ((spins & 0x3ff) == 0) {
      long long now = clock64();
      if (start == 0) start = now;
      if (now - start > kWaitBudgetCycles) {
        report_error(err, ERR_MBAR_TIMEOUT, tag);
        return false;
      }
      // Another role already failed: give up quickly so the CTA can unwind.
      if (err != nullptr && *reinterpret_cast<volatile int*>(err) != 0 &&
          now - start > 20000000LL)
        return false;
    }
  }
}

// Same bounded wait with acquire semantics at cluster scope: for barriers that threads of the peer CTA of a
// pair arrive on with `mbar_arrive_cluster`.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, int* err, int tag) {
  const uint32_t addr = smem_u32(bar);
  long long start = 0;
  uint32_t spins = 0;
  while (true) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
    ++spins;
    if ((spins & 0x3ff) == 0) {
      long long now = clock64();
      if (start == 0) start = now;
      if (now - start > kWaitBudgetCycles) {
        report_error(err, ERR_MBAR_TIMEOUT, tag);
        return false;
      }
      if (err != nullptr && *reinterpret_cast<volatile int*>(err) != 0 && now - start > 20000000LL) return false;
    }
  }
}

// ----------------------------------------------------------------------------------------
// Thread-block clusters (CTA pairs for cta_group::2)
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory location in CTA `rank` of this cluster (shared::cluster window).
__device__ __forceinline__ uint32_t mapa_shared(uint32_t cta_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(cta_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// Arrive on an mbarrier that may live in the peer CTA (address from mapa_shared).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// ----------------------------------------------------------------------------------------
// TMA (bulk tensor copies on this GPU's own memory; no load is ever multicast to several CTAs)
// ----------------------------------------------------------------------------------------
// Asks the L2 for `bytes` (a multiple of 16) from a 16-byte aligned global address; nothing waits for it.
__device__ __forceinline__ void bulk_prefetch_l2(const void* gptr, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gptr), "r"(bytes) : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const void* tmap, uint64_t* bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const void* tmap, uint64_t* bar, int x,
                                            int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_u32(dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// CTA-pair form: the destination is this CTA's shared memory, the mbarrier (a shared::cluster address) may be the
// pair leader's.  Every CTA still fetches its own tile from this GPU's memory.
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const void* tmap, uint32_t bar_cluster_addr, int x,
                                                 int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_u32(dst)), "l"(tmap), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// Asks for a tile to be brought into L2; completes nothing and signals nothing.
__device__ __forceinline__ void tma_prefetch_l2_3d(const void* tmap, int x, int y, int z) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" : : "l"(tmap), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const void* tmap, uint64_t* bar, int x,
                                            int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(smem_u32(dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const void* tmap, const void* src, int x, int y,
                                             int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
      :
      : "l"(tmap), "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ----------------------------------------------------------------------------------------
// tcgen05 / TMEM
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], bf16/fp16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// A operand taken from TMEM (used by attention: P stays on chip between the two GEMMs).
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier once every previously issued tcgen05.mma of this thread completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
// cta_group::2: one instruction drives the tensor cores of both CTAs of a pair (M = 256: 128 rows of A and half of B's
// columns from each CTA's shared memory at the same offsets; each CTA's TMEM receives its own 128 rows of D).
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives once on the mbarrier at `bar_cluster_addr` (own CTA or, through mapa_shared, the peer) when every MMA
// this thread issued for the pair has completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread t of the warp receives row (lane base + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
      : "memory");
}

// Shared-memory matrix descriptor for tcgen05.mma (128-byte swizzle, Blackwell version bit).
//   start address, leading byte offset, stride byte offset are encoded in 16-byte units.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= 1ull << 46;  // descriptor version for sm_100
  d |= 2ull << 61;  // SWIZZLE_128B
  return d;
}

// The descriptor of the tile `bytes` further on (a multiple of 16 that stays inside the same 256 KB window): one 32-bit add
// on the low word instead of rebuilding the descriptor.  The thread that issues the MMAs has about 64 cycles per 128 x 128 x 16
// instruction, so every instruction saved between two issues counts.
__device__ __forceinline__ uint64_t smem_desc_advance(uint64_t desc, uint32_t bytes) {
  const uint32_t lo = static_cast<uint32_t>(desc) + (bytes >> 4);
  return (desc & 0xFFFFFFFF00000000ull) | lo;
}

// Instruction descriptor for kind::f16 with bf16 (fmt=1) or fp16 (fmt=0) inputs, fp32 accum.
__host__ __device__ constexpr uint32_t make_idesc_f16(int fmt, int m, int n, int a_mn_major,
                                                      int b_mn_major) {
  return (1u << 4) | (static_cast<uint32_t>(fmt) << 7) | (static_cast<uint32_t>(fmt) << 10) |
         (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// ----------------------------------------------------------------------------------------
// small math helpers
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}

}  // namespace tyr
