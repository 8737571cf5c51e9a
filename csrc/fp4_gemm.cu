// Block-scaled NVFP4 grouped GEMM for the MoE experts on the 5th-generation tensor cores:
//   tcgen05.mma.kind::mxf4nvf4.block_scale  (e2m1 values, one UE4M3 scale per 16 elements, fp32 accumulate in TMEM)
//
//   C[rows of expert e, :] = (A_q . sa) (W_q[e] . sw[e])^T * row_scale_a / global_w[e]
//
// Both operands stay 4-bit from HBM to the tensor core: the weights are the checkpoint's banks (packed e2m1 bytes and
// UE4M3 block scales, re-laid once at load time), the activations are quantised on the fly by the gather kernel below
// (dynamic UE4M3 block scales under one fp32 scale per row).  Nothing is dequantised to bf16 and no dense copy of a
// bank exists.
//
// Data layout
//   * values: K-major, two e2m1 codes per byte (even element in the low nibble), rows of K/2 bytes; tiles of
//     128 rows x 128 bytes (256 elements) are fetched by TMA with the 128-byte swizzle.
//   * block scales: the tensor core's own order.  Per 128-row tile and per 64 elements of K one 512-byte chunk,
//       byte (row % 32) * 16 + (row / 32) * 4 + (k / 16) % 4,
//     chunks ordered [row tile][K / 64]; the four chunks of a 256-element stage are contiguous (2 KB, one bulk copy).
//     `tcgen05.cp.32x128b.warpx4` moves a chunk from shared memory into four TMEM columns.
//   * rows: every expert's rows start at a multiple of 128 (`128 * group_tiles[e]`, the exclusive prefix sum of
//     ceil(rows_e / 128) the routing kernels already produce), so a row tile never straddles two experts and the scale
//     chunks line up with the tiles.  Padding rows are computed and ignored.
//   * fixed-slot form (at most 128 tokens): expert e owns the padded rows [128 e, 128 e + 128), a row takes its slot with
//     one atomic on the expert's cursor (fp4_scatter_quantize_fixed_kernel) and the GEMM reads the cursors as row counts
//     (`group_tiles == nullptr`): its tile table counts only the experts that have rows.
//
// Kernel: persistent, 320 threads: warp 0 TMA producer (5 stages of 36 KB), warp 1 MMA issuer (scale copies + four
// K = 64 MMAs per stage, double-buffered 128-column accumulator), warps 2-9 epilogue.  Epilogues:
//   mode 0  bf16 store (down projection)
//   mode 1  SwiGLU over the tile's column halves (64 gate | 64 up rows interleaved at load time), then re-quantisation
//           of the 64 results to NVFP4 (values + scale bytes in the layout above): the down projection consumes them
//           without another pass.
// Every wait is bounded; a timeout records an error and unwinds through the normal teardown.  The kernel is launched as a
// programmatic dependent: barrier init, TMEM allocation and (when every expert is expected to have rows) an L2 prefetch of
// the first tiles' weights run before it waits for the kernel that produces its activations and row counts.
//
// The reference reaches a block-scaled tensor-core product only through cuBLASLt and only on compute capability 12
// (cc/src/tyr_laguna_moe.cu:839-982, gate at :1317-1319; scale order :612-627; activation quantisation :678-728;
// SwiGLU + re-quantise :730-766); on B200 it runs SIMT GEMV kernels.
#include "common.cuh"
#include <cuda_fp8.h>
#include <mutex>

namespace tyr {

constexpr int F4_BM = 128;
constexpr int F4_BN = 128;
constexpr int F4_BKB = 128;            // bytes of K per stage = 256 e2m1 elements = four MMAs of K = 64
constexpr int F4_STAGES = 5;
constexpr int F4_SF_STAGE = 2048;      // scale bytes per 128 rows and stage
constexpr uint32_t F4_COL_SFA = 256;   // TMEM columns: accumulators 0..255, then 16 columns per stage for each operand's scales
constexpr uint32_t F4_COL_SFB = 256 + 16 * F4_STAGES;
constexpr int F4_MAX_GROUPS = 1024;    // experts per call (their prefix tables are staged in shared memory)

struct Fp4Params {
  int N, K;                    // weight rows per expert, reduction length in elements (multiple of 256)
  int groups;                  // experts
  const int* group_tiles;      // [groups + 1] exclusive prefix of 128-row tiles (device memory)
  const int* group_rows;       // [groups + 1] exclusive prefix of true rows (device memory)
  const uint8_t* sfa;          // activation scales, tensor-core order over the padded rows
  const uint8_t* sfb;          // weight scales, tensor-core order, [groups][N / 128][K / 64][512]
  const uint8_t* w_tiled;      // weights as shared-memory images: [groups][N / 128][K / 256][128 rows x 128 bytes, 128B swizzle]
  const float* a_row_scale;    // [padded rows] or nullptr (= 1)
  const float* w_global;       // [groups]: result is divided by it
  const float* w_global2;      // mode 1: the global of the `up` bank (w_global is the gate bank's)
  int mode;
  int all_active;              // fixed-slot layout: the caller expects every expert to have rows (enables the weight prefetch)
  void* out;                   // mode 0: bf16 [padded rows, N]; mode 1: packed e2m1 [padded rows, N / 4] bytes
  uint8_t* out_sf;             // mode 1: scales of `out` in tensor-core order for a reduction length of N / 2
  int* err;
};

struct __align__(1024) Fp4Smem {
  uint8_t a[F4_STAGES][F4_BM * F4_BKB];
  uint8_t b[F4_STAGES][F4_BN * F4_BKB];
  uint8_t sfa[F4_STAGES][F4_SF_STAGE];
  uint8_t sfb[F4_STAGES][F4_SF_STAGE];
  uint64_t full[F4_STAGES];
  uint64_t empty[F4_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  // copies of the two per-expert prefix tables: every role finds a tile's expert by binary search, and with the tables in
  // global memory that was six dependent L2 round trips per tile in the producer (2 - 3 us during which the five-stage ring
  // ran dry: a decode-sized product has only three to eight stages per tile)
  int gt[F4_MAX_GROUPS + 1];
  int gr[F4_MAX_GROUPS + 1];
};

// kind::mxf4nvf4 instruction descriptor: e2m1 x e2m1 (format code 1), UE4M3 scales, K-major operands, dense K = 64.
__host__ __device__ constexpr uint32_t make_idesc_nvf4(int m, int n) {
  return (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (0u << 23) | (static_cast<uint32_t>(m >> 4) << 24);
}
// Shared-memory descriptor without swizzle for the scale chunks: 32 rows of 16 bytes, 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc_sf(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;   // stride byte offset between 8-row groups
  d |= 1ull << 46;
  return d;
}
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma_nvf4_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t tsfa, uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
      : "memory");
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// ---- e2m1 / UE4M3 helpers (round to nearest, ties to even, saturating) ---------------------------------------------
__device__ __forceinline__ uint32_t e2m1_code(float q) {
  const float a = fabsf(q);
  uint32_t m = 0;
  m += a > 0.25f;
  m += a >= 0.75f;
  m += a > 1.25f;
  m += a >= 1.75f;
  m += a > 2.5f;
  m += a >= 3.5f;
  m += a > 5.0f;
  return m | (q < 0.f ? 8u : 0u);
}
__device__ __forceinline__ uint8_t ue4m3_encode(float s) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(fminf(s, 448.f), __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float ue4m3_decode(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}
// offset of (row, 16-element block kb) in the tensor-core scale order, ktiles = K / 64
__device__ __forceinline__ long long sf_offset(int row, int kb, int ktiles) {
  return (static_cast<long long>(row >> 7) * ktiles + (kb >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (kb & 3);
}

// ---------------------------------------------------------------------------------------------------------------------
// Gather + quantise: expert-sorted position -> padded row; one warp per row.
//   x [T, h] bf16; pair_order[pos] = pair; ids[pair] = expert; offsets / group_tiles [E + 1]
//   out: packed [padded rows, h / 2], scales in tensor-core order, row_scale [padded rows], pair_ppos[pair] = padded row
// ---------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
fp4_gather_quantize_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ pair_order,
                           const int* __restrict__ ids, const int* __restrict__ offsets,
                           const int* __restrict__ group_tiles, uint8_t* __restrict__ packed, uint8_t* __restrict__ sf,
                           float* __restrict__ row_scale, int* __restrict__ pair_ppos, int pairs, int k, int h, int E) {
  pdl_entry();
  const int lane = threadIdx.x & 31;
  const int ktiles = h >> 6;
  for (int pos = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); pos < pairs; pos += gridDim.x * (blockDim.x >> 5)) {
    int tok = pos, prow = pos;
    if (pair_order != nullptr) {
      if (pos >= offsets[E]) continue;             // positions past the routed total (padding ids take no slot)
      const int pair = pair_order[pos];
      if (pair < 0 || pair >= pairs) continue;
      const int e = ids[pair];
      if (e < 0 || e >= E) continue;
      tok = pair / k;
      prow = 128 * group_tiles[e] + (pos - offsets[e]);
      if (lane == 0 && pair_ppos) pair_ppos[pair] = prow;
    }
    const __nv_bfloat16* src = x + static_cast<long long>(tok) * h;
    // pass 1: row maximum
    float amax = 0.f;
    for (int c = lane * 8; c < h; c += 256) {
      const uint4 u = *reinterpret_cast<const uint4*>(src + c);
      const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
      amax = fmaxf(amax, fmaxf(fmaxf(fabsf(f0.x), fabsf(f0.y)), fmaxf(fabsf(f1.x), fabsf(f1.y))));
      amax = fmaxf(amax, fmaxf(fmaxf(fabsf(f2.x), fabsf(f2.y)), fmaxf(fabsf(f3.x), fabsf(f3.y))));
    }
    amax = warp_max(amax);
    const float g = amax > 0.f ? amax * (1.f / (6.f * 448.f)) : 1.f;      // row scale: block scales fill UE4M3's range
    const float inv_g = 1.f / g;
    if (lane == 0) row_scale[prow] = g;
    // pass 2: 16-element blocks (two lanes share a block: 8 elements each)
    for (int c = lane * 8; c < h; c += 256) {
      const uint4 u = *reinterpret_cast<const uint4*>(src + c);
      float v[8];
      { const float2 f = unpack_bf16x2(u.x); v[0] = f.x; v[1] = f.y; }
      { const float2 f = unpack_bf16x2(u.y); v[2] = f.x; v[3] = f.y; }
      { const float2 f = unpack_bf16x2(u.z); v[4] = f.x; v[5] = f.y; }
      { const float2 f = unpack_bf16x2(u.w); v[6] = f.x; v[7] = f.y; }
      float bm = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) bm = fmaxf(bm, fabsf(v[j]));
      bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
      const uint8_t sb = ue4m3_encode(bm * inv_g * (1.f / 6.f));
      const float s = ue4m3_decode(sb) * g;
      const float inv_s = s > 0.f ? 1.f / s : 0.f;
      uint32_t w = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) w |= e2m1_code(v[j] * inv_s) << (4 * j);
      *reinterpret_cast<uint32_t*>(packed + static_cast<long long>(prow) * (h >> 1) + (c >> 1)) = w;
      if ((lane & 1) == 0) sf[sf_offset(prow, c >> 4, ktiles)] = sb;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Decode-sized batches (T <= 128): quantise + scatter without a sorted layout.  Every expert owns the fixed row tile
// [128 e, 128 e + 128): a token can reach an expert once, so 128 slots always suffice, and a slot is taken with one atomic on
// the expert's cursor (zero on entry, the expert's row count on exit: the grouped GEMM reads it in place of its row table).
// One warp per token: the row is quantised once into shared memory and written to each of its k experts' slots.  Replaces the
// offsets / scatter / zero-fill / gather launches of the sorted layout.
constexpr int F4_SCATTER_WARPS = 4;

__global__ void __launch_bounds__(F4_SCATTER_WARPS * 32)
fp4_scatter_quantize_fixed_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids, int* __restrict__ cursors,
                                  uint8_t* __restrict__ packed, uint8_t* __restrict__ sf, float* __restrict__ row_scale,
                                  int* __restrict__ pair_ppos, int T, int k, int h, int E, int* err) {
  extern __shared__ __align__(16) uint8_t sq_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_bytes = (h >> 1) + (h >> 4);                 // packed values then scale bytes
  uint8_t* q = sq_smem + warp * ((row_bytes + 15) & ~15);
  uint8_t* qs = q + (h >> 1);
  const int ktiles = h >> 6;
  const int tok = blockIdx.x * F4_SCATTER_WARPS + warp;
  pdl_entry();
  if (tok >= T) return;
  const __nv_bfloat16* src = x + static_cast<long long>(tok) * h;
  float amax = 0.f;
  for (int c = lane * 8; c < h; c += 256) {
    const uint4 u = *reinterpret_cast<const uint4*>(src + c);
    const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(f0.x), fabsf(f0.y)), fmaxf(fabsf(f1.x), fabsf(f1.y))));
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(f2.x), fabsf(f2.y)), fmaxf(fabsf(f3.x), fabsf(f3.y))));
  }
  amax = warp_max(amax);
  const float g = amax > 0.f ? amax * (1.f / (6.f * 448.f)) : 1.f;
  const float inv_g = 1.f / g;
  for (int c = lane * 8; c < h; c += 256) {
    const uint4 u = *reinterpret_cast<const uint4*>(src + c);
    float v[8];
    { const float2 f = unpack_bf16x2(u.x); v[0] = f.x; v[1] = f.y; }
    { const float2 f = unpack_bf16x2(u.y); v[2] = f.x; v[3] = f.y; }
    { const float2 f = unpack_bf16x2(u.z); v[4] = f.x; v[5] = f.y; }
    { const float2 f = unpack_bf16x2(u.w); v[6] = f.x; v[7] = f.y; }
    float bm = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) bm = fmaxf(bm, fabsf(v[j]));
    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
    const uint8_t sb = ue4m3_encode(bm * inv_g * (1.f / 6.f));
    const float sdec = ue4m3_decode(sb) * g;
    const float inv_s = sdec > 0.f ? 1.f / sdec : 0.f;
    uint32_t w = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) w |= e2m1_code(v[j] * inv_s) << (4 * j);
    *reinterpret_cast<uint32_t*>(q + (c >> 1)) = w;
    if ((lane & 1) == 0) qs[c >> 4] = sb;
  }
  __syncwarp();
  for (int j = 0; j < k; ++j) {
    const int pair = tok * k + j;
    const int e = ids[pair];
    if (e < 0 || e >= E) {                        // not routed (padding id): takes no slot
      if (lane == 0) pair_ppos[pair] = -1;
      continue;
    }
    int slot = 0;
    if (lane == 0) slot = atomicAdd(cursors + e, 1);
    slot = __shfl_sync(0xffffffffu, slot, 0);
    if (slot >= F4_BM) {                           // cannot happen while T <= 128; recorded, the row is dropped
      if (lane == 0) { report_error(err, ERR_BOUNDS, 1500); pair_ppos[pair] = -1; }
      continue;
    }
    const int prow = e * F4_BM + slot;
    uint8_t* dst = packed + static_cast<long long>(prow) * (h >> 1);
    for (int c = lane * 16; c < (h >> 1); c += 512) *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(q + c);
    for (int kb = lane; kb < (h >> 4); kb += 32) sf[sf_offset(prow, kb, ktiles)] = qs[kb];
    if (lane == 0) {
      row_scale[prow] = g;
      pair_ppos[pair] = prow;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// The GEMM
__global__ void __launch_bounds__(320, 1)
fp4_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, Fp4Params p) {
  extern __shared__ uint8_t smem_raw[];
  Fp4Smem& s = *reinterpret_cast<Fp4Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_n = p.N / F4_BN;
  const int num_ks = p.K / 256;                 // stages per tile
  const int ktiles = p.K >> 6;                  // 64-element scale chunks along K
  // set-up that reads nothing another kernel wrote: it may run while the kernel before this one drains
  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int i = 0; i < F4_STAGES; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.acc_full[i], 1);
      mbar_init(&s.acc_empty[i], 8);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&s.tmem_base, 512);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    if (p.all_active && p.group_tiles == nullptr) {
      // Which tiles this CTA gets depends on the row counts, which the kernel in front of this one is still writing.  When
      // (nearly) every expert has rows, tile t belongs to expert t / tiles_n: ask the L2 for the weights of the first tiles
      // under that assumption.  A wrong guess costs bandwidth, never correctness.
      const long long tiles_g = static_cast<long long>(p.groups) * tiles_n;
      const long long rounds_g = (tiles_g + gridDim.x - 1) / gridDim.x;
      const long long stride_g = (tiles_g + rounds_g - 1) / rounds_g;
      const int n_pref = num_ks >= 8 ? 1 : 8 / num_ks;
      if (blockIdx.x < stride_g)
        for (int i = 0; i < n_pref; ++i) {
          const long long t = blockIdx.x + i * stride_g;
          if (t >= tiles_g) break;
          bulk_prefetch_l2(p.w_tiled + t * num_ks * (F4_BN * F4_BKB), static_cast<uint32_t>(num_ks) * (F4_BN * F4_BKB));
          bulk_prefetch_l2(p.sfb + t * ktiles * 512, static_cast<uint32_t>(ktiles) * 512);
        }
    }
  }
  pdl_wait();
  if (p.group_tiles != nullptr) {
    for (int i = threadIdx.x; i <= p.groups; i += blockDim.x) {
      s.gt[i] = p.group_tiles[i];
      s.gr[i] = p.group_rows[i];
    }
  } else {
    // fixed-slot layout (decode-sized batches): expert e owns the padded rows [128 e, 128 e + 128) and `group_rows` holds the
    // experts' row COUNTS.  The tile table counts the experts that have rows, so an expert without rows costs no tile.
    if (warp == 0) {
      int carry_t = 0, carry_r = 0;
      if (lane == 0) s.gt[0] = s.gr[0] = 0;
      for (int base = 0; base < p.groups; base += 32) {
        const int i = base + lane;
        const int c = i < p.groups ? min(max(p.group_rows[i], 0), F4_BM) : 0;
        int t = c > 0 ? 1 : 0, r = c;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int tt = __shfl_up_sync(0xffffffffu, t, d), rr = __shfl_up_sync(0xffffffffu, r, d);
          if (lane >= d) { t += tt; r += rr; }
        }
        if (i < p.groups) {
          s.gt[i + 1] = carry_t + t;
          s.gr[i + 1] = carry_r + r;
        }
        carry_t += __shfl_sync(0xffffffffu, t, 31);
        carry_r += __shfl_sync(0xffffffffu, r, 31);
      }
    }
  }
  const bool fixed_slots = p.group_tiles == nullptr;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const long long tiles = static_cast<long long>(s.gt[p.groups]) * tiles_n;
  // The number of tiles is only known on the device.  All CTAs take the same number of rounds; the stride is the smallest
  // number of CTAs that finishes in that many rounds, so no round runs on a fraction of the SMs while the rest idle
  // (768 tiles on 148 SMs: 128 CTAs do six rounds each instead of 28 CTAs doing a sixth round alone).  The CTAs beyond the
  // stride find no tile.
  const long long rounds = (tiles + gridDim.x - 1) / gridDim.x;
  const long long stride = rounds > 0 ? (tiles + rounds - 1) / rounds : 1;
  const long long tile0 = blockIdx.x < stride ? blockIdx.x : tiles;

  const uint32_t tmem_base = s.tmem_base;
  constexpr uint32_t kStageBytes = F4_BM * F4_BKB + F4_BN * F4_BKB + 2 * F4_SF_STAGE;

  // -> expert e, padded row tile mt, column tile nt, lt = index of the row tile inside the expert
  auto decode = [&](long long tile, int& e, int& mt, int& nt, int& lt) {
    mt = static_cast<int>(tile / tiles_n);       // n fastest: the CTAs in flight share a row tile of activations
    nt = static_cast<int>(tile % tiles_n);
    int lo = 0, hi = p.groups;                   // group_tiles[lo] <= mt < group_tiles[hi]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s.gt[mid] <= mt) lo = mid; else hi = mid;
    }
    e = lo;
    lt = mt - s.gt[e];
    if (fixed_slots) mt = e;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (long long tile = tile0; tile < tiles && ok; tile += stride) {
        int e, mt, nt, lt;
        decode(tile, e, mt, nt, lt);
        const uint8_t* sfa = p.sfa + static_cast<long long>(mt) * ktiles * 512;
        const uint8_t* sfb = p.sfb + (static_cast<long long>(e) * tiles_n + nt) * ktiles * 512;
        // the weight tile of a stage is one contiguous 16 KB image (rows already swizzled): a plain bulk copy, and DRAM sees
        // 16 KB bursts instead of 128 separate 128-byte row segments
        const uint8_t* wt = p.w_tiled + (static_cast<long long>(e) * tiles_n + nt) * num_ks * (F4_BN * F4_BKB);
        for (int ks = 0; ks < num_ks; ++ks, ++it) {
          const int st = it % F4_STAGES;
          const uint32_t ph = (it / F4_STAGES) & 1;
          if (!mbar_wait(&s.empty[st], ph ^ 1, p.err, 1100 + st)) { ok = false; break; }
          mbar_expect_tx(&s.full[st], kStageBytes);
          tma_load_2d(s.a[st], &tmA, &s.full[st], ks * F4_BKB, mt * F4_BM);
          bulk_load(s.b[st], wt + static_cast<long long>(ks) * (F4_BN * F4_BKB), F4_BN * F4_BKB, &s.full[st]);
          bulk_load(s.sfa[st], sfa + static_cast<long long>(ks) * F4_SF_STAGE, F4_SF_STAGE, &s.full[st]);
          bulk_load(s.sfb[st], sfb + static_cast<long long>(ks) * F4_SF_STAGE, F4_SF_STAGE, &s.full[st]);
        }
      }
      if (!ok)   // let the copies in flight land before the CTA unwinds
        for (uint32_t j = (it > F4_STAGES ? it - F4_STAGES : 0); j < it; ++j)
          mbar_wait(&s.full[j % F4_STAGES], (j / F4_STAGES) & 1, nullptr, 0);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_nvf4(F4_BM, F4_BN);
      uint32_t it = 0, seg = 0;
      bool ok = true;
      for (long long tile = tile0; tile < tiles && ok; tile += stride, ++seg) {
        const uint32_t buf = seg & 1;
        if (!mbar_wait(&s.acc_empty[buf], ((seg >> 1) & 1) ^ 1, p.err, 1200 + buf)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * F4_BN;
        for (int ks = 0; ks < num_ks; ++ks, ++it) {
          const int st = it % F4_STAGES;
          if (!mbar_wait(&s.full[st], (it / F4_STAGES) & 1, p.err, 1300 + st)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(s.a[st]), b_addr = smem_u32(s.b[st]);
          const uint32_t sfa_t = tmem_base + F4_COL_SFA + st * 16, sfb_t = tmem_base + F4_COL_SFB + st * 16;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            tmem_cp_sf(sfa_t + c * 4, make_smem_desc_sf(smem_u32(s.sfa[st]) + c * 512));
            tmem_cp_sf(sfb_t + c * 4, make_smem_desc_sf(smem_u32(s.sfb[st]) + c * 512));
          }
#pragma unroll
          for (int c = 0; c < 4; ++c)
            umma_nvf4_ss(d_tmem, make_smem_desc_sw128(a_addr + c * 32, 16, 1024), make_smem_desc_sw128(b_addr + c * 32, 16, 1024),
                         idesc, sfa_t + c * 4, sfb_t + c * 4, (ks > 0 || c > 0) ? 1u : 0u);
          umma_commit(&s.empty[st]);
        }
        if (ok) umma_commit(&s.acc_full[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: 8 warps, two per TMEM lane quarter
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;          // mode 0: columns [64 half, 64 half + 64); mode 1: 32 of the 64 results
    uint32_t seg = 0;
    bool ok = true;
    for (long long tile = tile0; tile < tiles && ok; tile += stride, ++seg) {
      int e, mt, nt, lt;
      decode(tile, e, mt, nt, lt);
      const uint32_t buf = seg & 1;
      if (!mbar_wait(&s.acc_full[buf], (seg >> 1) & 1, p.err, 1400 + buf)) { ok = false; break; }
      tc_fence_after();
      const int prow = mt * F4_BM + quarter * 32 + lane;                       // padded row
      const int local = lt * F4_BM + quarter * 32 + lane;                      // row inside the expert
      const bool row_ok = local < s.gr[e + 1] - s.gr[e];
      const uint32_t t_row = tmem_base + buf * F4_BN + (static_cast<uint32_t>(quarter * 32) << 16);
      const float sa = p.a_row_scale ? p.a_row_scale[prow] : 1.f;
      if (p.mode == 0) {
        const float f = sa / p.w_global[e];
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(prow) * p.N + nt * F4_BN + half * 64;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + half * 64 + c * 32, r);
          tmem_wait_ld();
          if (c == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s.acc_empty[buf]);
          }
          if (!row_ok) continue;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(r[q * 8 + 0]) * f, __uint_as_float(r[q * 8 + 1]) * f);
            u.y = pack_bf16x2(__uint_as_float(r[q * 8 + 2]) * f, __uint_as_float(r[q * 8 + 3]) * f);
            u.z = pack_bf16x2(__uint_as_float(r[q * 8 + 4]) * f, __uint_as_float(r[q * 8 + 5]) * f);
            u.w = pack_bf16x2(__uint_as_float(r[q * 8 + 6]) * f, __uint_as_float(r[q * 8 + 7]) * f);
            *reinterpret_cast<uint4*>(out + c * 32 + q * 8) = u;
          }
        }
      } else {
        // gate columns [32 half, +32) and the matching up columns at +64: h = silu(gate) * up, then NVFP4 with a global of 1
        uint32_t rg[32], ru[32];
        tmem_ld_32x32(t_row + half * 32, rg);
        tmem_ld_32x32(t_row + 64 + half * 32, ru);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.acc_empty[buf]);
        const float fg = sa / p.w_global[e], fu = sa / p.w_global2[e];
        float hv[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float g = __uint_as_float(rg[j]) * fg;
          hv[j] = row_ok ? (g / (1.f + __expf(-g))) * (__uint_as_float(ru[j]) * fu) : 0.f;
        }
        const int kdown = p.N >> 1;                          // reduction length of the consumer
        uint32_t words[4];
        uint8_t sb[2];
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          float bm = 0.f;
#pragma unroll
          for (int j = 0; j < 16; ++j) bm = fmaxf(bm, fabsf(hv[b * 16 + j]));
          sb[b] = ue4m3_encode(bm * (1.f / 6.f));
          const float sdec = ue4m3_decode(sb[b]);
          const float inv_s = sdec > 0.f ? 1.f / sdec : 0.f;
#pragma unroll
          for (int w = 0; w < 2; ++w) {
            uint32_t acc = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc |= e2m1_code(hv[b * 16 + w * 8 + j] * inv_s) << (4 * j);
            words[b * 2 + w] = acc;
          }
        }
        const int col = nt * 64 + half * 32;                 // first of my 32 result columns
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.out) + static_cast<long long>(prow) * (kdown >> 1) + (col >> 1)) =
            make_uint4(words[0], words[1], words[2], words[3]);
        *reinterpret_cast<uint16_t*>(p.out_sf + sf_offset(prow, col >> 4, kdown >> 6)) =
            static_cast<uint16_t>(sb[0]) | (static_cast<uint16_t>(sb[1]) << 8);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---- host ------------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn f4_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}
// bytes [rows, kbytes] row-major, box 128 bytes x 128 rows, 128-byte swizzle
static int make_tmap_u8(CUtensorMap* tm, const void* base, uint64_t kbytes, uint64_t rows) {
  EncodeTiledFn fn = f4_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {kbytes, rows};
  cuuint64_t strides[1] = {kbytes};
  cuuint32_t box[2] = {128, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

}  // namespace tyr

using namespace tyr;

extern "C" {

// x [T, h] bf16 -> NVFP4 rows at their padded, expert-major positions (pair_order == nullptr: row i stays row i and
// `pairs` rows are converted, the dense case).  packed [padded_rows, h / 2]; sf: padded_rows / 128 * (h / 64) * 512 bytes.
TYR_EXPORT int tyr_fp4_gather_quantize(const void* x, const int* pair_order, const int* ids, const int* offsets,
                                       const int* group_tiles, void* packed, void* sf, float* row_scale, int* pair_ppos,
                                       int pairs, int k, int h, int E, void* stream) {
  if (pairs <= 0 || h <= 0 || (h & 255) || k <= 0) return -1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(packed)) & 15) return -2;
  long long blocks = (pairs + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  launch_dependent(fp4_gather_quantize_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
      reinterpret_cast<const __nv_bfloat16*>(x), pair_order, ids, offsets, group_tiles, reinterpret_cast<uint8_t*>(packed),
      reinterpret_cast<uint8_t*>(sf), row_scale, pair_ppos, pairs, k, h, E);
  return static_cast<int>(cudaGetLastError());
}

// Quantise + scatter into the fixed-slot layout (T <= 128 tokens; see fp4_scatter_quantize_fixed_kernel).  `cursors` [E]
// int32 zero on entry; packed [128 E, h / 2]; sf 128 E / 128 * (h / 64) * 512 bytes; row_scale [128 E]; pair_ppos [T k].
TYR_EXPORT int tyr_fp4_scatter_quantize_fixed(const void* x, const int* ids, int* cursors, void* packed, void* sf, float* row_scale,
                                              int* pair_ppos, int T, int k, int h, int E, int* err, void* stream) {
  if (T <= 0 || T > F4_BM || h <= 0 || (h & 255) || k <= 0 || E <= 0) return -1;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(packed)) & 15) return -2;
  const size_t per_warp = (static_cast<size_t>(h >> 1) + (h >> 4) + 15) & ~static_cast<size_t>(15);
  const size_t smem = per_warp * F4_SCATTER_WARPS;
  if (smem > 48 * 1024) return -3;
  return static_cast<int>(launch_dependent(
      fp4_scatter_quantize_fixed_kernel, dim3((T + F4_SCATTER_WARPS - 1) / F4_SCATTER_WARPS), dim3(F4_SCATTER_WARPS * 32), smem,
      reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<const __nv_bfloat16*>(x), ids, cursors,
      reinterpret_cast<uint8_t*>(packed), reinterpret_cast<uint8_t*>(sf), row_scale, pair_ppos, T, k, h, E, err));
}

struct TyrFp4GemmArgs {
  const void* a_packed;      // [padded_rows, K / 2]
  const void* a_sf;
  const float* a_row_scale;  // nullable
  const void* w_packed;      // weight tiles as shared-memory images (ops/fp4.py tile_weights): [groups][N / 128][K / 256][16 KB]
  const void* w_sf;
  const float* w_global;     // [groups]
  const float* w_global2;    // mode 1
  const int* group_tiles;    // [groups + 1]; nullptr: fixed-slot layout (expert e = row tile e)
  const int* group_rows;     // [groups + 1] prefix of true rows; fixed-slot layout: [groups] row counts
  void* out;
  void* out_sf;
  int padded_rows, N, K, groups, mode;
  int sm_count;
  int all_active;            // fixed-slot layout only: 1 = the caller expects every group to have rows (weight prefetch hint)
  int* err;
  void* stream;
};

// Returns 0 on success; negative = invalid argument; positive = CUDA / driver error.
TYR_EXPORT int tyr_fp4_grouped_gemm(const TyrFp4GemmArgs* a) {
  if (a->padded_rows <= 0 || (a->padded_rows & 127) || a->N <= 0 || (a->N & 127) || a->K <= 0 || (a->K & 255) || a->groups <= 0 ||
      a->groups > F4_MAX_GROUPS)
    return -1;
  if (a->mode != 0 && a->mode != 1) return -2;
  if (a->group_rows == nullptr || (a->group_tiles == nullptr && a->padded_rows < a->groups * 128)) return -5;
  if (a->mode == 1 && (a->out_sf == nullptr || a->w_global2 == nullptr || ((a->N >> 1) & 63))) return -3;
  if ((reinterpret_cast<uintptr_t>(a->a_packed) | reinterpret_cast<uintptr_t>(a->w_packed) | reinterpret_cast<uintptr_t>(a->a_sf) |
       reinterpret_cast<uintptr_t>(a->w_sf) | reinterpret_cast<uintptr_t>(a->out)) & 15)
    return -4;
  CUtensorMap tmA;
  int r = make_tmap_u8(&tmA, a->a_packed, static_cast<uint64_t>(a->K) / 2, static_cast<uint64_t>(a->padded_rows));
  if (r) return 3000 + r;
  constexpr size_t smem = sizeof(Fp4Smem) + 1024;
  static bool configured[64] = {false};
  static int sms[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fp4_grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return 1000 + static_cast<int>(e);
    cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    configured[dev] = true;
  }
  Fp4Params p;
  p.N = a->N; p.K = a->K; p.groups = a->groups;
  p.group_tiles = a->group_tiles; p.group_rows = a->group_rows;
  p.sfa = reinterpret_cast<const uint8_t*>(a->a_sf); p.sfb = reinterpret_cast<const uint8_t*>(a->w_sf);
  p.w_tiled = reinterpret_cast<const uint8_t*>(a->w_packed);
  p.a_row_scale = a->a_row_scale; p.w_global = a->w_global; p.w_global2 = a->w_global2;
  p.mode = a->mode; p.all_active = a->all_active; p.out = a->out; p.out_sf = reinterpret_cast<uint8_t*>(a->out_sf); p.err = a->err;
  int grid = a->sm_count > 0 ? a->sm_count : sms[dev];
  const long long max_tiles = static_cast<long long>(a->padded_rows / 128) * (a->N / 128);
  if (max_tiles < grid) grid = static_cast<int>(max_tiles);
  if (grid < 1) grid = 1;
  cudaError_t e = launch_dependent(fp4_grouped_gemm_kernel, dim3(grid), dim3(320), smem, reinterpret_cast<cudaStream_t>(a->stream), tmA, p);
  return e == cudaSuccess ? 0 : 2000 + static_cast<int>(e);
}

}  // extern "C"
