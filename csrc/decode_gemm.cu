// Weight-streaming linear layers for 17 .. 64 rows on the tensor cores (tcgen05, accumulators in TMEM).
//
//   y[M, N] = x[M, K] W[N, K]^T                       (plain)
//   y[M, N] = silu(x Wg^T) * (x Wu^T)                 (gated: both matrices streamed once, SwiGLU in the epilogue)
//
// At these row counts the product is bound by reading W once.  The operands are swapped so that the WEIGHTS fill the
// 128-row side of the MMA: a CTA owns 128 weight rows, walks the whole contraction in 64-element steps, and per step TMA
// brings one [128 x 64] weight tile (two when gated) and the [MPAD x 64] activation tile into a ring of shared-memory
// stages; one thread issues `tcgen05.mma` (M = 128 weight rows, N = MPAD tokens, K = 16) into TMEM; four warps read the
// accumulator back (a lane is a weight row, a column a token) and store y transposed.  The activations are re-read from
// L2 once per 128 weight rows (the mma.sync kernel of csrc/skinny_gemm.cu re-reads them once per 16 rows, which is what
// bounds it above 16 rows).
//
// A matrix with few rows (a down projection: 40 tiles of 128 rows) would leave most SMs idle, so the contraction can be split
// over the CTAs of a thread-block cluster: every CTA of the cluster accumulates its share of K for the same 128 rows, the
// others store their fp32 partial sums into the first CTA's shared memory (distributed shared memory, after a cluster barrier
// that tells them its tensor core no longer reads there), and the first CTA adds them in its epilogue.  One launch, no
// workspace, no atomics.
//
// The weights are constants, so the producer issues the weight loads of the first ring stages BEFORE it waits for the
// kernel in front of it (programmatic dependent launch); only the activation loads wait.
//
// The reference has no decode-sized GEMM of its own: its linear layers go to the library (cc/src/tyr.cpp, linear op).
#include "common.cuh"

#include <mutex>

namespace tyr {

constexpr int DG_ROWS = 128;   // weight rows per CTA
constexpr int DG_BK = 64;      // contraction elements per stage (128 bytes: one swizzle row)

// SUB: 64-element blocks of the contraction per ring stage.  With two, a stage fetches 256 contiguous bytes of every weight
// row in two back-to-back copies (DRAM sees longer bursts per open page) at the price of fewer, larger stages.
template <int MPAD, bool GATED, int SUB>
struct DgCfg {
  static constexpr int kWBytes = SUB * DG_ROWS * DG_BK * 2;
  static constexpr int kXBytes = SUB * MPAD * DG_BK * 2;
  static constexpr int kStageBytes = (GATED ? 2 : 1) * kWBytes + kXBytes;
  static constexpr int kStages = (218 * 1024) / kStageBytes > 10 ? 10 : (218 * 1024) / kStageBytes;
  static constexpr int kTmemCols = (GATED ? 2 : 1) * MPAD < 32 ? 32 : (GATED ? 2 : 1) * MPAD;
};

template <int MPAD, bool GATED, int SUB>
struct __align__(1024) DgSmem {
  using C = DgCfg<MPAD, GATED, SUB>;
  uint8_t w[C::kStages][C::kWBytes];
  uint8_t w2[GATED ? C::kStages : 1][GATED ? C::kWBytes : 1024];
  uint8_t x[C::kStages][C::kXBytes];
  uint64_t full[C::kStages];
  uint64_t empty[C::kStages];
  uint64_t acc_full;
  uint32_t tmem_base;
};

struct DgParams {
  __nv_bfloat16* y;
  long long ldy;
  int M, N, K;
  int* err;
};

template <int MPAD, bool GATED, int SUB>
__global__ void __launch_bounds__(192, 1)
decode_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmW2,
                   const __grid_constant__ CUtensorMap tmX, DgParams p) {
  using C = DgCfg<MPAD, GATED, SUB>;
  using Smem = DgSmem<MPAD, GATED, SUB>;
  extern __shared__ uint8_t dg_smem_raw[];
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(dg_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  constexpr int COLS = (GATED ? 2 : 1) * MPAD;    // accumulator columns
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int ks = static_cast<int>(cluster_nctarank());      // CTAs that share this row tile's contraction
  const int cr = static_cast<int>(cluster_ctarank());
  const int row0 = static_cast<int>(blockIdx.x / ks) * DG_ROWS;
  const int nkb_all = p.K / (DG_BK * SUB);                   // ring stages over the whole contraction
  const int kb0 = nkb_all * cr / ks;
  const int nkb = nkb_all * (cr + 1) / ks - kb0;             // this CTA's ring stages: [kb0, kb0 + nkb)
  constexpr int kTile = DG_ROWS * DG_BK * 2;                 // one [128 x 64] weight block
  constexpr int kXTile = MPAD * DG_BK * 2;

  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    mbar_init(&s.acc_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&s.tmem_base, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s.tmem_base;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (elect_one()) {
      tma_prefetch_desc(&tmW);
      if (GATED) tma_prefetch_desc(&tmW2);
      tma_prefetch_desc(&tmX);
      // the ring is empty: the weights of its first stages need nothing from the kernel in front of this one
      const int head = nkb < C::kStages ? nkb : C::kStages;
      for (int kb = 0; kb < head; ++kb) {
        mbar_expect_tx(&s.full[kb], C::kStageBytes);
#pragma unroll
        for (int j = 0; j < SUB; ++j) {
          const int kx = ((kb0 + kb) * SUB + j) * DG_BK;
          tma_load_2d(s.w[kb] + j * kTile, &tmW, &s.full[kb], kx, row0);
          if (GATED) tma_load_2d(s.w2[kb] + j * kTile, &tmW2, &s.full[kb], kx, row0);
        }
      }
      pdl_wait();
      for (int kb = 0; kb < head; ++kb)
#pragma unroll
        for (int j = 0; j < SUB; ++j)
          tma_load_2d(s.x[kb] + j * kXTile, &tmX, &s.full[kb], ((kb0 + kb) * SUB + j) * DG_BK, 0);
      bool ok = true;
      int issued = head;
      for (int kb = head; kb < nkb; ++kb) {
        const int st = kb % C::kStages;
        const uint32_t ph = (kb / C::kStages) & 1;
        if (!mbar_wait(&s.empty[st], ph ^ 1, p.err, 1700 + st)) { ok = false; break; }
        mbar_expect_tx(&s.full[st], C::kStageBytes);
#pragma unroll
        for (int j = 0; j < SUB; ++j) {
          const int kx = ((kb0 + kb) * SUB + j) * DG_BK;
          tma_load_2d(s.w[st] + j * kTile, &tmW, &s.full[st], kx, row0);
          if (GATED) tma_load_2d(s.w2[st] + j * kTile, &tmW2, &s.full[st], kx, row0);
          tma_load_2d(s.x[st] + j * kXTile, &tmX, &s.full[st], kx, 0);
        }
        issued = kb + 1;
      }
      if (!ok)   // let the copies in flight land before the CTA unwinds
        for (int j = (issued > C::kStages ? issued - C::kStages : 0); j < issued; ++j)
          mbar_wait(&s.full[j % C::kStages], (j / C::kStages) & 1, nullptr, 0);
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_f16(1, DG_ROWS, MPAD, 0, 0);
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int st = kb % C::kStages;
        if (!mbar_wait(&s.full[st], (kb / C::kStages) & 1, p.err, 1800 + st)) { ok = false; break; }
        tc_fence_after();
        const uint32_t w_addr = smem_u32(s.w[st]), x_addr = smem_u32(s.x[st]);
#pragma unroll
        for (int k = 0; k < SUB * (DG_BK / 16); ++k) {
          const uint32_t wo = (k >> 2) * kTile + (k & 3) * 32, xo = (k >> 2) * kXTile + (k & 3) * 32;
          const uint64_t dx = make_smem_desc_sw128(x_addr + xo, 16, 1024);
          umma_f16_ss(tmem_base, make_smem_desc_sw128(w_addr + wo, 16, 1024), dx, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          if (GATED)
            umma_f16_ss(tmem_base + MPAD, make_smem_desc_sw128(smem_u32(s.w2[st]) + wo, 16, 1024), dx, idesc,
                        (kb > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&s.empty[st]);
      }
      if (ok) umma_commit(&s.acc_full);
    }
  }

  // ------------------------------------------------------------------ epilogue: warps 2 .. 5, one per TMEM lane quarter
  const bool epi = warp >= 2;
  const int quarter = warp & 3;
  const int lrow = quarter * 32 + lane;            // row of the tile = TMEM lane
  const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
  bool acc_ok = false;
  if (epi) {
    pdl_wait();                                    // y may still be read by the kernel in front of this one
    acc_ok = nkb > 0 ? mbar_wait(&s.acc_full, 0, p.err, 1900) : true;
    tc_fence_after();
  }
  // Partial sums of the other CTAs of the cluster land in the first CTA's operand ring, [peer][column][row] fp32.  Every
  // thread of the cluster takes part in both barriers, on every path.
  float* red = reinterpret_cast<float*>(&s.w[0][0]);
  if (ks > 1) {
    cluster_arrive();                              // #1: no tensor core of the cluster reads its ring any more
    cluster_wait();
    if (epi && cr != 0) {
      const uint32_t dst0 = mapa_shared(smem_u32(red), 0) + static_cast<uint32_t>(((cr - 1) * COLS) * DG_ROWS + lrow) * 4u;
#pragma unroll 1
      for (int c = 0; c < COLS; c += 32) {
        uint32_t r[32];
        if (nkb > 0 && acc_ok) {
          tmem_ld_32x32(t_row + c, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j)
          asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(dst0 + static_cast<uint32_t>((c + j) * DG_ROWS) * 4u), "r"(r[j]) : "memory");
      }
    }
    cluster_arrive();                              // #2: the partial sums are in place
    cluster_wait();
  }
  if (epi && cr == 0 && acc_ok) {
    const int row = row0 + lrow;
#pragma unroll 1
    for (int c = 0; c < MPAD; c += 32) {
      uint32_t rg[32], ru[32];
      tmem_ld_32x32(t_row + c, rg);
      if (GATED) tmem_ld_32x32(t_row + MPAD + c, ru);
      tmem_wait_ld();
      for (int pr = 0; pr < ks - 1; ++pr) {
        const float* part = red + static_cast<long long>(pr * COLS) * DG_ROWS + lrow;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          rg[j] = __float_as_uint(__uint_as_float(rg[j]) + part[(c + j) * DG_ROWS]);
          if (GATED) ru[j] = __float_as_uint(__uint_as_float(ru[j]) + part[(MPAD + c + j) * DG_ROWS]);
        }
      }
      if (row < p.N) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int tok = c + j;
          float v = __uint_as_float(rg[j]);
          if (GATED) v = (v / (1.f + __expf(-v))) * __uint_as_float(ru[j]);
          if (tok < p.M) p.y[static_cast<long long>(tok) * p.ldy + row] = __float2bfloat16(v);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ---- host ------------------------------------------------------------------------------------------------------------
typedef CUresult (*DgEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static DgEncodeFn dg_encode_fn() {
  static DgEncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<DgEncodeFn>(ptr);
  });
  return fn;
}

// bf16 [rows, K] with row stride ld (elements); box = 64 elements (128 bytes, 128-byte swizzle) x box_rows.
static int dg_make_tmap(CUtensorMap* tm, const void* base, uint64_t K, uint64_t rows, uint64_t ld, uint32_t box_rows) {
  DgEncodeFn fn = dg_encode_fn();
  if (fn == nullptr) return 1;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {DG_BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2;
}

// How many CTAs share one row tile's contraction: enough to occupy the SMs in one wave, at least eight k steps each, and
// the partial sums of the others must fit the first CTA's operand ring.
template <int MPAD, bool GATED, int SUB>
static int dg_pick_split(int tiles, int nkb) {
  using C = DgCfg<MPAD, GATED, SUB>;
  constexpr int COLS = (GATED ? 2 : 1) * MPAD;
  constexpr int ring = C::kStages * C::kWBytes * (GATED ? 2 : 1);
  int ks = 148 / (tiles > 0 ? tiles : 1);
  if (ks > 4) ks = 4;
  while (ks > 1 && (nkb * SUB / ks < 8 || (ks - 1) * COLS * DG_ROWS * 4 > ring)) --ks;
  return ks < 1 ? 1 : ks;
}

template <int MPAD, bool GATED, int SUB>
static int dg_launch(const CUtensorMap& tW, const CUtensorMap& tW2, const CUtensorMap& tX, const DgParams& p, int split, cudaStream_t st) {
  constexpr size_t smem = sizeof(DgSmem<MPAD, GATED, SUB>) + 1024;
  static_assert(smem <= 227 * 1024, "decode GEMM shared memory");
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(decode_gemm_kernel<MPAD, GATED, SUB>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return 1000 + static_cast<int>(e);
    configured[dev] = true;
  }
  const int tiles = (p.N + DG_ROWS - 1) / DG_ROWS;
  const int nst = p.K / (DG_BK * SUB);
  const int ks = split > 0 ? split : dg_pick_split<MPAD, GATED, SUB>(tiles, nst);
  {
    using C = DgCfg<MPAD, GATED, SUB>;
    constexpr int COLS = (GATED ? 2 : 1) * MPAD;
    constexpr int ring = C::kStages * C::kWBytes * (GATED ? 2 : 1);
    if (ks > 1 && (ks > 8 || nst < ks || (ks - 1) * COLS * DG_ROWS * 4 > ring)) return -6;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(tiles * ks));
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  at[1].id = cudaLaunchAttributeClusterDimension;
  at[1].val.clusterDim.x = static_cast<unsigned>(ks); at[1].val.clusterDim.y = 1; at[1].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 2;
  cudaError_t e = cudaLaunchKernelEx(&cfg, decode_gemm_kernel<MPAD, GATED, SUB>, tW, tW2, tX, p);
  return e == cudaSuccess ? 0 : 2000 + static_cast<int>(e);
}

}  // namespace tyr

// x [M <= 64, K] bf16 (row stride ldx), w [N, K] bf16 (row stride ldw), optional w2 of the same shape and stride (gated form),
// y [M, N] bf16 (row stride ldy).  K a multiple of 64, strides multiples of 8 elements, bases 16-byte aligned.
// Returns 0, a negative number for an argument the kernel does not take, or a positive CUDA / driver error.
// `split`: CTAs per cluster that share a row tile's contraction (0 = chosen from the shape).
extern "C" TYR_EXPORT int tyr_decode_gemm_bf16(const void* x, const void* w, const void* w2, void* y, long long ldx, long long ldw,
                                               long long ldy, int M, int N, int K, int split, int* err, void* stream) {
  using namespace tyr;
  if (M < 1 || M > 64 || N < 1 || K < DG_BK || (K % DG_BK)) return -1;
  if ((ldx | ldw) & 7) return -2;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(w2)) & 15) return -3;
  const int mpad = M <= 32 ? 32 : 64;
  CUtensorMap tW, tW2, tX;
  int r = dg_make_tmap(&tW, w, K, N, ldw, DG_ROWS);
  if (r == 0) r = dg_make_tmap(&tW2, w2 != nullptr ? w2 : w, K, N, ldw, DG_ROWS);
  if (r == 0) r = dg_make_tmap(&tX, x, K, M, ldx, mpad);
  if (r) return 3000 + r;
  DgParams p{reinterpret_cast<__nv_bfloat16*>(y), ldy, M, N, K, err};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (split < 0) return -6;
  // one 64-element block per stage by default: two (TYR_DECODE_GEMM_SUB=2) measured the same within 3 % either way
  static const int sub_env = [] {
    const char* v = getenv("TYR_DECODE_GEMM_SUB");
    return v != nullptr && v[0] == '2' ? 2 : 1;
  }();
  const bool two = sub_env == 2 && (K % (2 * DG_BK)) == 0;
  if (two) {
    if (w2 != nullptr) return mpad == 32 ? dg_launch<32, true, 2>(tW, tW2, tX, p, split, st) : dg_launch<64, true, 2>(tW, tW2, tX, p, split, st);
    return mpad == 32 ? dg_launch<32, false, 2>(tW, tW2, tX, p, split, st) : dg_launch<64, false, 2>(tW, tW2, tX, p, split, st);
  }
  if (w2 != nullptr) return mpad == 32 ? dg_launch<32, true, 1>(tW, tW2, tX, p, split, st) : dg_launch<64, true, 1>(tW, tW2, tX, p, split, st);
  return mpad == 32 ? dg_launch<32, false, 1>(tW, tW2, tX, p, split, st) : dg_launch<64, false, 1>(tW, tW2, tX, p, split, st);
}
