// Flash-attention backward for sm_100a on tcgen05 / TMEM / TMA (head dim 128, bf16).
//
// One CTA owns one 128-key block of one (batch, KV head): K_j and V_j stay in shared memory, dK_j
// and dV_j accumulate in TMEM over every query block (and every query head of the GQA group) that
// sees the block, and are written once at the end.  Scores are produced TRANSPOSED (keys on the
// TMEM lanes, query rows on the columns), so P^T and dS^T are directly the A operands of the
// dV / dK products:
//
//   S^T  = K Q_i^T                 (SS)      TMEM columns   0..127
//   dP^T = V dO_i^T                (SS)      TMEM columns 256..383
//   P^T  = exp2(S^T * c - lse_i)             bf16, packed over the S^T columns it came from
//   dS^T = P^T o (dP^T - delta_i)            bf16, packed over the dP^T columns it came from
//   dV  += P^T dO_i                (TS)      TMEM columns 128..255
//   dK  += dS^T Q_i                (TS)      TMEM columns 384..511
//
// Both A operands that the score warps produce stay in TMEM, so shared memory holds only what TMA brings: K_j, V_j, a
// 3-stage ring of Q_i (with the rows' lse and delta) and a 2-stage ring of dO_i.  Q_i lives from S^T to dK (almost two
// iterations) and dO_i from dP^T to dV (one); with one stage more than each tile's lifetime the next tile's load is issued
// a whole iteration before its first product, which hides the TMA latency (with two 64 KB stages it was exposed every
// iteration: the tensor pipe idled about 1500 cycles of 3800).
//
// dQ comes from a second kernel with the loops the other way round (one CTA per 128-row query block, walking the key
// blocks): S = Q_i K_j^T and dP = dO_i V_j^T are recomputed, dS is packed over dP in TMEM and dQ_i += dS K_j accumulates in
// TMEM, so no partial dQ tile ever leaves the SM.  Seven products per (query block, key block) pair instead of five, but
// the first version, which reduced the dQ tiles of all key blocks into an fp32 accumulator with vector atomics, was bound by
// the L2 atomic rate (about 1.5 TB/s) at less than a quarter of the tensor throughput.  A small kernel before the two computes
// delta = rowsum(dO o O) and rescales the log-sum-exp to base 2 into padded rows.
//
// dK / dV kernel:
//   warps 0-15  scores: four warpgroups, each 32 of the block's 128 query-row columns (one thread per key / TMEM lane);
//               four score warps per scheduler hide each other's TMEM-load, exp2 and packing latencies
//   warp 16     MMA issuer, warp 17 TMA producer (Q_i, dO_i, lse_i, delta_i into a 2-stage ring)
//
// Masks are those of the forward kernel: causal with offset, sliding window, key length.  Query rows
// past Tq carry lse = +inf in the padded statistics, so their probabilities are exactly zero.
//
// The reference differentiates at::scaled_dot_product_attention through autograd
// (cc/include/tyr_attention.h:58-130).
#include "common.cuh"

#include <climits>

namespace tyr {

constexpr int BW_T = 128;                       // rows of a query block == keys of a key block == head dim
constexpr uint32_t BW_CHUNK = BW_T * 64 * 2;    // one [128 x 64] bf16 swizzled chunk
constexpr uint32_t BW_TILE = 2 * BW_CHUNK;      // 32 KB

struct BwdParams {
  int B, Hq, Hkv, Tq, Tk, Tpad;
  int q_offset, causal, window;
  float scale, scale_log2;
  const float* lse2;      // [B, Hq, Tpad], base-2, +inf on padded / empty rows
  const float* delta;     // [B, Hq, Tpad]
  __nv_bfloat16* dK;
  __nv_bfloat16* dV;
  __nv_bfloat16* dQ;
  long long dk_sb, dk_st, dk_sh, dv_sb, dv_st, dv_sh, dq_sb, dq_st, dq_sh;
  int* err;
};

constexpr int BW_QST = 3;    // stages of the Q ring (dK/dV kernel) and of the K ring (dQ kernel)

struct __align__(1024) BwdSmem {
  uint8_t k[BW_TILE];
  uint8_t v[BW_TILE];
  uint8_t q[BW_QST][BW_TILE];
  uint8_t dout[2][BW_TILE];
  float lse[BW_QST][BW_T];       // travels with Q_i: the stage is released after dK, long after the exponentials read it
  float delta[2][BW_T];          // a ring of its own, released by the score warps (dO_i's stage is free again before they
                                 // read delta_i, and a third stage next to Q_i's would not fit in 227 KB)
  uint64_t kv_full;
  uint64_t q_full[BW_QST];       // Q_i + lse_i
  uint64_t q_empty[BW_QST];
  uint64_t do_full[2];
  uint64_t do_empty[2];
  uint64_t delta_full[2];
  uint64_t delta_empty[2];       // one arrival per score warp
  uint64_t s_ready, dp_ready, p_ready, ds_ready, acc_done;
  uint32_t tmem_base;
};

static_assert(sizeof(BwdSmem) <= 227 * 1024, "backward tiles exceed the shared memory of one CTA");

__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// Query blocks [lo, hi) that see at least one key of block j.
__device__ __forceinline__ void q_range(const BwdParams& p, int j, int& lo, int& hi) {
  const int nq = (p.Tq + BW_T - 1) / BW_T;
  lo = 0;
  hi = nq;
  if (p.causal) lo = max(0, j * BW_T - p.q_offset) / BW_T;
  if (p.window > 0) {
    const int kmax = min(p.Tk - 1, j * BW_T + BW_T - 1);
    const int last_row = kmax - p.q_offset + p.window - 1;
    hi = last_row < 0 ? 0 : min(nq, last_row / BW_T + 1);
  }
  if (hi < lo) hi = lo;
}

__global__ void __launch_bounds__(640, 1)
flash_bwd_d128_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                      BwdParams p) {
  pdl_trigger();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  BwdSmem& s = *reinterpret_cast<BwdSmem*>(smem_raw);
  if ((smem_u32(smem_raw) & 1023u) != 0) {       // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) report_error(p.err, ERR_TMEM, 800);
    return;
  }
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int j = blockIdx.x;
  const int kvh = blockIdx.y;
  const int batch = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  int ilo, ihi;
  q_range(p, j, ilo, ihi);
  const int ni = ihi - ilo;
  const int n_it = ni * G;

  if (threadIdx.x == 0) {
    mbar_init(&s.kv_full, 1);
    for (int i = 0; i < BW_QST; ++i) {
      mbar_init(&s.q_full[i], 1);
      mbar_init(&s.q_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.do_full[i], 1);
      mbar_init(&s.do_empty[i], 1);
      mbar_init(&s.delta_full[i], 1);
      mbar_init(&s.delta_empty[i], 16);
    }
    mbar_init(&s.s_ready, 1);
    mbar_init(&s.dp_ready, 1);
    mbar_init(&s.p_ready, 16);      // one arrival per score warp (512 single-thread arrivals on one barrier serialise)
    mbar_init(&s.ds_ready, 16);
    mbar_init(&s.acc_done, 1);
    mbar_fence_init();
  }
  if (warp == 16) {
    tmem_alloc(&s.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s.tmem_base;
  pdl_wait();                                   // everything above touched no global memory
  constexpr uint32_t COL_S = 0, COL_DV = 128, COL_DP = 256, COL_DK = 384;

  if (warp >= 16) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 17) {
      // ---------------------------------------------------------------- TMA producer
      if (elect_one() && n_it > 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmDO);
        mbar_expect_tx(&s.kv_full, 2 * BW_TILE);
        for (int c = 0; c < 2; ++c) {
          tma_load_4d(s.k + c * BW_CHUNK, &tmK, &s.kv_full, c * 64, kvh, j * BW_T, batch);
          tma_load_4d(s.v + c * BW_CHUNK, &tmV, &s.kv_full, c * 64, kvh, j * BW_T, batch);
        }
        bool ok = true;
        int it = 0, qs = 0, n_do = 0, n_dl = 0;
        uint32_t qph = 0;
        for (; it < n_it; ++it) {
          const int ds_ = it & 1;
          const uint32_t dph = (it >> 1) & 1;
          const int head = kvh * G + it / ni;
          const int i = ilo + it % ni;
          if (!mbar_wait(&s.q_empty[qs], qph ^ 1, p.err, 810 + qs)) { ok = false; break; }
          const long long stat = (static_cast<long long>(batch) * p.Hq + head) * p.Tpad + i * BW_T;
          mbar_expect_tx(&s.q_full[qs], BW_TILE + BW_T * 4);
          for (int c = 0; c < 2; ++c)
            tma_load_4d(s.q[qs] + c * BW_CHUNK, &tmQ, &s.q_full[qs], c * 64, head, i * BW_T, batch);
          bulk_load_1d(s.lse[qs], p.lse2 + stat, BW_T * 4, &s.q_full[qs]);
          if (!mbar_wait(&s.do_empty[ds_], dph ^ 1, p.err, 814 + ds_)) { ++it; ok = false; break; }
          mbar_expect_tx(&s.do_full[ds_], BW_TILE);
          for (int c = 0; c < 2; ++c)
            tma_load_4d(s.dout[ds_] + c * BW_CHUNK, &tmDO, &s.do_full[ds_], c * 64, head, i * BW_T, batch);
          ++n_do;
          if (!mbar_wait(&s.delta_empty[ds_], dph ^ 1, p.err, 816 + ds_)) { ++it; ok = false; break; }
          mbar_expect_tx(&s.delta_full[ds_], BW_T * 4);
          bulk_load_1d(s.delta[ds_], p.delta + stat, BW_T * 4, &s.delta_full[ds_]);
          ++n_dl;
          if (++qs == BW_QST) { qs = 0; qph ^= 1; }
        }
        if (!ok) {   // let the copies in flight land before the CTA unwinds (a Q tile whose dO was not issued included)
          mbar_wait(&s.kv_full, 0, nullptr, 0);
          for (int q = max(0, it - BW_QST); q < it; ++q) mbar_wait(&s.q_full[q % BW_QST], (q / BW_QST) & 1, nullptr, 0);
          for (int q = max(0, n_do - 2); q < n_do; ++q) mbar_wait(&s.do_full[q & 1], (q >> 1) & 1, nullptr, 0);
          for (int q = max(0, n_dl - 2); q < n_dl; ++q) mbar_wait(&s.delta_full[q & 1], (q >> 1) & 1, nullptr, 0);
        }
      }
    } else if (warp == 16) {
      // ---------------------------------------------------------------- MMA issuer
      if (elect_one() && n_it > 0) {
        constexpr uint32_t idesc_kk = make_idesc_f16(1, BW_T, BW_T, 0, 0);   // both operands K-major
        constexpr uint32_t idesc_kn = make_idesc_f16(1, BW_T, BW_T, 0, 1);   // B MN-major
        const uint32_t ka = smem_u32(s.k), va = smem_u32(s.v);
        // D = A[128 x 128, K-major] * B[128 x 128, K-major]^T
        auto mma_kk = [&](uint32_t d_col, uint32_t a, uint32_t b) {
          const uint64_t da = make_smem_desc_sw128(a, 16, 1024), db = make_smem_desc_sw128(b, 16, 1024);
#pragma unroll
          for (int k = 0; k < BW_T / 16; ++k) {
            const uint32_t off = (k >> 2) * BW_CHUNK + (k & 3) * 32;
            umma_f16_ss(tmem_base + d_col, smem_desc_advance(da, off), smem_desc_advance(db, off), idesc_kk, k > 0 ? 1u : 0u);
          }
        };
        // D += A^T-in-TMEM [128 keys x 128 rows] * B[rows][d] (MN-major).  A: 16 bf16 per K step = 8 columns; the four score
        // warpgroups packed their quarters over the first 16 of their own 32 columns (0, 32, 64, 96).
        auto mma_ts = [&](uint32_t d_col, uint32_t a_col, uint32_t b, bool first) {
          const uint64_t db = make_smem_desc_sw128(b, BW_CHUNK, 1024);
          const uint32_t d = tmem_base + d_col, a0 = tmem_base + a_col;
          umma_f16_ts(d, a0, db, idesc_kn, first ? 0u : 1u);
#pragma unroll
          for (int k = 1; k < BW_T / 16; ++k)
            umma_f16_ts(d, a0 + (k >> 1) * 32 + (k & 1) * 8, smem_desc_advance(db, k * 2048), idesc_kn, 1u);
        };
        bool ok = mbar_wait(&s.kv_full, 0, p.err, 820);
        ok = ok && mbar_wait(&s.q_full[0], 0, p.err, 821);
        if (ok) {
          tc_fence_after();
          mma_kk(COL_S, ka, smem_u32(s.q[0]));
          umma_commit(&s.s_ready);
          ok = mbar_wait(&s.do_full[0], 0, p.err, 822);
        }
        if (ok) {
          tc_fence_after();
          mma_kk(COL_DP, va, smem_u32(s.dout[0]));
          umma_commit(&s.dp_ready);
        }
        int qs = 0;            // ring stage of Q_it
        uint32_t qph = 0;
        for (int it = 0; it < n_it && ok; ++it) {
          const int dst = it & 1;
          const uint32_t par = it & 1;
          int qn = qs + 1;     // ring stage and parity of Q_{it+1}
          uint32_t qnph = qph;
          if (qn == BW_QST) { qn = 0; qnph ^= 1; }
          // dV += P^T dO_i
          if (!mbar_wait(&s.p_ready, par, p.err, 830)) { ok = false; break; }
          tc_fence_after();
          mma_ts(COL_DV, COL_S, smem_u32(s.dout[dst]), it == 0);
          umma_commit(&s.do_empty[dst]);
          // S^T of the next block over the P^T that dV has just consumed
          if (it + 1 < n_it) {
            if (!mbar_wait(&s.q_full[qn], qnph, p.err, 831)) { ok = false; break; }
            tc_fence_after();
            mma_kk(COL_S, ka, smem_u32(s.q[qn]));
            umma_commit(&s.s_ready);
          }
          // dK += dS^T Q_i, then dP^T of the next block over the dS^T that dK has just consumed
          if (!mbar_wait(&s.ds_ready, par, p.err, 832)) { ok = false; break; }
          tc_fence_after();
          mma_ts(COL_DK, COL_DP, smem_u32(s.q[qs]), it == 0);
          umma_commit(&s.q_empty[qs]);
          if (it + 1 < n_it) {
            const int dn = (it + 1) & 1;
            if (!mbar_wait(&s.do_full[dn], ((it + 1) >> 1) & 1, p.err, 833)) { ok = false; break; }
            tc_fence_after();
            mma_kk(COL_DP, va, smem_u32(s.dout[dn]));
            umma_commit(&s.dp_ready);
          }
          qs = qn;
          qph = qnph;
        }
        if (ok) umma_commit(&s.acc_done);
      }
    }
  } else {
    // ------------------------------------------------------------------ score warps: 4 warpgroups x 32 query-row columns
    asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
    const int wg = warp >> 2;
    const int r = (warp & 3) * 32 + lane;                // key row of this thread inside the block
    const int key = j * BW_T + r;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_addr = tmem_base + COL_S + wg * 32 + lane_addr;
    const uint32_t dp_addr = tmem_base + COL_DP + wg * 32 + lane_addr;
    const int rmin = p.causal ? key - p.q_offset : INT_MIN;                 // rows that see this key: [rmin, rmax)
    const int rmax = p.window > 0 ? key - p.q_offset + p.window : INT_MAX;
    const bool key_ok = key < p.Tk;
    bool ok = true;
    int st = 0;              // ring stage of Q_it (and of its lse row)
    uint32_t ph = 0;
    for (int it = 0; it < n_it && ok; ++it) {
      const int i = ilo + it % ni;
      const int row0 = i * BW_T + wg * 32;               // first query row of this thread's columns
      if (!mbar_wait(&s.q_full[st], ph, p.err, 850)) { ok = false; break; }
      if (!mbar_wait(&s.s_ready, it & 1, p.err, 851)) { ok = false; break; }
      tc_fence_after();
      float pr[32];
      {
        uint32_t t[32];
        tmem_ld_32x32(s_addr, t);
        tmem_wait_ld();
        const int blk_lo = i * BW_T, blk_hi = i * BW_T + BW_T - 1;
        const bool full = (j * BW_T + BW_T <= p.Tk) && (!p.causal || j * BW_T + BW_T - 1 <= blk_lo + p.q_offset) &&
                          (p.window <= 0 || j * BW_T > blk_hi + p.q_offset - p.window);
        const float4* l4 = reinterpret_cast<const float4*>(&s.lse[st][wg * 32]);
        if (full) {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const float4 l = l4[c];
            pr[4 * c + 0] = exp2f(fmaf(__uint_as_float(t[4 * c + 0]), p.scale_log2, -l.x));
            pr[4 * c + 1] = exp2f(fmaf(__uint_as_float(t[4 * c + 1]), p.scale_log2, -l.y));
            pr[4 * c + 2] = exp2f(fmaf(__uint_as_float(t[4 * c + 2]), p.scale_log2, -l.z));
            pr[4 * c + 3] = exp2f(fmaf(__uint_as_float(t[4 * c + 3]), p.scale_log2, -l.w));
          }
        } else {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const float4 l = l4[c];
            const float lv[4] = {l.x, l.y, l.z, l.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int row = row0 + 4 * c + e;
              const bool keep = key_ok && row >= rmin && row < rmax;
              pr[4 * c + e] = keep ? exp2f(fmaf(__uint_as_float(t[4 * c + e]), p.scale_log2, -lv[e])) : 0.f;
            }
          }
        }
      }
      // P^T as packed bf16 over the first 16 of this warpgroup's own 32 score columns
      {
        uint32_t pk[16];
#pragma unroll
        for (int q = 0; q < 16; ++q) pk[q] = pack_bf16x2(pr[2 * q], pr[2 * q + 1]);
        tmem_st_32x16(s_addr, pk);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.p_ready);
      // dP^T_it was queued behind dK of the previous block, so its completion also says that the dS^T columns are free
      if (!mbar_wait(&s.delta_full[it & 1], (it >> 1) & 1, p.err, 852)) { ok = false; break; }
      if (!mbar_wait(&s.dp_ready, it & 1, p.err, 853)) { ok = false; break; }
      tc_fence_after();
      const float4* d4 = reinterpret_cast<const float4*>(&s.delta[it & 1][wg * 32]);
      {
        uint32_t t[32];
        tmem_ld_32x32(dp_addr, t);
        tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float4 da = d4[u * 2], db = d4[u * 2 + 1];
          const float* pp = pr + u * 8;
          pk[u * 4 + 0] = pack_bf16x2(pp[0] * (__uint_as_float(t[u * 8 + 0]) - da.x), pp[1] * (__uint_as_float(t[u * 8 + 1]) - da.y));
          pk[u * 4 + 1] = pack_bf16x2(pp[2] * (__uint_as_float(t[u * 8 + 2]) - da.z), pp[3] * (__uint_as_float(t[u * 8 + 3]) - da.w));
          pk[u * 4 + 2] = pack_bf16x2(pp[4] * (__uint_as_float(t[u * 8 + 4]) - db.x), pp[5] * (__uint_as_float(t[u * 8 + 5]) - db.y));
          pk[u * 4 + 3] = pack_bf16x2(pp[6] * (__uint_as_float(t[u * 8 + 6]) - db.z), pp[7] * (__uint_as_float(t[u * 8 + 7]) - db.w));
        }
        tmem_st_32x16(dp_addr, pk);     // dS^T over the first 16 of this warpgroup's own 32 dP^T columns
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (++st == BW_QST) { st = 0; ph ^= 1; }
      if (lane == 0) {
        mbar_arrive(&s.ds_ready);
        mbar_arrive(&s.delta_empty[it & 1]);
      }
    }
    // ---------------------------------------------------------------- dK / dV epilogue
    if (ok && n_it > 0) ok = mbar_wait(&s.acc_done, 0, p.err, 860);
    tc_fence_after();
    if (ok) {
      // warpgroups 0, 1 write the two channel halves of dV, warpgroups 2, 3 those of dK (scaled)
      const bool is_dv = wg < 2;
      const uint32_t src = tmem_base + (is_dv ? COL_DV : COL_DK) + (wg & 1) * 64 + lane_addr;
      const float f = is_dv ? 1.f : p.scale;
      __nv_bfloat16* out = (is_dv ? p.dV + batch * p.dv_sb + static_cast<long long>(key) * p.dv_st + kvh * p.dv_sh
                                  : p.dK + batch * p.dk_sb + static_cast<long long>(key) * p.dk_st + kvh * p.dk_sh) + (wg & 1) * 64;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t o[32];
        if (n_it > 0) {
          tmem_ld_32x32(src + c * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int q = 0; q < 32; ++q) o[q] = 0u;
        }
        if (key_ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(o[q * 8 + 0]) * f, __uint_as_float(o[q * 8 + 1]) * f);
            u.y = pack_bf16x2(__uint_as_float(o[q * 8 + 2]) * f, __uint_as_float(o[q * 8 + 3]) * f);
            u.z = pack_bf16x2(__uint_as_float(o[q * 8 + 4]) * f, __uint_as_float(o[q * 8 + 5]) * f);
            u.w = pack_bf16x2(__uint_as_float(o[q * 8 + 6]) * f, __uint_as_float(o[q * 8 + 7]) * f);
            *reinterpret_cast<uint4*>(out + c * 32 + q * 8) = u;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 16) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// Sixteen threads per (batch, head, padded row), 16 bytes each: delta = sum_d dO*O and lse in base 2 (+inf where the row is
// padding or saw no key).  32-bit index arithmetic (the row count is checked on the host).
__global__ void __launch_bounds__(256)
flash_bwd_prepare_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                         const float* __restrict__ lse, float* __restrict__ lse2, float* __restrict__ delta, int B, int H,
                         int Tq, int Tpad, long long do_sb, long long do_st, long long do_sh, long long o_sb, long long o_st,
                         long long o_sh) {
  pdl_entry();
  const int total = B * H * Tpad;
  const int sub = threadIdx.x & 15;
  for (int w = blockIdx.x * 16 + (threadIdx.x >> 4); w < total; w += gridDim.x * 16) {
    const int row = w % Tpad;
    const int bh = w / Tpad;
    const int h = bh % H, b = bh / H;
    float acc = 0.f, l2 = INFINITY;
    if (row < Tq) {
      const uint4 a = *reinterpret_cast<const uint4*>(dO + b * do_sb + static_cast<long long>(row) * do_st + h * do_sh + sub * 8);
      const uint4 c = *reinterpret_cast<const uint4*>(O + b * o_sb + static_cast<long long>(row) * o_st + h * o_sh + sub * 8);
      const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
      const float2 c0 = unpack_bf16x2(c.x), c1 = unpack_bf16x2(c.y), c2 = unpack_bf16x2(c.z), c3 = unpack_bf16x2(c.w);
      acc = (a0.x * c0.x + a0.y * c0.y) + (a1.x * c1.x + a1.y * c1.y) + (a2.x * c2.x + a2.y * c2.y) + (a3.x * c3.x + a3.y * c3.y);
      if (sub == 0) {
        const float l = lse[static_cast<long long>(bh) * Tq + row];
        l2 = (l == -INFINITY) ? INFINITY : l * 1.4426950408889634f;
      }
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (sub == 0) {
      delta[w] = acc;
      lse2[w] = l2;
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// dQ: one CTA per 128-row query block of one (batch, head).  Q_i and dO_i stay in shared memory, K_j streams through a
// 3-stage ring (it lives from S, computed two blocks ahead, to dQ) and V_j through a 2-stage ring (dP only); per key block:
// S = Q_i K_j^T (TMEM columns 0..127 or 384..511), dP = dO_i V_j^T (128..255), the score warps turn them into
// dS = P o (dP - delta) packed as bf16 over the dP columns (the A operand of the next product, read from TMEM), and
// dQ_i += dS K_j accumulates at columns 256..383.
//   warps 0-15  scores: four warpgroups of 32 key columns each (one thread per query row / TMEM lane)
//   warp 16     MMA issuer, warp 17 TMA producer
// ------------------------------------------------------------------------------------------------------------------
struct __align__(1024) DqSmem {
  uint8_t q[BW_TILE];
  uint8_t dout[BW_TILE];
  uint8_t k[BW_QST][BW_TILE];
  uint8_t v[2][BW_TILE];
  uint64_t qdo_full;
  uint64_t k_full[BW_QST], k_empty[BW_QST], v_full[2], v_empty[2];
  uint64_t s_ready[2], s_free[2], dp_ready, ds_ready, acc_done;
  uint32_t tmem_base;
};
static_assert(sizeof(DqSmem) <= 227 * 1024, "dQ tiles exceed the shared memory of one CTA");

// Key blocks [lo, hi) that the query rows [r0, r0 + 128) see.
__device__ __forceinline__ void k_range(const BwdParams& p, int r0, int& lo, int& hi) {
  int last_key = p.Tk - 1;
  if (p.causal) last_key = min(last_key, r0 + BW_T - 1 + p.q_offset);
  int first_key = 0;
  if (p.window > 0) first_key = max(0, r0 + p.q_offset - p.window + 1);
  lo = first_key / BW_T;
  hi = last_key < 0 ? lo : last_key / BW_T + 1;
  if (hi < lo) hi = lo;
}

__global__ void __launch_bounds__(576, 1)
flash_bwd_dq_d128_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, BwdParams p) {
  pdl_trigger();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  DqSmem& s = *reinterpret_cast<DqSmem*>(smem_raw);
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) report_error(p.err, ERR_TMEM, 900);
    return;
  }
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int i = gridDim.x - 1 - blockIdx.x;      // late query blocks see the most keys: start them first
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int kvh = head / (p.Hq / p.Hkv);
  int jlo, jhi;
  k_range(p, i * BW_T, jlo, jhi);
  const int n_it = jhi - jlo;

  if (threadIdx.x == 0) {
    mbar_init(&s.qdo_full, 1);
    for (int q = 0; q < BW_QST; ++q) {
      mbar_init(&s.k_full[q], 1);
      mbar_init(&s.k_empty[q], 1);
    }
    for (int q = 0; q < 2; ++q) {
      mbar_init(&s.v_full[q], 1);
      mbar_init(&s.v_empty[q], 1);
    }
    mbar_init(&s.s_ready[0], 1);
    mbar_init(&s.s_ready[1], 1);
    mbar_init(&s.s_free[0], 16);
    mbar_init(&s.s_free[1], 16);
    mbar_init(&s.dp_ready, 1);
    mbar_init(&s.ds_ready, 16);
    mbar_init(&s.acc_done, 1);
    mbar_fence_init();
  }
  if (warp == 16) {
    tmem_alloc(&s.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s.tmem_base;
  pdl_wait();                                   // everything above touched no global memory
  // S is double buffered (columns 0..127 and 384..511): S_{j+1} is computed while the score warps still work on block j,
  // so they go from dS_j straight to the exponentials of block j+1.
  constexpr uint32_t COL_S0 = 0, COL_DP = 128, COL_DQ = 256, COL_S1 = 384;

  if (warp == 17) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one() && n_it > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      tma_prefetch_desc(&tmDO);
      mbar_expect_tx(&s.qdo_full, 2 * BW_TILE);
      for (int c = 0; c < 2; ++c) {
        tma_load_4d(s.q + c * BW_CHUNK, &tmQ, &s.qdo_full, c * 64, head, i * BW_T, batch);
        tma_load_4d(s.dout + c * BW_CHUNK, &tmDO, &s.qdo_full, c * 64, head, i * BW_T, batch);
      }
      bool ok = true;
      int it = 0, ks = 0, n_v = 0;
      uint32_t kph = 0;
      for (; it < n_it; ++it) {
        const int vs = it & 1;
        const uint32_t vph = (it >> 1) & 1;
        if (!mbar_wait(&s.k_empty[ks], kph ^ 1, p.err, 910 + ks)) { ok = false; break; }
        mbar_expect_tx(&s.k_full[ks], BW_TILE);
        for (int c = 0; c < 2; ++c)
          tma_load_4d(s.k[ks] + c * BW_CHUNK, &tmK, &s.k_full[ks], c * 64, kvh, (jlo + it) * BW_T, batch);
        if (++ks == BW_QST) { ks = 0; kph ^= 1; }
        if (!mbar_wait(&s.v_empty[vs], vph ^ 1, p.err, 914 + vs)) { ++it; ok = false; break; }
        mbar_expect_tx(&s.v_full[vs], BW_TILE);
        for (int c = 0; c < 2; ++c)
          tma_load_4d(s.v[vs] + c * BW_CHUNK, &tmV, &s.v_full[vs], c * 64, kvh, (jlo + it) * BW_T, batch);
        ++n_v;
      }
      if (!ok) {   // let the copies in flight land before the CTA unwinds
        mbar_wait(&s.qdo_full, 0, nullptr, 0);
        for (int q = max(0, it - BW_QST); q < it; ++q) mbar_wait(&s.k_full[q % BW_QST], (q / BW_QST) & 1, nullptr, 0);
        for (int q = max(0, n_v - 2); q < n_v; ++q) mbar_wait(&s.v_full[q & 1], (q >> 1) & 1, nullptr, 0);
      }
    }
  } else if (warp == 16) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one() && n_it > 0) {
      constexpr uint32_t idesc_kk = make_idesc_f16(1, BW_T, BW_T, 0, 0);
      constexpr uint32_t idesc_kn = make_idesc_f16(1, BW_T, BW_T, 0, 1);
      const uint32_t qa = smem_u32(s.q), doa = smem_u32(s.dout);
      auto mma_kk = [&](uint32_t d_col, uint32_t a, uint32_t b) {
        const uint64_t da = make_smem_desc_sw128(a, 16, 1024), db = make_smem_desc_sw128(b, 16, 1024);
#pragma unroll
        for (int k = 0; k < BW_T / 16; ++k) {
          const uint32_t off = (k >> 2) * BW_CHUNK + (k & 3) * 32;
          umma_f16_ss(tmem_base + d_col, smem_desc_advance(da, off), smem_desc_advance(db, off), idesc_kk, k > 0 ? 1u : 0u);
        }
      };
      bool ok = mbar_wait(&s.qdo_full, 0, p.err, 920);
      ok = ok && mbar_wait(&s.k_full[0], 0, p.err, 921);
      if (ok) {
        tc_fence_after();
        mma_kk(COL_S0, qa, smem_u32(s.k[0]));
        umma_commit(&s.s_ready[0]);
        ok = mbar_wait(&s.v_full[0], 0, p.err, 922);
      }
      if (ok) {
        tc_fence_after();
        mma_kk(COL_DP, doa, smem_u32(s.v[0]));
        umma_commit(&s.dp_ready);
        umma_commit(&s.v_empty[0]);
      }
      // S of the second block right away: its TMEM buffer is free and K_1 sits in the next ring stage
      if (ok && n_it > 1) {
        ok = mbar_wait(&s.k_full[1], 0, p.err, 923);
        if (ok) {
          tc_fence_after();
          mma_kk(COL_S1, qa, smem_u32(s.k[1]));
          umma_commit(&s.s_ready[1]);
        }
      }
      int ks = 0;                        // ring stage of K_it; K_{it+2} sits in stage (ks + 2) % 3
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it & 1;
        int k2 = ks + 2;
        if (k2 >= BW_QST) k2 -= BW_QST;
        // the score warps have read S_j and dP_j and written dS_j over dP_j
        if (!mbar_wait(&s.ds_ready, it & 1, p.err, 930)) { ok = false; break; }
        tc_fence_after();
        // dQ_i += dS K_j : A = dS [rows][keys] from TMEM (16 bf16 per K step = 8 columns; the four score warpgroups packed
        // their quarters over the first 16 of their own 32 columns), B = K_j [keys][d] MN-major
        const uint32_t ka = smem_u32(s.k[ks]);
        const uint64_t dk = make_smem_desc_sw128(ka, BW_CHUNK, 1024);
        umma_f16_ts(tmem_base + COL_DQ, tmem_base + COL_DP, dk, idesc_kn, it == 0 ? 0u : 1u);
#pragma unroll
        for (int k = 1; k < BW_T / 16; ++k)
          umma_f16_ts(tmem_base + COL_DQ, tmem_base + COL_DP + (k >> 1) * 32 + (k & 1) * 8, smem_desc_advance(dk, k * 2048),
                      idesc_kn, 1u);
        umma_commit(&s.k_empty[ks]);
        // dP of the next block over the dS that dQ has just consumed
        if (it + 1 < n_it) {
          const int sn = (it + 1) & 1;
          const uint32_t phn = ((it + 1) >> 1) & 1;
          if (!mbar_wait(&s.v_full[sn], phn, p.err, 932)) { ok = false; break; }
          tc_fence_after();
          mma_kk(COL_DP, doa, smem_u32(s.v[sn]));
          umma_commit(&s.dp_ready);
          umma_commit(&s.v_empty[sn]);
        }
        // S of block it + 2 into the buffer block it used: the score warps released it after their exponentials
        if (it + 2 < n_it) {
          if (!mbar_wait(&s.s_free[st], (it >> 1) & 1, p.err, 933)) { ok = false; break; }
          if (!mbar_wait(&s.k_full[k2], static_cast<uint32_t>(((it + 2) / BW_QST) & 1), p.err, 931)) { ok = false; break; }
          tc_fence_after();
          mma_kk(st ? COL_S1 : COL_S0, qa, smem_u32(s.k[k2]));
          umma_commit(&s.s_ready[st]);
        }
        if (++ks == BW_QST) ks = 0;
      }
      if (ok) umma_commit(&s.acc_done);
    }
  } else {
    // ------------------------------------------------------------------ score warps: 4 warpgroups x 32 key columns
    const int wg = warp >> 2;
    const int r = (warp & 3) * 32 + lane;                 // query row of this thread inside the block
    const int row = i * BW_T + r;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_addr0 = tmem_base + COL_S0 + wg * 32 + lane_addr;
    const uint32_t s_addr1 = tmem_base + COL_S1 + wg * 32 + lane_addr;
    const uint32_t dp_addr = tmem_base + COL_DP + wg * 32 + lane_addr;
    const long long stat = (static_cast<long long>(batch) * p.Hq + head) * p.Tpad + row;
    const float lse2 = p.lse2[stat];                      // +inf on padded / empty rows: their probabilities are 0
    const float delta = p.delta[stat];
    const int kmin = p.window > 0 ? row + p.q_offset - p.window + 1 : INT_MIN;      // keys this row sees: [kmin, kmax]
    const int kmax = min(p.Tk - 1, p.causal ? row + p.q_offset : INT_MAX);
    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      const int j = jlo + it;
      const int key0 = j * BW_T + wg * 32;
      if (!mbar_wait(&s.s_ready[it & 1], (it >> 1) & 1, p.err, 950)) { ok = false; break; }
      tc_fence_after();
      float pr[32];
      {
        uint32_t t[32];
        tmem_ld_32x32((it & 1) ? s_addr1 : s_addr0, t);
        tmem_wait_ld();
        // the scores are in registers: the buffer may take S of block it + 2
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.s_free[it & 1]);
        const bool full = (j * BW_T + BW_T <= p.Tk) && (!p.causal || j * BW_T + BW_T - 1 <= i * BW_T + p.q_offset) &&
                          (p.window <= 0 || j * BW_T > i * BW_T + BW_T - 1 + p.q_offset - p.window);
        if (full) {
#pragma unroll
          for (int c = 0; c < 32; ++c) pr[c] = exp2f(fmaf(__uint_as_float(t[c]), p.scale_log2, -lse2));
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int key = key0 + c;
            pr[c] = (key >= kmin && key <= kmax) ? exp2f(fmaf(__uint_as_float(t[c]), p.scale_log2, -lse2)) : 0.f;
          }
        }
      }
      // dP_it was queued behind dQ of the previous block, so its completion also says that the dS columns are free
      if (!mbar_wait(&s.dp_ready, it & 1, p.err, 951)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t t[32];
        tmem_ld_32x32(dp_addr, t);
        tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int q = 0; q < 16; ++q)
          pk[q] = pack_bf16x2(pr[2 * q] * (__uint_as_float(t[2 * q]) - delta), pr[2 * q + 1] * (__uint_as_float(t[2 * q + 1]) - delta));
        tmem_st_32x16(dp_addr, pk);     // dS over the first 16 of this warpgroup's own 32 dP columns
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.ds_ready);
    }
    // ---------------------------------------------------------------- dQ epilogue: each warpgroup writes 32 channels
    if (ok && n_it > 0) ok = mbar_wait(&s.acc_done, 0, p.err, 960);
    tc_fence_after();
    if (ok) {
      const uint32_t src = tmem_base + COL_DQ + wg * 32 + lane_addr;
      __nv_bfloat16* out = p.dQ + batch * p.dq_sb + static_cast<long long>(row) * p.dq_st + head * p.dq_sh + wg * 32;
#pragma unroll
      for (int c = 0; c < 1; ++c) {
        uint32_t o[32];
        if (n_it > 0) {
          tmem_ld_32x32(src + c * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int q = 0; q < 32; ++q) o[q] = 0u;
        }
        if (row < p.Tq) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(o[q * 8 + 0]) * p.scale, __uint_as_float(o[q * 8 + 1]) * p.scale);
            u.y = pack_bf16x2(__uint_as_float(o[q * 8 + 2]) * p.scale, __uint_as_float(o[q * 8 + 3]) * p.scale);
            u.z = pack_bf16x2(__uint_as_float(o[q * 8 + 4]) * p.scale, __uint_as_float(o[q * 8 + 5]) * p.scale);
            u.w = pack_bf16x2(__uint_as_float(o[q * 8 + 6]) * p.scale, __uint_as_float(o[q * 8 + 7]) * p.scale);
            *reinterpret_cast<uint4*>(out + c * 32 + q * 8) = u;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 16) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace tyr

using namespace tyr;

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}
// [B, T, H, 128] bf16 given by element strides; box = 64 channels x 1 head x 128 positions.
int make_map(CUtensorMap* tm, const void* base, int B, int T, int H, long long sb, long long st, long long sh) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)BW_T, (cuuint64_t)H, (cuuint64_t)T, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)sh * 2, (cuuint64_t)st * 2, (cuuint64_t)sb * 2};
  if (H == 1) strides[0] = (cuuint64_t)BW_T * 2;
  if (B == 1) strides[2] = (cuuint64_t)st * 2 * T;
  cuuint32_t box[4] = {64, 1, (cuuint32_t)BW_T, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
}  // namespace

// Bytes of scratch the backward needs: the padded base-2 lse and delta rows.
extern "C" TYR_EXPORT long long tyr_flash_bwd_workspace_bytes(int B, int Hq, int Tq) {
  const long long tpad = (Tq + BW_T - 1) / BW_T * BW_T;
  return static_cast<long long>(B) * Hq * tpad * 2 * 4;
}

// Every tensor is a [B, T, H, 128] view given by (batch, row, head) element strides; lse is the
// forward's [B, Hq, Tq] fp32 natural-log statistics.  strides: q, k, v, o, do, dq, dk, dv (3 each).
extern "C" TYR_EXPORT int tyr_flash_bwd(const void* dout, const void* q, const void* k, const void* v, const void* o,
                                        const float* lse, void* dq, void* dk, void* dv, void* workspace, int B,
                                        int Hq, int Hkv, int Tq, int Tk, int D, const long long* strides, int causal,
                                        int window, int q_offset, float scale, int* err, void* stream) {
  if (D != BW_T) return -1;
  if (Hq % Hkv != 0 || B <= 0 || Tq <= 0 || Tk <= 0 || !workspace) return -2;
  for (int i = 0; i < 24; ++i)
    if (strides[i] & 7) return -3;
  if (((uintptr_t)dout | (uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o | (uintptr_t)dq | (uintptr_t)dk |
       (uintptr_t)dv | (uintptr_t)workspace) & 15)
    return -4;
  const long long* sq = strides;
  const long long* sk = strides + 3;
  const long long* sv = strides + 6;
  const long long* so = strides + 9;
  const long long* sdo = strides + 12;
  const long long* sdq = strides + 15;
  const long long* sdk = strides + 18;
  const long long* sdv = strides + 21;
  const int tpad = (Tq + BW_T - 1) / BW_T * BW_T;
  const long long rows = static_cast<long long>(B) * Hq * tpad;
  float* lse2 = static_cast<float*>(workspace);
  float* delta = lse2 + rows;
  CUtensorMap tq, tk, tv, tdo;
  int r;
  if ((r = make_map(&tq, q, B, Tq, Hq, sq[0], sq[1], sq[2]))) return 3000 + r;
  if ((r = make_map(&tk, k, B, Tk, Hkv, sk[0], sk[1], sk[2]))) return 4000 + r;
  if ((r = make_map(&tv, v, B, Tk, Hkv, sv[0], sv[1], sv[2]))) return 5000 + r;
  if ((r = make_map(&tdo, dout, B, Tq, Hq, sdo[0], sdo[1], sdo[2]))) return 6000 + r;
  constexpr size_t smem = sizeof(BwdSmem), smem_dq = sizeof(DqSmem);
  static bool configured_dev[64] = {false};     // the attribute is per device
  int cfg_dev = 0;
  if (cudaGetDevice(&cfg_dev) != cudaSuccess || cfg_dev < 0 || cfg_dev >= 64) cfg_dev = 0;
  bool& configured = configured_dev[cfg_dev];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(flash_bwd_d128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(flash_bwd_dq_d128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dq);
    if (e != cudaSuccess) return 1000 + (int)e;
    configured = true;
  }
  cudaStream_t cs = (cudaStream_t)stream;
  if (rows >= (1LL << 31) - 4096) return -5;
  {
    long long blocks = (rows + 15) / 16;
    if (blocks > 148LL * 64) blocks = 148LL * 64;
    launch_dependent(flash_bwd_prepare_kernel, dim3((unsigned)blocks), dim3(256), 0, cs,
        (const __nv_bfloat16*)dout, (const __nv_bfloat16*)o, lse, lse2, delta, B, Hq, Tq, tpad, sdo[0], sdo[1],
        sdo[2], so[0], so[1], so[2]);
  }
  BwdParams p;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Tq = Tq; p.Tk = Tk; p.Tpad = tpad;
  p.q_offset = q_offset; p.causal = causal; p.window = window;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.lse2 = lse2; p.delta = delta;
  p.dK = (__nv_bfloat16*)dk; p.dV = (__nv_bfloat16*)dv;
  p.dk_sb = sdk[0]; p.dk_st = sdk[1]; p.dk_sh = sdk[2];
  p.dv_sb = sdv[0]; p.dv_st = sdv[1]; p.dv_sh = sdv[2];
  p.dQ = (__nv_bfloat16*)dq;
  p.dq_sb = sdq[0]; p.dq_st = sdq[1]; p.dq_sh = sdq[2];
  p.err = err;
  dim3 grid((Tk + BW_T - 1) / BW_T, Hkv, B);
  launch_dependent(flash_bwd_d128_kernel, dim3(grid), dim3(640), smem, cs, tq, tk, tv, tdo, p);
  launch_dependent(flash_bwd_dq_d128_kernel, dim3((Tq + BW_T - 1) / BW_T, Hq, B), dim3(576), smem_dq, cs, tq, tk, tv, tdo, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 2000 + (int)e;
}
