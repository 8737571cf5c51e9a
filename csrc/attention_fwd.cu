// Flash-attention forward for sm_100a on tcgen05 / TMEM / TMA.
//
// One CTA owns TWO 128-row query tiles of one (batch, head) and walks the key/value sequence
// in 128-row blocks:
//
//   warp 17      TMA producer: Q tiles once, then K_j / V_j into a 2-stage shared-memory ring
//   warp 16      MMA issuer:   S_t = Q_t K_j^T  (SS, fp32 in TMEM)  and  O_t += P_t V_j  (TS: the
//                              bf16 probabilities are read straight from TMEM, they never touch
//                              shared memory)
//   warps 0-7    softmax for query tile 0, warps 8-15 for query tile 1.  TWO threads share a score row
//                (TMEM lane): warps 0-3 / 8-11 take key columns 0..63 of the block, warps 4-7 / 12-15
//                columns 64..127.  The halves exchange their row maxima (and, once, their row sums)
//                through a pair of shared-memory slots with a bounded pairwise handshake.  Four softmax
//                warps per scheduler partition instead of two: with one thread per row each warp ran a
//                dependent chain of about 900 instructions per key block and the partition issued on a
//                third of its cycles.
//
// The two tiles ping-pong: while the softmax warps of one tile run exp2 on the SFUs, the tensor
// core works on the other tile.  TMEM map (512 columns): S0 | S1 | O0 | O1, 128 columns each;
// P_t overwrites S_t as packed bf16: each half of a row writes its 32 packed columns over the start of its own 64
// score columns (columns 0..31 and 64..95 of the tile), which only it reads.
// Online softmax uses a lazily updated running maximum: O is only rescaled (read-modify-write
// of its TMEM tile) when some row's maximum grew by more than 2^8, which keeps the result exact
// because the same stale maximum is used for the row sum.
//
// Masks: causal with an offset (query i sees keys <= i + q_offset), sliding window (keys
// > i + q_offset - window), key length (keys >= Tk are masked).  GQA by head grouping.
// Outputs: O [B, Tq, Hq, D] bf16 (strided) and the log-sum-exp [B, Hq, Tq] fp32 for backward.
//
// The reference calls at::scaled_dot_product_attention, or a query-chunked masked-math fallback
// for windows (cc/include/tyr_attention.h:58-130).
#include "common.cuh"

namespace tyr {

constexpr int ATT_BM = 128;   // query rows per tile
constexpr int ATT_BN = 128;   // key rows per block
constexpr int ATT_D = 128;    // head dim handled by this kernel
constexpr int ATT_STAGES = 2;

struct AttnParams {
  int B, Hq, Hkv, Tq, Tk;
  int q_offset;       // query row i attends keys <= i + q_offset (causal)
  int causal;
  int window;         // 0 = none
  float scale_log2;   // softmax scale * log2(e)
  __nv_bfloat16* O;
  long long o_row_stride, o_batch_stride, o_head_stride;
  float* lse;         // [B, Hq, Tq]
  int* err;
};

struct __align__(1024) AttnSmem {
  uint8_t q[2][ATT_BM * ATT_D * 2];                 // 2 tiles x (2 chunks of [128 x 64])
  uint8_t k[ATT_STAGES][ATT_BN * ATT_D * 2];
  uint8_t v[ATT_STAGES][ATT_BN * ATT_D * 2];
  uint64_t q_full;
  uint64_t k_full[ATT_STAGES];
  uint64_t v_full[ATT_STAGES];
  uint64_t k_empty[ATT_STAGES];   // K_j is free once both S products of block j retired (long before V_j is)
  uint64_t v_empty[ATT_STAGES];
  uint64_t s_ready[2];     // MMA -> softmax: S_t written
  uint64_t p_ready[2];     // softmax -> MMA: P_t written (one arrival per softmax warp)
  uint64_t o_done[2];      // MMA -> softmax: all PV of tile t retired
  uint2 xch[2][2][2][ATT_BM];   // [tile][parity][column half][row]: {value bits, sequence} of the row-maximum exchange
  uint2 xsum[2][2][ATT_BM];     // [tile][column half][row]: the row-sum exchange of the epilogue
  uint32_t tmem_base;
};

// Pairwise exchange between the two threads of a row: publish {value, seq} in my slot, poll the partner's slot until it
// carries the same sequence number.  Bounded: gives up after about a second and records an error.
__device__ __forceinline__ bool pair_exchange(uint2* mine, const uint2* theirs, float v, uint32_t seq, float& other,
                                              int* err, int tag) {
  asm volatile("st.volatile.shared.v2.u32 [%0], {%1, %2};" ::"r"(smem_u32(mine)), "r"(__float_as_uint(v)), "r"(seq) : "memory");
  const uint32_t addr = smem_u32(theirs);
  uint32_t a, b;
  long long start = 0;
  for (uint32_t spins = 0;; ++spins) {
    asm volatile("ld.volatile.shared.v2.u32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "r"(addr) : "memory");
    if (b == seq) break;
    if ((spins & 0xfff) == 0xfff) {
      const long long now = clock64();
      if (start == 0) start = now;
      if (now - start > kWaitBudgetCycles) {
        report_error(err, ERR_MBAR_TIMEOUT, tag);
        return false;
      }
    }
  }
  other = __uint_as_float(a);
  return true;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

__device__ __forceinline__ void tmem_ld_32x32_nowait(uint32_t taddr, uint32_t* r) {
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
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// Block range [lo, hi) of key blocks that query rows [r0, r0 + 128) touch.
__device__ __forceinline__ void kv_range(const AttnParams& p, int r0, int& lo, int& hi) {
  int last_key = p.Tk - 1;
  if (p.causal) last_key = min(last_key, r0 + ATT_BM - 1 + p.q_offset);
  int first_key = 0;
  if (p.window > 0) first_key = max(0, r0 + p.q_offset - p.window + 1);
  lo = first_key / ATT_BN;
  hi = last_key < 0 ? lo : last_key / ATT_BN + 1;
  if (hi < lo) hi = lo;
}

__global__ void __launch_bounds__(640, 1)
flash_fwd_d128_kernel(const __grid_constant__ CUtensorMap tmQ,
                      const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, AttnParams p) {
  pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  AttnSmem& s = *reinterpret_cast<AttnSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // heavy (late) query tiles first: causal work grows with the row index
  const int pair = gridDim.x - 1 - blockIdx.x;
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int row0 = pair * 2 * ATT_BM;

  int lo[2], hi[2];
  kv_range(p, row0, lo[0], hi[0]);
  kv_range(p, row0 + ATT_BM, lo[1], hi[1]);
  const bool tile1_live = (row0 + ATT_BM) < p.Tq;
  if (!tile1_live) { lo[1] = 0; hi[1] = 0; }
  int jlo = lo[0], jhi = hi[0];
  if (tile1_live) { jlo = min(lo[0], lo[1]); jhi = max(hi[0], hi[1]); }

  if (threadIdx.x == 0) {
    mbar_init(&s.q_full, 1);
    for (int i = 0; i < ATT_STAGES; ++i) {
      mbar_init(&s.k_full[i], 1);
      mbar_init(&s.v_full[i], 1);
      mbar_init(&s.k_empty[i], 1);
      mbar_init(&s.v_empty[i], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s.s_ready[t], 1);
      mbar_init(&s.p_ready[t], 8);             // one arrival per softmax warp of the tile
      mbar_init(&s.o_done[t], 1);
    }
    mbar_fence_init();
  }
  for (int i = threadIdx.x; i < 2 * 2 * 2 * ATT_BM; i += blockDim.x) (&s.xch[0][0][0][0])[i] = make_uint2(0u, 0u);
  for (int i = threadIdx.x; i < 2 * 2 * ATT_BM; i += blockDim.x) (&s.xsum[0][0][0])[i] = make_uint2(0u, 0u);
  if (warp == 16) {
    tmem_alloc(&s.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s.tmem_base;
  pdl_wait();                                   // everything above touched no global memory
  constexpr uint32_t kChunk = ATT_BM * 64 * 2;   // one [128 x 64] bf16 swizzled chunk = 16 KB

  // Register re-allocation between warpgroups: the four softmax warpgroups keep 64 scores per thread in registers, the
  // producer / MMA warpgroup (warps 16-19, two of them idle) needs few.  The launch allocates 96 registers per thread
  // (640 threads); 40 x 128 + 104 x 512 stays below that total, so setmaxnreg.inc never waits for registers nobody
  // releases.
  if (warp >= 16) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
  if (warp == 17) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      const int ntile = tile1_live ? 2 : 1;
      mbar_expect_tx(&s.q_full, ntile * 2 * kChunk);
      for (int t = 0; t < ntile; ++t)
        for (int c = 0; c < 2; ++c)
          tma_load_4d(s.q[t] + c * kChunk, &tmQ, &s.q_full, c * 64, head, row0 + t * ATT_BM, batch);
      uint32_t it = 0;
      bool ok = true;
      for (int j = jlo; j < jhi && ok; ++j, ++it) {
        const int st = it % ATT_STAGES;
        const uint32_t ph = (it / ATT_STAGES) & 1;
        // K and V have separate rings: a K stage is released a whole iteration before the V stage of the same block, so
        // its next load has that much longer to arrive
        if (!mbar_wait(&s.k_empty[st], ph ^ 1, p.err, 500 + st)) { ok = false; break; }
        mbar_expect_tx(&s.k_full[st], 2 * kChunk);
        for (int c = 0; c < 2; ++c)
          tma_load_4d(s.k[st] + c * kChunk, &tmK, &s.k_full[st], c * 64, kv_head, j * ATT_BN, batch);
        if (!mbar_wait(&s.v_empty[st], ph ^ 1, p.err, 510 + st)) { ok = false; ++it; break; }
        mbar_expect_tx(&s.v_full[st], 2 * kChunk);
        for (int c = 0; c < 2; ++c)
          tma_load_4d(s.v[st] + c * kChunk, &tmV, &s.v_full[st], c * 64, kv_head, j * ATT_BN, batch);
      }
      if (!ok) {   // let the K copies in flight land before the CTA unwinds (a V copy is only issued after its wait succeeded)
        for (uint32_t q = (it > ATT_STAGES ? it - ATT_STAGES : 0); q < it; ++q)
          mbar_wait(&s.k_full[q % ATT_STAGES], (q / ATT_STAGES) & 1, nullptr, 0);
      }
    }
  } else if (warp == 16) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_f16(1, ATT_BM, ATT_BN, 0, 0);   // Q K^T
      constexpr uint32_t idesc_o = make_idesc_f16(1, ATT_BM, ATT_D, 0, 1);    // P V (V is MN-major)
      bool ok = mbar_wait(&s.q_full, 0, p.err, 600);
      tc_fence_after();
      auto issue_s = [&](int t, int st) {
        const uint32_t qa = smem_u32(s.q[t]);
        const uint32_t ka = smem_u32(s.k[st]);
#pragma unroll
        for (int k = 0; k < ATT_D / 16; ++k) {
          const uint32_t off = (k >> 2) * kChunk + (k & 3) * 32;
          umma_f16_ss(tmem_base + t * 128, make_smem_desc_sw128(qa + off, 16, 1024),
                      make_smem_desc_sw128(ka + off, 16, 1024), idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(&s.s_ready[t]);
      };
      auto issue_pv = [&](int t, int st, bool first) {
        const uint32_t va = smem_u32(s.v[st]);
#pragma unroll
        for (int k = 0; k < ATT_BN / 16; ++k) {
          // A: 16 bf16 of P per lane = 8 TMEM columns; B: 16 key rows of V = 2 KB, d-chunks 16 KB apart
          umma_f16_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + (k >> 2) * 64 + (k & 3) * 8,
                      make_smem_desc_sw128(va + k * 2048, kChunk, 1024), idesc_o,
                      (first && k == 0) ? 0u : 1u);
        }
      };
      uint32_t p_cnt[2] = {0, 0};
      uint32_t it = 0;
      // prologue: S for the first block of each live tile
      if (ok && jhi > jlo) {
        ok = mbar_wait(&s.k_full[0], 0, p.err, 610);
        tc_fence_after();
        for (int t = 0; t < 2 && ok; ++t)
          if (jlo >= lo[t] && jlo < hi[t]) issue_s(t, 0);
        umma_commit(&s.k_empty[0]);                              // K of the first block: its S products are queued
      }
      for (int j = jlo; j < jhi && ok; ++j, ++it) {
        const int st = it % ATT_STAGES;
        const uint32_t ph = (it / ATT_STAGES) & 1;
        const int st_n = (it + 1) % ATT_STAGES;
        const uint32_t ph_n = ((it + 1) / ATT_STAGES) & 1;
        bool next_k_ready = false;
        for (int t = 0; t < 2 && ok; ++t) {
          const bool cur = (j >= lo[t] && j < hi[t]);
          if (cur) {
            if (!mbar_wait(&s.v_full[st], ph, p.err, 620 + st)) { ok = false; break; }
            if (!mbar_wait(&s.p_ready[t], p_cnt[t] & 1, p.err, 630 + t)) { ok = false; break; }
            ++p_cnt[t];
            tc_fence_after();
            issue_pv(t, st, j == lo[t]);
            if (j + 1 == hi[t]) umma_commit(&s.o_done[t]);
          }
          // next block's S for this tile (its S/P columns are free once PV above is queued)
          const bool nxt = (j + 1 >= lo[t] && j + 1 < hi[t]);
          if (nxt) {
            if (!next_k_ready) {
              if (!mbar_wait(&s.k_full[st_n], ph_n, p.err, 640 + st_n)) { ok = false; break; }
              tc_fence_after();
              next_k_ready = true;
            }
            issue_s(t, st_n);
          }
        }
        if (ok) {
          umma_commit(&s.v_empty[st]);                           // V_j: both PV products are queued
          if (j + 1 < jhi) umma_commit(&s.k_empty[st_n]);        // K_{j+1}: both S products are queued
        }
      }
    }
  }
  } else {
    // ------------------------------------------------------------------ softmax warps (two threads per row)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
    const int t = warp >> 3;                // query tile of this warp
    const int h = (warp >> 2) & 1;          // column half of the key block
    const int lrow = (warp & 3) * 32 + lane;
    const int row = row0 + t * ATT_BM + lrow;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_addr = tmem_base + t * 128 + h * 64 + lane_addr;     // my 64 score columns
    const uint32_t p_addr = tmem_base + t * 128 + h * 64 + lane_addr;     // my 32 packed-probability columns: the start of my own score columns
    const uint32_t o_addr = tmem_base + 256 + t * 128 + h * 64 + lane_addr;
    const bool tile_live = (t == 0) || tile1_live;
    float m_used = -INFINITY;   // running maximum the exponentials are taken against
    float l_sum = 0.f;          // this half's part of the row sum
    bool ok = true;
    uint32_t cnt = 0;
    if (tile_live) {
      for (int j = lo[t]; j < hi[t] && ok; ++j, ++cnt) {
        if (!mbar_wait(&s.s_ready[t], cnt & 1, p.err, 700 + t)) { ok = false; break; }
        tc_fence_after();
        const int col0 = j * ATT_BN + h * 64;
        // mask needed on boundary blocks only
        const int qi = row + p.q_offset;
        const bool need_mask = (j * ATT_BN + ATT_BN > p.Tk) || (p.causal && j * ATT_BN + ATT_BN - 1 > row0 + t * ATT_BM + p.q_offset) ||
                               (p.window > 0 && j * ATT_BN < row0 + t * ATT_BM + ATT_BM - 1 + p.q_offset - p.window + 1);
        auto masked = [&](uint32_t (&v)[32], int base) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int col = base + c;
            bool keep = col < p.Tk;
            if (p.causal) keep = keep && (col <= qi);
            if (p.window > 0) keep = keep && (col > qi - p.window);
            if (!keep) v[c] = __float_as_uint(-INFINITY);
          }
        };
        // Pass 1: row maximum of my 64 columns on the raw scores (the softmax scale is positive, so it commutes with
        // max).  The scores are NOT kept: pass 2 reads them from TMEM again, 32 at a time, which costs one more TMEM load
        // (about 100 cycles) and keeps the live registers far below the 96 the 640-thread launch allows (holding all 64
        // scores spilled, and the maximum alone took 500 cycles per block).
        float mx;
        {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32_nowait(s_addr, r0);
          tmem_ld_32x32_nowait(s_addr + 32, r1);
          tmem_wait_ld();
          if (need_mask) {
            masked(r0, col0);
            masked(r1, col0 + 32);
          }
          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              mx4[u] = max3(mx4[u], __uint_as_float(r0[c + 2 * u]), __uint_as_float(r0[c + 2 * u + 1]));
              mx4[u] = max3(mx4[u], __uint_as_float(r1[c + 2 * u]), __uint_as_float(r1[c + 2 * u + 1]));
            }
          }
          mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        }
        float other;
        if (!pair_exchange(&s.xch[t][cnt & 1][h][lrow], &s.xch[t][cnt & 1][h ^ 1][lrow], mx, cnt + 1, other, p.err, 720 + t)) {
          ok = false;
          break;
        }
        mx = fmaxf(mx, other) * p.scale_log2;
        // lazy rescale: move the reference maximum only when it grew by more than 8 (log2 units); both halves of a row
        // take the same decision because they see the same maximum
        const bool first = (j == lo[t]);
        float m_new = fmaxf(m_used, mx);
        const bool want = first || (m_new > m_used + 8.f);
        if (__any_sync(0xffffffffu, want && !first)) {
          // O is idle here: S_j was queued behind PV_{j-1}, so its completion implies PV_{j-1}'s.
          const float f = want ? exp2f(m_used - m_new) : 1.f;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[16];
            tmem_ld_32x16(o_addr + c * 16, o);
            tmem_wait_ld();
#pragma unroll
            for (int q = 0; q < 16; ++q) o[q] = __float_as_uint(__uint_as_float(o[q]) * f);
            tmem_st_32x16(o_addr + c * 16, o);
          }
          tmem_wait_st();
          if (want) l_sum *= f;
        }
        if (want) m_used = (m_new == -INFINITY) ? 0.f : m_new;
        // Pass 2: probabilities exp2(s * scale - m) -> bf16 -> TMEM, 32 scores at a time.  My packed probabilities go to
        // the first 32 columns of MY OWN 64 score columns (chunk c lands on columns 16 c .. 16 c + 15, which chunk c
        // itself or an earlier chunk was read from), so neither half ever writes where the other half still reads.
        float ls4[4] = {0.f, 0.f, 0.f, 0.f};
        const float neg_m = -m_used;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(s_addr + c * 32, r);
          tmem_wait_ld();
          if (need_mask) masked(r, col0 + c * 32);
          uint32_t pk[16];
#pragma unroll
          for (int q = 0; q < 16; ++q) {
            const float p0 = exp2f(fmaf(__uint_as_float(r[2 * q]), p.scale_log2, neg_m));
            const float p1 = exp2f(fmaf(__uint_as_float(r[2 * q + 1]), p.scale_log2, neg_m));
            pk[q] = pack_bf16x2(p0, p1);
            ls4[q & 3] += p0 + p1;
          }
          tmem_st_32x16(p_addr + c * 16, pk);
        }
        l_sum += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.p_ready[t]);   // one arrival per warp
      }
      // ---------------------------------------------------------------- epilogue
      if (ok && hi[t] > lo[t]) ok = mbar_wait(&s.o_done[t], 0, p.err, 710 + t);
      tc_fence_after();
      if (ok && hi[t] > lo[t]) {
        float other;
        ok = pair_exchange(&s.xsum[t][h][lrow], &s.xsum[t][h ^ 1][lrow], l_sum, 1u, other, p.err, 730 + t);
        l_sum += other;
      }
      if (ok && hi[t] > lo[t]) {
        const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
        const bool row_ok = row < p.Tq;
        __nv_bfloat16* out = p.O + batch * p.o_batch_stride + static_cast<long long>(row) * p.o_row_stride +
                             head * p.o_head_stride + h * 64;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t o[32];
          tmem_ld_32x32_nowait(o_addr + c * 32, o);   // warp-collective: every lane takes part
          tmem_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 u;
              u.x = pack_bf16x2(__uint_as_float(o[q * 8 + 0]) * inv, __uint_as_float(o[q * 8 + 1]) * inv);
              u.y = pack_bf16x2(__uint_as_float(o[q * 8 + 2]) * inv, __uint_as_float(o[q * 8 + 3]) * inv);
              u.z = pack_bf16x2(__uint_as_float(o[q * 8 + 4]) * inv, __uint_as_float(o[q * 8 + 5]) * inv);
              u.w = pack_bf16x2(__uint_as_float(o[q * 8 + 6]) * inv, __uint_as_float(o[q * 8 + 7]) * inv);
              *reinterpret_cast<uint4*>(out + c * 32 + q * 8) = u;
            }
          }
        }
        if (p.lse && row_ok && h == 0)
          p.lse[(static_cast<long long>(batch) * p.Hq + head) * p.Tq + row] =
              l_sum > 0.f ? (m_used + log2f(l_sum)) * 0.6931471805599453f : -INFINITY;
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
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
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
// [B, T, H, D] bf16 with element strides; box = 64 channels x 1 head x `rows` positions.
int make_tmap_bthd(CUtensorMap* tm, const void* base, int B, int T, int H, int D, long long sb,
                   long long st, long long sh, int rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)T, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)sh * 2, (cuuint64_t)st * 2, (cuuint64_t)sb * 2};
  if (H == 1) strides[0] = (cuuint64_t)D * 2;
  if (B == 1) strides[2] = (cuuint64_t)st * 2 * T;
  cuuint32_t box[4] = {64, 1, (cuuint32_t)rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
}  // namespace

// q/k/v/o are [B, T, H, D] views given by (batch, row, head) element strides; D must be 128.
extern "C" TYR_EXPORT int tyr_flash_fwd(const void* q, const void* k, const void* v, void* o,
                                        float* lse, int B, int Hq, int Hkv, int Tq, int Tk, int D,
                                        long long q_sb, long long q_st, long long q_sh,
                                        long long k_sb, long long k_st, long long k_sh,
                                        long long v_sb, long long v_st, long long v_sh,
                                        long long o_sb, long long o_st, long long o_sh, int causal,
                                        int window, int q_offset, float scale, int* err,
                                        void* stream) {
  if (D != ATT_D) return -1;
  if (Hq % Hkv != 0 || B <= 0 || Tq <= 0 || Tk <= 0) return -2;
  if ((q_st | q_sh | q_sb | k_st | k_sh | k_sb | v_st | v_sh | v_sb | o_st | o_sh | o_sb) & 7) return -3;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o) & 15) return -4;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = make_tmap_bthd(&tq, q, B, Tq, Hq, D, q_sb, q_st, q_sh, ATT_BM))) return 3000 + r;
  if ((r = make_tmap_bthd(&tk, k, B, Tk, Hkv, D, k_sb, k_st, k_sh, ATT_BN))) return 4000 + r;
  if ((r = make_tmap_bthd(&tv, v, B, Tk, Hkv, D, v_sb, v_st, v_sh, ATT_BN))) return 5000 + r;
  constexpr size_t smem = sizeof(AttnSmem) + 1024;
  static bool configured_dev[64] = {false};     // the attribute is per device
  int cfg_dev = 0;
  if (cudaGetDevice(&cfg_dev) != cudaSuccess || cfg_dev < 0 || cfg_dev >= 64) cfg_dev = 0;
  bool& configured = configured_dev[cfg_dev];
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(flash_fwd_d128_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return 1000 + (int)e;
    configured = true;
  }
  AttnParams p;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Tq = Tq; p.Tk = Tk;
  p.q_offset = q_offset; p.causal = causal; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.O = (__nv_bfloat16*)o; p.o_row_stride = o_st; p.o_batch_stride = o_sb; p.o_head_stride = o_sh;
  p.lse = lse; p.err = err;
  dim3 grid((Tq + 2 * ATT_BM - 1) / (2 * ATT_BM), Hq, B);
  launch_dependent(flash_fwd_d128_kernel, dim3(grid), dim3(640), smem, (cudaStream_t)stream, tq, tk, tv, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 2000 + (int)e;
}
