// Persistent, warp-specialised bf16 GEMM for sm_100a built directly on tcgen05.mma + TMEM + TMA.
//
//   C[b] = alpha * act(A[b] * B[b]^T-or-not) + beta * Aux[b]
//
// * Operands are bf16 in global memory.  Each operand is either K-major (reduction dimension
//   contiguous) or MN-major (row/column dimension contiguous), so the forward (X*W^T), the
//   data-gradient (dY*W) and the weight-gradient (dY^T*X) products of a linear layer all run
//   without a transpose pass.
// * One CTA per SM, 256 threads: warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
//   warps 6-7 = gather warps (only busy in tp_mode 2, see GemmParams),
//   warps 2..5 = epilogue (one TMEM lane quarter each).  The fp32 accumulator lives in TMEM
//   and is double buffered (2 x BN columns) so the epilogue of tile i overlaps the main loop
//   of tile i+1.
// * Work is either split at tile granularity (plain stores) or, for the weight-gradient shapes
//   (few output tiles, very long K), along K with fp32 `red.global.add` accumulation into a
//   zero-initialised (or gradient-accumulating) output: whole tiles for as many full rounds as
//   there are, the remaining tiles cut into k slabs dealt round-robin.  All CTAs then sweep the
//   same k blocks at the same time, so operand slabs are shared through L2 (see GemmParams).
// * Every mbarrier wait is bounded; a timeout records an error and unwinds through the normal
//   teardown (TMEM is released).
//
// What the reference does for the same products: cuBLAS through torch::linear / mm / bmm
// (cc/src/tyr.cpp:1003-1036, 1267-1300) followed by separate elementwise kernels.
#include "common.cuh"
#include <cstdio>
#include <cstdlib>
#include <mutex>

namespace tyr {

constexpr int BM = 128;
constexpr int BK = 64;        // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;

struct GemmParams {
  int M, N, K, batch;
  void* C;
  const __nv_bfloat16* aux;
  long long ldc, ldaux, sC, sAux;
  float alpha, beta;
  int act;        // 0 none, 1 relu(x)^2, 2 relu, 3 acc * 2*sqrt(aux), 4 SwiGLU of column halves, 5 GELU(tanh)-gate of column halves
  int out_mode;   // 0 bf16 store, 1 fp32 store, 2 fp32 atomic add (stream-K)
  // out_mode 2 only.  > 0: the first (tiles / grid) * grid tiles are reduced whole, one per CTA and round, and every
  // remaining tile is cut into sk_slabs equal k ranges that are dealt round-robin, slab by slab.  All CTAs then sweep the
  // same k blocks at the same time, so a k slab of both operands is read from HBM once and served to the other CTAs from
  // L2.  0: an even split of the linear (tile, k-block) sequence (grouped mode, where the tile count lives on the device).
  int sk_slabs;
  // Tile order of the non-grouped walk: 0 = column tiles fastest (the tiles in flight share a few A row tiles and keep all
  // of B in L2: right while B is the smaller operand), 1 = row tiles fastest (A stays in L2 and B streams once: an lm_head
  // whose vocabulary matrix is larger than L2).
  int raster_m;
  // > 0 (plain mode only; TYR_GEMM_L2_PREFETCH, off by default): the producer asks L2 for the operand tiles of the k block
  // this many steps ahead of the one it loads, across tile boundaries.  Measured at 8 and 16 steps it made every NanoChat
  // shape slower (forward qkv 1248 -> 1108 TFLOP/s): all CTAs that share a tile repeat the request.
  int l2_prefetch;
  int* err;
  // Grouped mode (MoE): batch = number of groups, A and C are packed [rows, *] with group g owning
  // rows [group_offsets[g], group_offsets[g+1]).  group_tiles[g] is the exclusive prefix sum of
  // ceil(rows_g / 128) (batch + 1 entries): the kernel walks exactly the non-empty m-tiles without
  // the host ever reading the counts.
  const int* group_offsets;
  const int* group_tiles;
  // Tensor-parallel fusion over peer memory (ranks of one NVLink domain, plain peer loads / stores):
  //  tp_mode 1, GEMM -> reduce-scatter: row r of the product belongs to rank r / rows_per_rank; the
  //    epilogue stores the bf16 partial straight into that rank's slot buffer peer_c[owner] at row
  //    tp_rank * rows_per_rank + r % rows_per_rank (the owner sums its tp_world slots afterwards).
  //  tp_mode 2, all-gather -> GEMM: rows [j * rows_per_rank, (j+1) * rows_per_rank) of A live on rank j
  //    (peer_c[j] points at that shard).  Own rows are read in place.  Remote rows cross NVLink exactly
  //    once: the gather warps of all CTAs copy them, row tile by row tile in the order the tiles are
  //    consumed, into the local buffer `gather_buf` ([M, K], described by tmA) with plain peer loads and
  //    bump tile_ready[row tile]; the producer warp waits (bounded) for 2 * gridDim.x arrivals before its
  //    first TMA load of such a tile.  Gather warps never wait, so the kernel cannot deadlock.
  //  m_rot rotates the order of row tiles so that every rank starts with a different peer (mode 1)
  //  or with its own rows (mode 2).
  int tp_mode, tp_rank, tp_world, rows_per_rank, m_rot;
  void* peer_c[8];
  __nv_bfloat16* gather_buf;
  int* tile_ready;
  long long lda;
};

struct TmapPeers {
  CUtensorMap m[8];
};

// EPI_WARPS epilogue warps with EPI_BUFS staging tiles each (32 rows x 128 bytes, 128B swizzle) for the TMA stores.
template <int BN, int STAGES, int EPI_WARPS = 4, int EPI_BUFS = 2>
struct __align__(1024) GemmSmem {
  uint8_t a[STAGES][BM * BK * 2];
  uint8_t b[STAGES][BN * BK * 2];
  uint8_t out_stage[EPI_WARPS][EPI_BUFS][32 * 128];
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == 1) {
    float r = fmaxf(v, 0.f);
    return r * r;
  } else if (act == 2) {
    return fmaxf(v, 0.f);
  }
  return v;
}

// One 32-column chunk of the epilogue with the activation fixed at compile time (no per-element branches):
//   ACT 0: v = alpha * acc (+ beta * aux)      1: alpha * relu(acc)^2 (+ ...)      2: alpha * relu(acc) (+ ...)
//   ACT 3: v = alpha * acc * 2 * sqrt(aux)     (gradient of y = relu(z)^2 given aux = y)
template <int ACT>
__device__ __forceinline__ void epi_chunk(const uint32_t (&r)[32], const float (&ax)[32], bool use_aux, float alpha,
                                          float beta, float (&v)[32]) {
  if constexpr (ACT == 3) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = alpha * __uint_as_float(r[j]) * 2.f * sqrtf(fmaxf(ax[j], 0.f));
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      float a = __uint_as_float(r[j]);
      if constexpr (ACT == 1) { a = fmaxf(a, 0.f); a = a * a; }
      if constexpr (ACT == 2) a = fmaxf(a, 0.f);
      v[j] = alpha * a;
    }
    if (use_aux) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = fmaf(beta, ax[j], v[j]);
    }
  }
}

// PAIR = true: the grid is launched as clusters of two CTAs that share one 256 x BN output tile through
// tcgen05.mma.cta_group::2.  Each CTA loads its own 128 rows of A and its own half (BN / 2 columns) of B with plain TMA
// loads whose completion is counted on the leader's `full` barrier; the leader (cluster rank 0) issues every MMA and
// commits to the `empty` / `acc_full` barriers of both CTAs; each CTA's epilogue drains its own 128 accumulator rows
// and arrives on the leader's `acc_empty`.  A stage costs 32 KB instead of 48 KB and every operand byte in shared
// memory feeds twice the tensor-core work, which is what the single-CTA form runs short of.  Plain and K-split products
// in all four operand layouts; grouped rows and the tensor-parallel fusions stay on the single-CTA form.
//
// The pair form runs 320 threads: warps 2-5 drain the left half of the accumulator columns and warps 6-9 the right half
// (two epilogue warps per scheduler partition hide each other's latencies; with one, a 128 x 256 tile took about
// 15 000 cycles to drain, longer than its main loop at K = 1280).
template <int BN, int STAGES, bool A_MN, bool B_MN, bool PAIR>
__global__ void __launch_bounds__(PAIR ? 320 : 256, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA,
                         const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmC,
                         const __grid_constant__ TmapPeers tmP, GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int BNL = PAIR ? BN / 2 : BN;          // columns of B this CTA keeps in shared memory
  constexpr int TILE_M = PAIR ? 2 * BM : BM;       // rows of the tile one scheduler unit covers
  constexpr int EPI_WARPS = PAIR ? 8 : 4;
  constexpr int EPI_BUFS = PAIR ? 1 : 2;
  constexpr int EPI_CHUNKS = BN / 32 / (EPI_WARPS / 4);   // 32-column chunks each epilogue warp drains per tile
  using Smem = GemmSmem<BNL, STAGES, EPI_WARPS, EPI_BUFS>;
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                     ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
  // scheduler units: CTAs, or CTA pairs
  const int n_workers = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  const int worker = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);

  const int tiles_m = (p.M + TILE_M - 1) / TILE_M;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_kb = (p.K + BK - 1) / BK;
  // set-up that reads nothing another kernel wrote: it may overlap the tail of the kernel before this one
  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.acc_full[i], 1);
      mbar_init(&s.acc_empty[i], PAIR ? 2 * EPI_WARPS : EPI_WARPS);  // one arrival per epilogue warp (of both CTAs of a pair)
    }
    s.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(&s.tmem_base, 2 * BN);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&s.tmem_base, 2 * BN);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) {   // the peer's barriers must exist before anything arrives on them
    cluster_arrive();
    cluster_wait();
  }
  tc_fence_after();
  const uint32_t tmem_base = s.tmem_base;
  pdl_wait();

  const bool grouped = p.group_offsets != nullptr;
  const long long tiles = grouped ? static_cast<long long>(p.group_tiles[p.batch]) * tiles_n
                                  : static_cast<long long>(tiles_m) * tiles_n * p.batch;

  // Work range for this CTA, in (tile, k-block) units.
  long long unit_begin, unit_end;
  if (p.out_mode == 2) {
    const long long units = tiles * num_kb;
    unit_begin = units * worker / n_workers;
    unit_end = units * (worker + 1) / n_workers;
  } else {
    // tile-granular, strided assignment expressed in the same unit space
    unit_begin = 0;
    unit_end = 0;
  }

  constexpr uint32_t kStageBytes = BM * BK * 2 + BNL * BK * 2;

  // Segment iterator shared by the three roles (identical sequence in each).
  const long long whole_tiles = (tiles / n_workers) * n_workers;
  auto next_segment = [&](long long& cursor, long long& tile, int& kb0, int& kb1) -> bool {
    if (p.out_mode == 2 && p.sk_slabs > 0) {
      if (cursor < whole_tiles) {
        tile = cursor;
        kb0 = 0;
        kb1 = num_kb;
      } else {
        const long long rest = tiles - whole_tiles, v = cursor - whole_tiles;
        if (v >= rest * p.sk_slabs) return false;
        const int slab = static_cast<int>(v / rest);
        tile = whole_tiles + v % rest;
        kb0 = static_cast<int>(static_cast<long long>(num_kb) * slab / p.sk_slabs);
        kb1 = static_cast<int>(static_cast<long long>(num_kb) * (slab + 1) / p.sk_slabs);
      }
      cursor += n_workers;
      return true;
    } else if (p.out_mode == 2) {
      if (cursor >= unit_end) return false;
      tile = cursor / num_kb;
      kb0 = static_cast<int>(cursor % num_kb);
      long long remain = unit_end - cursor;
      kb1 = static_cast<int>(min(static_cast<long long>(num_kb), kb0 + remain));
      cursor += kb1 - kb0;
      return true;
    } else {
      if (cursor >= tiles) return false;
      tile = cursor;
      kb0 = 0;
      kb1 = num_kb;
      cursor += n_workers;
      return true;
    }
  };
  auto decode_tile = [&](long long tile, int& bi, int& m0, int& n0) {
    if (grouped) {
      // m-tile index over all groups -> owning group by binary search in the prefix table
      const int mt = static_cast<int>(tile / tiles_n);
      int lo = 0, hi = p.batch;                       // invariant: group_tiles[lo] <= mt < group_tiles[hi]
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (p.group_tiles[mid] <= mt) lo = mid; else hi = mid;
      }
      bi = lo;
      m0 = (mt - p.group_tiles[lo]) * BM;
      n0 = static_cast<int>(tile % tiles_n) * BN;
      return;
    }
    const int per_batch = tiles_m * tiles_n;
    bi = static_cast<int>(tile / per_batch);
    const int r = static_cast<int>(tile % per_batch);
    // n fastest: concurrently resident tiles share A rows and keep B (weights) in L2.
    if (p.raster_m) {
      m0 = (r % tiles_m) * TILE_M;
      n0 = (r / tiles_m) * BN;
    } else {
      m0 = ((r / tiles_n + p.m_rot) % tiles_m) * TILE_M;
      n0 = (r % tiles_n) * BN;
    }
    if (PAIR) m0 += static_cast<int>(cta_rank) * BM;   // this CTA's half of the pair's rows
  };
  const long long cursor0 = (p.out_mode == 2 && p.sk_slabs == 0) ? unit_begin : static_cast<long long>(worker);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      long long cursor = cursor0, tile;
      int kb0, kb1;
      uint32_t it = 0;
      bool ok = true;
      // second walk over the same segments, p.l2_prefetch k blocks ahead of the loads
      long long pf_cursor = cursor0, pf_tile;
      int pf_kb = 0, pf_kb1 = 0, pf_bi = 0, pf_m0 = 0, pf_n0 = 0;
      bool pf_live = p.l2_prefetch > 0;
      auto pf_step = [&]() {
        if (!pf_live) return;
        if (pf_kb >= pf_kb1) {
          if (!next_segment(pf_cursor, pf_tile, pf_kb, pf_kb1)) {
            pf_live = false;
            return;
          }
          decode_tile(pf_tile, pf_bi, pf_m0, pf_n0);
        }
        const int k0 = pf_kb * BK;
        if (!A_MN) {
          tma_prefetch_l2_3d(&tmA, k0, pf_m0, pf_bi);
        } else {
#pragma unroll
          for (int c = 0; c < BM / 64; ++c) tma_prefetch_l2_3d(&tmA, pf_m0 + c * 64, k0, pf_bi);
        }
        if (!B_MN) {
          tma_prefetch_l2_3d(&tmB, k0, pf_n0, pf_bi);
        } else {
#pragma unroll
          for (int c = 0; c < BN / 64; ++c) tma_prefetch_l2_3d(&tmB, pf_n0 + c * 64, k0, pf_bi);
        }
        ++pf_kb;
      };
      for (int i = 0; i < p.l2_prefetch; ++i) pf_step();
      while (ok && next_segment(cursor, tile, kb0, kb1)) {
        int bi, m0, n0;
        decode_tile(tile, bi, m0, n0);
        const int a_src = p.tp_mode == 2 ? m0 / p.rows_per_rank : 0;
        if (p.tp_mode == 2 && a_src != p.tp_rank) {
          // rows of a peer: wait until every gather warp has copied its part of this row tile
          const int* flag = p.tile_ready + m0 / BM;
          const int target = 2 * static_cast<int>(gridDim.x);
          const long long t0 = clock64();
          int seen;
          do {
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
            if (seen >= target) break;
            if (clock64() - t0 > kWaitBudgetCycles) {
              report_error(p.err, ERR_PEER_FLAG_TIMEOUT, m0 / BM);
              ok = false;
              break;
            }
            __nanosleep(100);
          } while (true);
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int st = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&s.empty[st], ph ^ 1, p.err, 100 + st)) {
            ok = false;
            break;
          }
          pf_step();
          const int k0 = kb * BK;
          if (PAIR) {
            // both CTAs' bytes are counted on the leader's barrier; only the leader arms it
            const uint32_t bar = mapa_shared(smem_u32(&s.full[st]), 0);
            if (cta_rank == 0) mbar_expect_tx(&s.full[st], 2 * kStageBytes);
            if (!A_MN) {
              tma_load_3d_pair(s.a[st], &tmA, bar, k0, m0, bi);
            } else {
#pragma unroll
              for (int c = 0; c < BM / 64; ++c)
                tma_load_3d_pair(s.a[st] + c * (64 * BK * 2), &tmA, bar, m0 + c * 64, k0, bi);
            }
            const int nb = n0 + static_cast<int>(cta_rank) * BNL;
            if (!B_MN) {
              tma_load_3d_pair(s.b[st], &tmB, bar, k0, nb, bi);
            } else {
#pragma unroll
              for (int c = 0; c < BNL / 64; ++c)
                tma_load_3d_pair(s.b[st] + c * (64 * BK * 2), &tmB, bar, nb + c * 64, k0, bi);
            }
            continue;
          }
          mbar_expect_tx(&s.full[st], kStageBytes);
          if (!A_MN) {
            if (p.group_offsets != nullptr)
              tma_load_3d(s.a[st], &tmA, &s.full[st], k0, p.group_offsets[bi] + m0, 0);
            else if (p.tp_mode == 2 && a_src == p.tp_rank)
              tma_load_3d(s.a[st], &tmP.m[a_src], &s.full[st], k0, m0 - a_src * p.rows_per_rank, bi);
            else
              tma_load_3d(s.a[st], &tmA, &s.full[st], k0, m0, bi);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_3d(s.a[st] + c * (64 * BK * 2), &tmA, &s.full[st], m0 + c * 64, k0, bi);
          }
          if (!B_MN) {
            tma_load_3d(s.b[st], &tmB, &s.full[st], k0, n0, bi);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_3d(s.b[st] + c * (64 * BK * 2), &tmB, &s.full[st], n0 + c * 64, k0, bi);
          }
        }
      }
      if (!ok) {
        s.abort_flag = 1;
        // Drain copies that were issued: each issued stage completes its own full barrier.
        for (uint32_t j = (it > STAGES ? it - STAGES : 0); j < it; ++j)
          mbar_wait(&s.full[j % STAGES], (j / STAGES) & 1, nullptr, 0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if ((!PAIR || cta_rank == 0) && elect_one()) {
      constexpr uint32_t idesc = make_idesc_f16(1, TILE_M, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      long long cursor = cursor0, tile;
      int kb0, kb1;
      uint32_t it = 0, seg = 0;
      bool ok = true;
      while (ok && next_segment(cursor, tile, kb0, kb1)) {
        const uint32_t buf = seg & 1;
        const uint32_t acc_ph = (seg >> 1) & 1;
        if (!(PAIR ? mbar_wait_cluster(&s.acc_empty[buf], acc_ph ^ 1, p.err, 200 + buf)
                   : mbar_wait(&s.acc_empty[buf], acc_ph ^ 1, p.err, 200 + buf))) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int st = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&s.full[st], ph, p.err, 300 + st)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(s.a[st]);
          const uint32_t b_addr = smem_u32(s.b[st]);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t da, db;
            if (!A_MN)
              da = make_smem_desc_sw128(a_addr + k * (UMMA_K * 2), 16, 1024);
            else
              da = make_smem_desc_sw128(a_addr + k * (UMMA_K * 128), 64 * BK * 2, 1024);
            if (!B_MN)
              db = make_smem_desc_sw128(b_addr + k * (UMMA_K * 2), 16, 1024);
            else
              db = make_smem_desc_sw128(b_addr + k * (UMMA_K * 128), 64 * BK * 2, 1024);
            if (PAIR)
              umma_f16_ss_pair(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            else
              umma_f16_ss(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          // frees the smem stage (in both CTAs of a pair) once these MMAs retire
          if (PAIR) {
            umma_commit_pair(smem_u32(&s.empty[st]));
            umma_commit_pair(mapa_shared(smem_u32(&s.empty[st]), 1));
          } else {
            umma_commit(&s.empty[st]);
          }
        }
        if (ok) {
          if (PAIR) {
            umma_commit_pair(smem_u32(&s.acc_full[buf]));
            umma_commit_pair(mapa_shared(smem_u32(&s.acc_full[buf]), 1));
          } else {
            umma_commit(&s.acc_full[buf]);
          }
        }
        ++seg;
      }
      if (!ok) s.abort_flag = 1;
    }
  } else if (!PAIR && warp >= 6) {
    // ------------------------------------------------------------------ gather warps (tp_mode 2)
    if (p.tp_mode == 2) {
      const long long nvec = static_cast<long long>(BM) * p.K / 8;       // 16-byte vectors per row tile (lda == K)
      const long long gid = static_cast<long long>(blockIdx.x) * 64 + (threadIdx.x - 192);
      const long long gstride = static_cast<long long>(gridDim.x) * 64;
      for (int i = 0; i < tiles_m; ++i) {
        const int mt = (i + p.m_rot) % tiles_m;
        const int src = mt * BM / p.rows_per_rank;
        if (src == p.tp_rank) continue;
        const uint4* from = reinterpret_cast<const uint4*>(
            reinterpret_cast<const __nv_bfloat16*>(p.peer_c[src]) + static_cast<long long>(mt * BM - src * p.rows_per_rank) * p.lda);
        uint4* to = reinterpret_cast<uint4*>(p.gather_buf + static_cast<long long>(mt) * BM * p.lda);
        for (long long v = gid; v < nvec; v += 8 * gstride) {
          uint4 buf[8];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (v + j * gstride < nvec) buf[j] = from[v + j * gstride];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (v + j * gstride < nvec) to[v + j * gstride] = buf[j];
        }
        __threadfence();
        asm volatile("fence.proxy.async;" ::: "memory");
        __syncwarp();
        if (lane == 0) asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(p.tile_ready + mt) : "memory");
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int quarter = warp & 3;  // TMEM lane quarter this warp may access
    const int epi = warp - 2;      // staging slot
    const int c_begin = (epi >> 2) * EPI_CHUNKS;
    long long cursor = cursor0, tile;
    int kb0, kb1;
    uint32_t seg = 0;
    bool ok = true;
    // bf16 outputs leave through shared memory and TMA stores (full 128-byte rows; also the efficient
    // packet size for stores that cross NVLink in tp_mode 1); grouped / SwiGLU outputs need row masks
    // and keep the direct stores.
    const bool tma_out = p.out_mode == 0 && p.group_offsets == nullptr && p.act != 4 && p.act != 5;
    uint32_t n_stores = 0;
    while (ok && next_segment(cursor, tile, kb0, kb1)) {
      int bi, m0, n0;
      decode_tile(tile, bi, m0, n0);
      const uint32_t buf = seg & 1;
      const uint32_t acc_ph = (seg >> 1) & 1;
      if (!mbar_wait(&s.acc_full[buf], acc_ph, p.err, 400 + buf)) {
        ok = false;
        break;
      }
      tc_fence_after();
      int row = m0 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + buf * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      bool row_ok = row < p.M;
      long long c_off, x_off;
      if (p.group_offsets != nullptr) {
        const int g0 = p.group_offsets[bi];
        row_ok = row < p.group_offsets[bi + 1] - g0;
        row += g0;
        c_off = static_cast<long long>(row) * p.ldc;
        x_off = static_cast<long long>(row) * p.ldaux;
      } else {
        c_off = static_cast<long long>(bi) * p.sC + static_cast<long long>(row) * p.ldc;
        x_off = static_cast<long long>(bi) * p.sAux + static_cast<long long>(row) * p.ldaux;
      }
      void* c_base = p.C;
      if (p.tp_mode == 1 && row_ok) {
        const int owner = row / p.rows_per_rank;
        c_base = p.peer_c[owner];
        c_off = (static_cast<long long>(p.tp_rank) * p.rows_per_rank + (row - owner * p.rows_per_rank)) * p.ldc;
      }
      if (p.act == 4 || p.act == 5) {
        // gated MLP over column halves of the tile: out[:, n0/2 + j] = act(acc[:, j]) * acc[:, BN/2 + j], act = SiLU (4) or
        // tanh-GELU (5)
        // with eight epilogue warps (CTA pairs) each set of four takes half of the output columns
        const int gc0 = (EPI_WARPS == 8) ? (epi >> 2) * (BN / 128) : 0;
        const int gc1 = (EPI_WARPS == 8) ? gc0 + BN / 128 : BN / 64;
#pragma unroll 1
        for (int c = gc0; c < gc1; ++c) {
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(t_row + c * 32, rg);
          tmem_ld_32x32(t_row + BN / 2 + c * 32, ru);
          tmem_wait_ld();
          if (c == gc1 - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
            if (PAIR) mbar_arrive_cluster(mapa_shared(smem_u32(&s.acc_empty[buf]), 0));
            else mbar_arrive(&s.acc_empty[buf]);
          }
          }
          const int col = n0 / 2 + c * 32;
          if (!row_ok || col >= p.N / 2) continue;
          __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + c_off + col;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float g = p.alpha * __uint_as_float(rg[j]);
            const float a = p.act == 4 ? g / (1.f + __expf(-g))
                                       : 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
            v[j] = a * (p.beta * __uint_as_float(ru[j]));
          }
          if (col + 32 <= p.N / 2) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 u;
              u.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
              u.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
              u.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
              u.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
              *reinterpret_cast<uint4*>(out + q * 8) = u;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col + j < p.N / 2) out[j] = __float2bfloat16(v[j]);
          }
        }
        ++seg;
        continue;
      }
#pragma unroll 1
      for (int c = c_begin; c < c_begin + EPI_CHUNKS; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_wait_ld();
        if (c == c_begin + EPI_CHUNKS - 1) {
          // this warp's part of the accumulator is read: hand the TMEM buffer back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (PAIR) mbar_arrive_cluster(mapa_shared(smem_u32(&s.acc_empty[buf]), 0));
            else mbar_arrive(&s.acc_empty[buf]);
          }
        }
        const int col = n0 + c * 32;
        if (tma_out) {
          if (col >= p.N) continue;            // a tile that ends inside the last valid chunk was flushed there
          if (!(c & 1)) {                      // about to refill a staging tile: its previous store must have read it
            if (lane == 0) tma_store_wait_read<EPI_BUFS - 1>();
            __syncwarp();
          }
        } else if (!row_ok || col >= p.N) {
          continue;
        }
        float v[32];
        const bool full = (col + 32 <= p.N);
        const bool use_aux = p.aux != nullptr && (p.beta != 0.f || p.act == 3) && row_ok;
        float ax[32];
        if (use_aux) {
          const __nv_bfloat16* axp = p.aux + x_off + col;
          if (full) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 u = *reinterpret_cast<const uint4*>(axp + q * 8);
              float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z),
                     f3 = unpack_bf16x2(u.w);
              ax[q * 8 + 0] = f0.x; ax[q * 8 + 1] = f0.y; ax[q * 8 + 2] = f1.x; ax[q * 8 + 3] = f1.y;
              ax[q * 8 + 4] = f2.x; ax[q * 8 + 5] = f2.y; ax[q * 8 + 6] = f3.x; ax[q * 8 + 7] = f3.y;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) ax[j] = (col + j < p.N) ? __bfloat162float(axp[j]) : 0.f;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) ax[j] = 0.f;
        }
        if (p.act == 0) epi_chunk<0>(r, ax, use_aux, p.alpha, p.beta, v);
        else if (p.act == 1) epi_chunk<1>(r, ax, use_aux, p.alpha, p.beta, v);
        else if (p.act == 2) epi_chunk<2>(r, ax, use_aux, p.alpha, p.beta, v);
        else epi_chunk<3>(r, ax, use_aux, p.alpha, p.beta, v);
        if (tma_out) {
          uint8_t* st = s.out_stage[epi][n_stores % EPI_BUFS] + lane * 128;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u;
            u.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
            u.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
            u.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
            u.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
            const int chunk = (c & 1) * 4 + q;                       // 16-byte chunk of the 128-byte row
            *reinterpret_cast<uint4*>(st + ((chunk ^ (lane & 7)) << 4)) = u;
          }
          if ((c & 1) || col + 32 >= p.N) {
            fence_proxy_async();
            __syncwarp();
            if (lane == 0 && m0 + quarter * 32 < p.M) {
              int y = m0 + quarter * 32;
              const CUtensorMap* tm = &tmC;
              if (p.tp_mode == 1) {
                const int owner = m0 / p.rows_per_rank;
                tm = &tmP.m[owner];
                y = p.tp_rank * p.rows_per_rank + (y - owner * p.rows_per_rank);
              }
              tma_store_3d(tm, s.out_stage[epi][n_stores % EPI_BUFS], col - (c & 1) * 32, y, bi);
              tma_store_commit();
            }
            ++n_stores;
          }
        } else if (p.out_mode == 0) {
          __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(c_base) + c_off + col;
          if (full) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 u;
              u.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
              u.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
              u.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
              u.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
              *reinterpret_cast<uint4*>(out + q * 8) = u;
            }
          } else {
            #pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col + j < p.N) out[j] = __float2bfloat16(v[j]);
          }
        } else if (p.out_mode == 1) {
          float* out = reinterpret_cast<float*>(p.C) + c_off + col;
          if (full) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<float4*>(out + q * 4) =
                  make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
          } else {
            #pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col + j < p.N) out[j] = v[j];
          }
        } else {
          float* out = reinterpret_cast<float*>(p.C) + c_off + col;
          if (full) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(out + q * 4),
                           "f"(v[q * 4]), "f"(v[q * 4 + 1]), "f"(v[q * 4 + 2]), "f"(v[q * 4 + 3])
                           : "memory");
          } else {
            #pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col + j < p.N) atomicAdd(out + j, v[j]);
          }
        }
      }
      ++seg;
    }
    if (tma_out && lane == 0) tma_store_wait_all();   // stores must have left shared memory before the CTA exits
  }

  tc_fence_before();
  __syncthreads();
  if (PAIR) {   // neither CTA may leave (or free TMEM) while its peer can still touch its shared memory or TMEM
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, 2 * BN);
    else tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ----------------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// 3-D bf16 tensor map {inner, outer, batch} with a 128-byte swizzled box {64, box_outer, 1}.
int make_tmap_bf16_3d(CUtensorMap* tm, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t batch, uint64_t ld_elems, uint64_t batch_stride_elems,
                      uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[3] = {inner, outer, batch};
  cuuint64_t strides[2] = {ld_elems * 2, batch_stride_elems * 2};
  if (batch <= 1) strides[1] = ld_elems * 2 * outer;
  cuuint32_t box[3] = {64, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

}  // namespace tyr

extern "C" {

struct TyrGemmArgs {
  const void* A;
  const void* B;
  void* C;
  const void* aux;
  int M, N, K, batch;
  long long lda, ldb, ldc, ldaux;   // leading strides in elements
  long long sA, sB, sC, sAux;       // batch strides in elements
  int a_mn, b_mn;                   // 0 = K-major (K contiguous), 1 = MN-major
  int out_mode;                     // 0 bf16, 1 fp32, 2 fp32 atomic accumulate (stream-K)
  int act;                          // 0 none, 1 relu^2, 2 relu
  float alpha, beta;
  int bn;                           // 128 or 256 (0 = choose)
  int sm_count;                     // CTAs to launch (0 = all SMs)
  int* err;
  void* stream;
  const int* group_offsets;         // grouped (MoE) mode, see GemmParams
  const int* group_tiles;
};

}  // extern "C"

// Per-device launch state: SM count, and which kernel instantiations already had their dynamic shared-memory limit
// raised on that device (the attribute is per device, so a second GPU used from the same process needs its own call).
constexpr int kMaxGemmDevices = 64;
static int g_sm_count_dev[kMaxGemmDevices] = {0};
static int g_pair_clusters_dev[kMaxGemmDevices] = {0};
static std::mutex g_gemm_mu;
static int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxGemmDevices) return 0;
  return dev;
}
static int device_sm_count() {
  const int dev = current_device();
  if (g_sm_count_dev[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    g_sm_count_dev[dev] = n > 0 ? n : 1;
  }
  return g_sm_count_dev[dev];
}
static const bool g_pair_enabled = [] { const char* e = getenv("TYR_GEMM_PAIR"); return e == nullptr || e[0] != '0'; }();
static const int g_l2_prefetch = [] { const char* e = getenv("TYR_GEMM_L2_PREFETCH"); const int v = e ? atoi(e) : 0; return v < 0 ? 0 : (v > 64 ? 64 : v); }();
static const bool g_raster_m = [] { const char* e = getenv("TYR_GEMM_RASTER_M"); return e == nullptr || e[0] != '0'; }();
static const bool g_aligned_split = [] { const char* e = getenv("TYR_GEMM_ALIGNED_SPLIT"); return e == nullptr || e[0] != '0'; }();

template <int BN, int STAGES, bool A_MN, bool B_MN, bool PAIR = false>
static int launch_gemm(const TyrGemmArgs& a, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                       const tyr::TmapPeers& tmP, const tyr::GemmParams& tp) {
  using namespace tyr;
  auto kern = gemm_bf16_tcgen05_kernel<BN, STAGES, A_MN, B_MN, PAIR>;
  constexpr size_t smem = sizeof(GemmSmem<PAIR ? BN / 2 : BN, STAGES, PAIR ? 8 : 4, PAIR ? 1 : 2>) + 1024;
  constexpr unsigned kThreads = PAIR ? 320 : 256;
  static bool configured[kMaxGemmDevices] = {false};
  const int dev = current_device();
  const int g_sm_count = device_sm_count();
  if (!configured[dev]) {
    std::lock_guard<std::mutex> lock(g_gemm_mu);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return 1000 + static_cast<int>(e);
    if (PAIR && g_pair_clusters_dev[dev] == 0) {
      // how many CTA pairs the device can keep resident at once (one CTA per SM, pairs within a TPC)
      cudaLaunchConfig_t qc = {};
      qc.gridDim = dim3(static_cast<unsigned>(g_sm_count & ~1));
      qc.blockDim = dim3(kThreads);
      qc.dynamicSmemBytes = smem;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = 2; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
      qc.attrs = qa; qc.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &qc) != cudaSuccess || n <= 0) n = g_sm_count / 2;
      if (n > g_sm_count / 2) n = g_sm_count / 2;
      g_pair_clusters_dev[dev] = n;
    }
    configured[dev] = true;
  }
  GemmParams p;
  p.M = a.M; p.N = a.N; p.K = a.K; p.batch = a.batch;
  p.C = a.C; p.aux = reinterpret_cast<const __nv_bfloat16*>(a.aux);
  p.ldc = a.ldc; p.ldaux = a.ldaux; p.sC = a.sC; p.sAux = a.sAux;
  p.alpha = a.alpha; p.beta = a.beta; p.act = a.act; p.out_mode = a.out_mode; p.err = a.err;
  p.group_offsets = a.group_offsets;
  p.group_tiles = a.group_tiles;
  p.tp_mode = tp.tp_mode; p.tp_rank = tp.tp_rank; p.tp_world = tp.tp_world;
  p.rows_per_rank = tp.rows_per_rank; p.m_rot = tp.m_rot;
  for (int i = 0; i < 8; ++i) p.peer_c[i] = tp.peer_c[i];
  p.gather_buf = tp.gather_buf; p.tile_ready = tp.tile_ready; p.lda = a.lda;
  constexpr int TILE_M = PAIR ? 2 * BM : BM;
  long long tiles = static_cast<long long>((a.M + TILE_M - 1) / TILE_M) * ((a.N + BN - 1) / BN) * a.batch;
  if (a.group_offsets != nullptr)   // host-side bound: every group may add one partial m-tile
    tiles = ((a.sA + BM - 1) / BM + (a.batch < a.sA ? a.batch : a.sA)) * ((a.N + BN - 1) / BN);
  // `grid` counts scheduler units: CTAs, or CTA pairs
  int grid = a.sm_count > 0 ? a.sm_count : g_sm_count;
  if (PAIR) {
    grid /= 2;
    if (g_pair_clusters_dev[dev] < grid) grid = g_pair_clusters_dev[dev];
    if (grid < 1) grid = 1;
  }
  if (a.out_mode != 2 && tiles < grid) grid = static_cast<int>(tiles);
  p.raster_m = (a.group_offsets == nullptr && tp.tp_mode == 0 && a.M < a.N && g_raster_m) ? 1 : 0;
  p.l2_prefetch = (a.group_offsets == nullptr && tp.tp_mode == 0) ? g_l2_prefetch : 0;
  p.sk_slabs = 0;
  if (a.out_mode == 2) {
    const int num_kb = (a.K + BK - 1) / BK;
    const long long units = tiles * num_kb;
    if (units < grid) grid = static_cast<int>(units);
    if (grid < 1) grid = 1;
    if (a.group_offsets == nullptr && g_aligned_split) {
      // Slab count for the tiles that do not fill a whole round: fewest k-block times over all rounds, an accumulate
      // epilogue counted as kEpilogueBlocks of them.
      const long long rest = tiles - (tiles / grid) * grid;
      constexpr int kEpilogueBlocks = 8;
      long long best = -1;
      p.sk_slabs = 1;
      for (int sl = 1; rest > 0 && sl <= num_kb && sl <= 128; ++sl) {
        const long long rounds = (rest * sl + grid - 1) / grid;
        const long long cost = rounds * ((num_kb + sl - 1) / sl + kEpilogueBlocks);
        if (best < 0 || cost < best) { best = cost; p.sk_slabs = sl; }
      }
    }
  }
  if (grid < 1) grid = 1;
  if (PAIR) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(2 * grid));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = reinterpret_cast<cudaStream_t>(a.stream);
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = at; cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, tmP, p);
    return e == cudaSuccess ? 0 : 2000 + static_cast<int>(e);
  }
  launch_dependent(kern, dim3(grid), dim3(256), smem, reinterpret_cast<cudaStream_t>(a.stream), tmA, tmB, tmC, tmP, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 2000 + static_cast<int>(e);
}

// Binds the given device (and its primary context) to the calling thread.  Host threads that
// never touched the runtime of this library (for example autograd worker threads) have no
// current context for the driver-level tensor-map encoder, and would default to device 0.
extern "C" TYR_EXPORT int tyr_bind_device(int device) {
  static thread_local int bound = -1;
  if (bound == device) return 0;
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return (int)e;
  e = cudaFree(0);
  if (e != cudaSuccess) return (int)e;
  bound = device;
  return 0;
}

extern "C" {
// Tensor-parallel fusion request for tyr_gemm_bf16_tp.
struct TyrTpArgs {
  int mode;            // 1: GEMM -> reduce-scatter slots, 2: all-gather -> GEMM
  int world, rank;
  int rows_per_rank;   // multiple of 128
  void* peers[8];      // mode 1: slot buffers [world * rows_per_rank, N] bf16 of every rank (row stride ldc)
                       // mode 2: A shards [rows_per_rank, K] bf16 of every rank (contiguous rows, lda == K)
  void* gather_buf;    // mode 2: local [world * rows_per_rank, K] bf16 landing buffer for the peers' rows
  int* tile_ready;     // mode 2: world * rows_per_rank / 128 counters (zeroed by this call)
};
}

static int gemm_impl(const TyrGemmArgs& a, const TyrTpArgs* tpa) {
  using namespace tyr;
  GemmParams tp{};
  TmapPeers tmP{};
  if (tpa != nullptr) {
    if (tpa->world < 1 || tpa->world > 8 || tpa->rank < 0 || tpa->rank >= tpa->world) return -10;
    if (tpa->rows_per_rank <= 0 || (tpa->rows_per_rank % BM) != 0 || a.M != tpa->rows_per_rank * tpa->world) return -11;
    if (a.a_mn || a.batch != 1 || a.out_mode != 0 || a.group_offsets != nullptr) return -12;
    tp.tp_mode = tpa->mode; tp.tp_rank = tpa->rank; tp.tp_world = tpa->world; tp.rows_per_rank = tpa->rows_per_rank;
    const int tiles_per_rank = tpa->rows_per_rank / BM;
    if (tpa->mode == 1) {
      tp.m_rot = ((tpa->rank + 1) % tpa->world) * tiles_per_rank;     // remote owners first, own rows last
      for (int i = 0; i < tpa->world; ++i) {
        if (tpa->peers[i] == nullptr || (reinterpret_cast<uintptr_t>(tpa->peers[i]) & 15)) return -13;
        tp.peer_c[i] = tpa->peers[i];
      }
    } else if (tpa->mode == 2) {
      tp.m_rot = tpa->rank * tiles_per_rank;                          // own rows first
      if (a.lda != a.K || tpa->gather_buf == nullptr || tpa->tile_ready == nullptr ||
          (reinterpret_cast<uintptr_t>(tpa->gather_buf) & 15))
        return -14;
      for (int i = 0; i < tpa->world; ++i) {
        if (tpa->peers[i] == nullptr || (reinterpret_cast<uintptr_t>(tpa->peers[i]) & 15)) return -13;
        tp.peer_c[i] = tpa->peers[i];
      }
      int r = make_tmap_bf16_3d(&tmP.m[tpa->rank], tpa->peers[tpa->rank], a.K, tpa->rows_per_rank, 1, a.lda, 0, BM);
      if (r) return 5000 + r;
      tp.gather_buf = reinterpret_cast<__nv_bfloat16*>(tpa->gather_buf);
      tp.tile_ready = tpa->tile_ready;
      cudaError_t e = cudaMemsetAsync(tpa->tile_ready, 0, sizeof(int) * tpa->world * tiles_per_rank,
                                      reinterpret_cast<cudaStream_t>(a.stream));
      if (e != cudaSuccess) return 7000 + static_cast<int>(e);
    } else {
      return -10;
    }
  }
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.batch <= 0) return -1;
  if ((reinterpret_cast<uintptr_t>(a.A) & 15) || (reinterpret_cast<uintptr_t>(a.B) & 15) ||
      (reinterpret_cast<uintptr_t>(a.C) & 15))
    return -2;
  if ((a.lda & 7) || (a.ldb & 7) || (a.group_offsets == nullptr && (a.sA & 7)) || (a.sB & 7)) return -3;
  if (a.out_mode == 0 ? (a.ldc & 7) : (a.ldc & 3)) return -4;
  if (a.aux && ((a.ldaux & 7) || (reinterpret_cast<uintptr_t>(a.aux) & 15))) return -5;
  int bn = a.bn;
  if (bn == 0) bn = (a.N <= 128) ? 128 : 256;
  CUtensorMap tmA, tmB;
  int r;
  if (a.group_offsets != nullptr) {
    if (a.a_mn || a.out_mode == 2 || a.sA <= 0 || a.group_tiles == nullptr) return -9;   // packed rows: K-major A, sA = total rows
    r = make_tmap_bf16_3d(&tmA, a.A, a.K, static_cast<uint64_t>(a.sA), 1, a.lda, 0, BM);
  } else if (!a.a_mn)
    r = make_tmap_bf16_3d(&tmA, (tpa != nullptr && tpa->mode == 2) ? tpa->gather_buf : a.A, a.K, a.M, a.batch, a.lda,
                          a.sA, BM);
  else
    r = make_tmap_bf16_3d(&tmA, a.A, a.M, a.K, a.batch, a.lda, a.sA, BK);
  if (r) return 3000 + r;
  // CTA pairs: plain products with a K-major A whose tiles are 256 columns wide
  const bool pair = g_pair_enabled && tpa == nullptr && a.group_offsets == nullptr && bn == 256 &&
                    (a.out_mode != 2 || g_aligned_split);
  if (!a.b_mn)
    r = make_tmap_bf16_3d(&tmB, a.B, a.K, a.N, a.batch, a.ldb, a.sB, pair ? bn / 2 : bn);
  else
    r = make_tmap_bf16_3d(&tmB, a.B, a.N, a.K, a.batch, a.ldb, a.sB, BK);
  if (r) return 4000 + r;
  CUtensorMap tmC{};
  if (a.out_mode == 0 && a.group_offsets == nullptr && a.act != 4 && a.act != 5) {
    if (tpa != nullptr && tpa->mode == 1) {
      for (int i = 0; i < tpa->world; ++i) {
        r = make_tmap_bf16_3d(&tmP.m[i], tpa->peers[i], a.N, static_cast<uint64_t>(tpa->world) * tpa->rows_per_rank, 1,
                              a.ldc, 0, 32);
        if (r) return 6000 + r;
      }
      tmC = tmP.m[tpa->rank];
    } else {
      r = make_tmap_bf16_3d(&tmC, a.C, a.N, a.M, a.batch, a.ldc, a.sC, 32);
      if (r) return 6000 + r;
    }
  }
#define TYR_DISPATCH(BNv, ST)                                                   \
  do {                                                                          \
    if (!a.a_mn && !a.b_mn) return launch_gemm<BNv, ST, false, false>(a, tmA, tmB, tmC, tmP, tp); \
    if (!a.a_mn && a.b_mn) return launch_gemm<BNv, ST, false, true>(a, tmA, tmB, tmC, tmP, tp);   \
    if (a.a_mn && a.b_mn) return launch_gemm<BNv, ST, true, true>(a, tmA, tmB, tmC, tmP, tp);     \
    return launch_gemm<BNv, ST, true, false>(a, tmA, tmB, tmC, tmP, tp);                      \
  } while (0)
  if (pair) {
    if (!a.a_mn && !a.b_mn) return launch_gemm<256, 6, false, false, true>(a, tmA, tmB, tmC, tmP, tp);
    if (!a.a_mn && a.b_mn) return launch_gemm<256, 6, false, true, true>(a, tmA, tmB, tmC, tmP, tp);
    if (a.a_mn && a.b_mn) return launch_gemm<256, 6, true, true, true>(a, tmA, tmB, tmC, tmP, tp);
    return launch_gemm<256, 6, true, false, true>(a, tmA, tmB, tmC, tmP, tp);
  }
  if (bn == 256) TYR_DISPATCH(256, 4);
  if (bn == 128) TYR_DISPATCH(128, 6);
#undef TYR_DISPATCH
  return -6;
}

// Returns 0 on success; negative = invalid argument; positive = CUDA/driver error.
extern "C" TYR_EXPORT int tyr_gemm_bf16(const TyrGemmArgs* args) { return gemm_impl(*args, nullptr); }

// The same product with its collective fused in (see GemmParams::tp_mode).  Mode 2 ignores args->A.
extern "C" TYR_EXPORT int tyr_gemm_bf16_tp(const TyrGemmArgs* args, const TyrTpArgs* tp) {
  if (tp == nullptr) return -10;
  return gemm_impl(*args, tp);
}

// ----------------------------------------------------------------------------------------
// Newton-Schulz iteration chain on the GEMM above (Muon orthogonalisation).
//
//   X <- a X + (b A + c A A) X,   A = X X^T        (X: [batch, R, C] bf16, already normalised)
//
// Tall matrices (R > C) run the same iteration on X^T through operand layouts.  Each iteration is
// three GEMM launches with the scale/add terms in the epilogue.  Needs scratch for A, bA + cAA
// (both [batch, S, S], S = min(R, C)) and one extra X buffer; the result is written back to `x`.
// Reference: cc/src/tyr_polar.cpp:267-317 (15 cuBLAS GEMMs + 15 elementwise kernels per matrix).
// ----------------------------------------------------------------------------------------
extern "C" TYR_EXPORT long long tyr_newton_schulz_scratch_bytes(int batch, int R, int C) {
  const long long S = R < C ? R : C;
  return (2LL * batch * S * S + 1LL * batch * R * C) * 2;
}

static int ns_chain(void* x, void* scratch, int batch, int R, int C, int iters, float a, float b,
                    float c, int* err, void* stream) {
  const long long S = R < C ? R : C;
  __nv_bfloat16* A = reinterpret_cast<__nv_bfloat16*>(scratch);
  __nv_bfloat16* Bm = A + 1LL * batch * S * S;
  __nv_bfloat16* X2 = Bm + 1LL * batch * S * S;
  __nv_bfloat16* cur = reinterpret_cast<__nv_bfloat16*>(x);
  __nv_bfloat16* nxt = X2;
  const bool tall = R > C;
  for (int it = 0; it < iters; ++it) {
    TyrGemmArgs g;
    memset(&g, 0, sizeof(g));
    g.batch = batch; g.alpha = 1.f; g.beta = 0.f; g.err = err; g.stream = stream;
    // A = X X^T (wide) or X^T X (tall)
    g.A = cur; g.B = cur; g.C = A; g.M = (int)S; g.N = (int)S; g.K = tall ? R : C;
    g.lda = C; g.ldb = C; g.ldc = S; g.sA = 1LL * R * C; g.sB = 1LL * R * C; g.sC = S * S;
    g.a_mn = tall ? 1 : 0; g.b_mn = tall ? 1 : 0;
    int rc = tyr_gemm_bf16(&g);
    if (rc) return rc;
    // Bm = c A A + b A   (A symmetric)
    memset(&g, 0, sizeof(g));
    g.batch = batch; g.err = err; g.stream = stream;
    g.A = A; g.B = A; g.C = Bm; g.aux = A; g.M = g.N = g.K = (int)S;
    g.lda = g.ldb = g.ldc = g.ldaux = S; g.sA = g.sB = g.sC = g.sAux = S * S;
    g.alpha = c; g.beta = b;
    rc = tyr_gemm_bf16(&g);
    if (rc) return rc;
    // X' = Bm X + a X (wide)   or   X' = X Bm + a X (tall)
    memset(&g, 0, sizeof(g));
    g.batch = batch; g.err = err; g.stream = stream; g.alpha = 1.f; g.beta = a;
    g.C = nxt; g.aux = cur; g.ldc = C; g.ldaux = C; g.sC = g.sAux = 1LL * R * C;
    g.M = R; g.N = C;
    if (!tall) {
      g.A = Bm; g.lda = S; g.sA = S * S; g.a_mn = 0;
      g.B = cur; g.ldb = C; g.sB = 1LL * R * C; g.b_mn = 1; g.K = R;
    } else {
      g.A = cur; g.lda = C; g.sA = 1LL * R * C; g.a_mn = 0;
      g.B = Bm; g.ldb = S; g.sB = S * S; g.b_mn = 0; g.K = C;
    }
    rc = tyr_gemm_bf16(&g);
    if (rc) return rc;
    __nv_bfloat16* t = cur; cur = nxt; nxt = t;
  }
  if (cur != x) {
    cudaError_t e = cudaMemcpyAsync(x, cur, 2LL * batch * R * C, cudaMemcpyDeviceToDevice,
                                    reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return 2000 + static_cast<int>(e);
  }
  return 0;
}

// Caller-provided scratch of at least tyr_newton_schulz_scratch_bytes(batch, R, C) bytes.
extern "C" TYR_EXPORT int tyr_newton_schulz_bf16(void* x, void* scratch, long long scratch_bytes,
                                                 int batch, int R, int C, int iters, float a, float b,
                                                 float c, int* err, void* stream) {
  if (batch <= 0 || R <= 0 || C <= 0 || iters < 0 || (R & 7) || (C & 7)) return -1;
  if (scratch_bytes < tyr_newton_schulz_scratch_bytes(batch, R, C)) return -7;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(scratch) & 15)) return -2;
  return ns_chain(x, scratch, batch, R, C, iters, a, b, c, err, stream);
}

// ----------------------------------------------------------------------------------------
// Allocation-free variant (declared in no_alloc.h): temporaries in a file-scope device array.
// ----------------------------------------------------------------------------------------
#include "no_alloc.h"

static __device__ __align__(256) unsigned char g_ns_static_scratch[TYR_NS_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void* g_ns_static_ptr[kMaxDevices] = {nullptr};
std::mutex g_ns_static_mu;

// `g_ns_static_scratch` is only a host-side handle here; the address a kernel can use has to be
// asked for, per device, with that device current.
int ns_static_address(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return 9000 + static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return 9000;
  std::lock_guard<std::mutex> lock(g_ns_static_mu);
  if (g_ns_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_ns_static_scratch);
    if (e != cudaSuccess) return 9000 + static_cast<int>(e);
    g_ns_static_ptr[dev] = p;
  }
  *out = g_ns_static_ptr[dev];
  return 0;
}
}  // namespace

extern "C" TYR_EXPORT int tyr_newton_schulz_bf16_static(void* x, int batch, int R, int C, int iters,
                                                        float a, float b, float c, int* err,
                                                        void* stream) {
  if (batch <= 0 || R <= 0 || C <= 0 || iters < 0 || (R & 7) || (C & 7)) return -1;
  if (reinterpret_cast<uintptr_t>(x) & 15) return -2;
  if (tyr_newton_schulz_scratch_bytes(batch, R, C) > TYR_NS_STATIC_SCRATCH_BYTES) return -8;
  void* scratch = nullptr;
  int rc = ns_static_address(&scratch);
  if (rc) return rc;
  return ns_chain(x, scratch, batch, R, C, iters, a, b, c, err, stream);
}
