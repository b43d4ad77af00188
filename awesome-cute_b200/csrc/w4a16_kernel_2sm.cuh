// The W4A16 GEMM for large batches on CTA PAIRS (tcgen05 cta_group::2).
//
// Same formulation as w4a16_kernel.cuh (D[n, m] = sum_k W[n, k] * A[m, k], dequantised weights as the UMMA A
// operand in tensor memory, activations as the B operand in shared memory), but two CTAs of a cluster, on
// neighbouring SMs, share one tile of 256 weight columns x TM batch rows:
//   * CTA r of the pair owns weight columns [256 T + 128 r, +128): it streams, dequantises and keeps them in ITS
//     tensor memory, and holds ITS 128 accumulator rows;
//   * CTA r loads only rows [m0 + r TM/2, +TM/2) of the activation tile: the UMMA (M = 256, N = TM) reads the B
//     operand half from each CTA's shared memory.  Per CTA a 128-k stage is 8 KB of weights + TM x 128 B of
//     activations instead of + TM x 256 B: the single-CTA kernel is bound by bytes in flight (all of shared memory
//     holds only 4 stages of a 192-row tile); here 6 stages fit;
//   * the leader (cluster rank 0) issues every MMA; completion is signalled to both CTAs with one commit.
// Barriers the leader's MMA warp waits on live in the leader: the partner's dequant and epilogue warps arrive on
// them through the cluster address space, and the partner's activation loads count their bytes there.
// Everything else (roles, stream-K with sentinel slots, bounded waits, dependent launch) is as in the single-CTA
// kernel.  The reference has no counterpart (it is an sm_80 kernel, gemm/marlin_gemm/marlin_cute_trait.h).
#pragma once
#include "w4a16_kernel.cuh"

namespace w4a16 {

template <int TM, int KS_ = 128, int OUT = OUT_PLAIN>
struct Config2 {
  static_assert(TM == 32 || TM == 64 || TM == 128 || TM == 192, "batch tile of the pair");
  static_assert(KS_ == 128 || KS_ == 256, "k per stage");
  static constexpr int KS = KS_;
  static constexpr int KCHUNKS = KS / 64;
  static constexpr int GROUPS = KS / 128;
  static constexpr int HALF_ROWS = TM / 2;                   // activation rows held by each CTA
  static constexpr int W_BYTES = KS * TILE_N / 2;            // 8 or 16 KB
  static constexpr int A_BYTES = HALF_ROWS * KS * 2;         // [KS/64 chunks][TM/2 rows][128 B]
  static constexpr int S_BYTES = GROUPS * TILE_N * 2;
  static constexpr int STAGE_BYTES = W_BYTES + A_BYTES + S_BYTES;
  static constexpr int ACC_STRIDE = TM;
  static constexpr int WBUF_COL0 = 2 * ACC_STRIDE;
  static constexpr int WBUF_COLS = KS / 2;
  static constexpr int TMEM_COLS = 512;
  static constexpr int WBUFS_RAW = (TMEM_COLS - WBUF_COL0) / WBUF_COLS;
  static constexpr int WBUFS = WBUFS_RAW > 4 ? 4 : WBUFS_RAW;
  static_assert(WBUFS >= 2, "TMEM budget");
  static constexpr int BAR_BYTES = 1024;
  static constexpr int GATHER_BYTES = OUT != OUT_PLAIN ? GATHER_SLAB_BYTES : 0;
  static constexpr int SMEM_MAX = 227 * 1024;
  static constexpr int STAGES_RAW = (SMEM_MAX - BAR_BYTES - GATHER_BYTES - 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static_assert(STAGES >= 3, "ring too shallow");
  static constexpr int NSETS = 2, NDQ = 8;
  static constexpr int THREADS = (NDQ + EPI_WARPS + 2) * 32;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + GATHER_BYTES + 1024;
};

struct Bars2 {  // same offsets in both CTAs of the pair
  uint64_t wsfull[8];    // weights + scales of a stage landed in THIS CTA                    (local)
  uint64_t afull[8];     // both halves of the activation tile landed                         (used in the leader)
  uint64_t empty[8];     // stage free again: this CTA's dequant warps + the pair's MMA commit (local)
  uint64_t wfull[4];     // TMEM operand buffer written in both CTAs                          (used in the leader)
  uint64_t wempty[4];    // ... read by the MMAs (commit to both CTAs)                        (local)
  uint64_t accfull[2];   // accumulator complete (commit to both CTAs)                        (local)
  uint64_t accempty[2];  // accumulator drained by both CTAs' epilogue warps                  (used in the leader)
  uint64_t drain;
  uint64_t gfull[2];     // gathering epilogue: this CTA's four epilogue warps have staged a chunk     (local)
  uint32_t tmem_base;
  int abort;
};
static_assert(sizeof(Bars2) <= 1024, "barrier block");

// The segments (tile, k-stages [kb, ke)) of one pair, in the order it runs them: first whole tiles taken round-robin
// (tile = pair, pair + workers, ... below sk_tile0), then its contiguous range of the stream-K part.  Round-robin
// whole tiles keep the tiles in flight at one time next to each other (they share activation rows and weight columns,
// so both stay in L2); with contiguous ranges alone the pairs are spread over the whole problem and a batch whose
// activations exceed L2 is re-read from HBM for every tile.  The stream-K part at the end levels the last wave, as in
// the reference's dense stream-K demo (gemm/streamk_gemm/dp_sk_block.h:82-173 splits full waves from the remainder).
struct Walk {
  int dp_tile, stride, sk_tile0, it, it_end, k_iters;
  __device__ __forceinline__ Walk(const Params &p, int pair)
      : dp_tile(pair), stride(p.workers), sk_tile0(p.sk_tile0), k_iters(p.k_iters) {
    it = min(p.total_iters, pair * p.iters_per_cta);
    it_end = min(p.total_iters, it + p.iters_per_cta);
  }
  __device__ __forceinline__ bool next(int &tile, int &kb, int &ke) {
    if (dp_tile < sk_tile0) {
      tile = dp_tile, kb = 0, ke = k_iters;
      dp_tile += stride;
      return true;
    }
    if (it >= it_end) return false;
    const int t = it / k_iters;
    kb = it - t * k_iters;
    ke = min(k_iters, kb + (it_end - it));
    tile = sk_tile0 + t;
    it += ke - kb;
    return true;
  }
};

// tile index -> (256-column tile, batch tile)
__device__ __forceinline__ void tile_nm(const Params &p, int tile, int &n_idx2, int &m_idx) {
  if (p.m_fast) {
    n_idx2 = tile / p.m_tiles;
    m_idx = tile - n_idx2 * p.m_tiles;
  } else {
    m_idx = tile / p.n_tiles;
    n_idx2 = tile - m_idx * p.n_tiles;
  }
}

// Batch rows the MMAs of a tile starting at row m0 cover: the rows that exist, rounded up to the UMMA N granule of 16.
// A ragged last batch tile (and a batch smaller than the tile) then costs tensor time and fix-up traffic for its own
// rows only.  Each CTA of the pair supplies half of them, so CTA r loads rows [m0 + r * width / 2, ...).
template <int TM>
__device__ __forceinline__ int tile_width(const Params &p, int m0) {
  const int rows = min(TM, p.m - m0);
  return max(16, (rows + 15) & ~15);
}

template <int TM, int KS_, bool GROUPED, int OUT = OUT_PLAIN>
__global__ void __launch_bounds__(Config2<TM, KS_>::THREADS, 1)
w4a16_tc2_kernel(const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmA,
                 const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmC, const Params p) {
  using Cfg = Config2<TM, KS_, OUT>;
  constexpr bool GATHER = OUT == OUT_GATHER;
  using namespace sm100;
  constexpr int S = Cfg::STAGES, NDQ = Cfg::NDQ, KS = Cfg::KS;
  constexpr int PRODUCER_WARP = NDQ + EPI_WARPS, MMA_WARP = NDQ + EPI_WARPS + 1;
  constexpr bool HELP = TM >= 64 && OUT == OUT_PLAIN;   // dequant warps help to finish a split tile (as in the single-CTA kernel)
  constexpr uint32_t WS_TX = Cfg::W_BYTES + (GROUPED ? Cfg::S_BYTES : 0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *sW = smem;
  uint8_t *sA = sW + S * Cfg::W_BYTES;
  uint8_t *sS = sA + S * Cfg::A_BYTES;
  Bars2 *bars = reinterpret_cast<Bars2 *>(sS + S * Cfg::S_BYTES);
  volatile int *abort = &bars->abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const int pair = blockIdx.x >> 1;

  // ---- the PAIR's share: dp_waves whole tiles, then its slice of the linearised (256-column tile, k-stage) space of
  // the stream-K part; p.n_tiles counts 256-column tiles
  const int it_begin = min(p.total_iters, pair * p.iters_per_cta);
  const int it_end = min(p.total_iters, it_begin + p.iters_per_cta);
  const int nsteps = p.dp_waves * p.k_iters + (it_end - it_begin);

  auto issue_weights = [&](int st, int n_idx2, int kk) {   // this CTA's 128 columns of the pair's tile
    const uint32_t full = smem_u32(&bars->wsfull[st]);
    const int n_idx = 2 * n_idx2 + (int)rank;
    mbar_expect_tx(full, WS_TX);
    tma_load_3d(smem_u32(sW) + st * Cfg::W_BYTES, &tmB, 0, n_idx * 8, kk * (KS / 16), full);
    if (GROUPED) tma_load_2d(smem_u32(sS) + st * Cfg::S_BYTES, &tmS, n_idx * TILE_N, kk * Cfg::GROUPS, full);
  };
  auto issue_acts = [&](int st, int m0, int kk) {          // this CTA's half of the activation rows
    const uint32_t leader_full = map_to_cta(smem_u32(&bars->afull[st]), 0);
    if (rank == 0) mbar_expect_tx(smem_u32(&bars->afull[st]), 2 * Cfg::A_BYTES);
    tma_load_3d_pair(smem_u32(sA) + st * Cfg::A_BYTES, &tmA, 0, m0 + (int)rank * (tile_width<TM>(p, m0) >> 1), kk * Cfg::KCHUNKS, leader_full);
  };

  // ---- prologue
  if (warp == PRODUCER_WARP && lane == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(smem_u32(&bars->wsfull[i]), 1);
      mbar_init(smem_u32(&bars->afull[i]), 1);
      mbar_init(smem_u32(&bars->empty[i]), 4 + 1);
    }
    for (int i = 0; i < Cfg::WBUFS; ++i) {
      mbar_init(smem_u32(&bars->wfull[i]), 8);       // four dequant warps of each CTA
      mbar_init(smem_u32(&bars->wempty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars->accfull[i]), 1);
      mbar_init(smem_u32(&bars->accempty[i]), 2 * EPI_WARPS);
      mbar_init(smem_u32(&bars->gfull[i]), EPI_WARPS);
    }
    mbar_init(smem_u32(&bars->drain), 1);
    bars->abort = 0;
    mbar_fence_init();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == MMA_WARP) {          // one warp in EACH CTA of the pair, same warp index, same destination offset
    tmem_alloc_pair(smem_u32(&bars->tmem_base), Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();              // both CTAs' barriers exist before anything can arrive on them
  tc_fence_after();
  const uint32_t tmem = __shfl_sync(0xffffffffu, bars->tmem_base, 0);

  if (warp < NDQ) {
    // =========================================================== dequant warps (as in the single-CTA kernel)
    const int quad = warp & 3, set = warp >> 2;
    const int row = quad * 32 + lane;
    const int nr = row & 63, blk = row >> 6;
    const int j = nr >> 4, r8 = nr & 7;
    const uint32_t shift = ((nr >> 3) & 1) ? 8u : 0u;
    const uint32_t base_off = (uint32_t)((4 * blk + (r8 >> 1)) * 128 + 64 * ((r8 & 1) ^ blk) + 4 * j);
    uint32_t toff[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) toff[t] = base_off + 16u * (uint32_t)(t ^ (r8 >> 1));
    const uint32_t s_off = (uint32_t)(2 * (64 * blk + 8 * (nr & 7) + (nr >> 3)));
    const uint32_t sW_u = smem_u32(sW), sS_u = smem_u32(sS);
    const uint32_t one2 = 0x3c003c00u;
    const uint32_t t_lane = tmem + ((uint32_t)(quad * 32) << 16) + Cfg::WBUF_COL0;
    long long d_full = 0, d_wempty = 0, d_work = 0;
    for (int g = set; g < nsteps; g += Cfg::NSETS) {
      const int st = g % S, wb = g % Cfg::WBUFS;
      const long long c0 = W4A16_CLK();
      if (!warp_wait(smem_u32(&bars->wsfull[st]), (g / S) & 1, abort, p.wait_ns)) { give_up(p, abort, 11); break; }
      const long long c1 = W4A16_CLK();
      d_full += c1 - c0;
      const uint32_t wbase = sW_u + st * Cfg::W_BYTES;
      __half2 sc = *reinterpret_cast<const __half2 *>(&one2);
      bool buf_ok = true;
#pragma unroll
      for (int half = 0; half < Cfg::KCHUNKS; ++half) {
        if (GROUPED && (half & 1) == 0) {   // a new 128-k group starts every second 64-k chunk
          uint16_t sv;
          asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sv) : "r"(sS_u + st * Cfg::S_BYTES + (half >> 1) * (TILE_N * 2) + s_off));
          sc = __half2half2(__ushort_as_half(sv));
        }
        uint32_t v[32];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            uint32_t w;
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w) : "r"(wbase + (half * 4 + r) * 1024 + toff[t]));
            dequant_word<GROUPED>(w >> shift, sc, v[r * 8 + t], v[r * 8 + 4 + t]);
          }
        }
        if (half == 0) {
          const long long c2 = W4A16_CLK();
          buf_ok = warp_wait(smem_u32(&bars->wempty[wb]), ((g / Cfg::WBUFS) & 1) ^ 1, abort, p.wait_ns);
          tc_fence_after();
          d_wempty += W4A16_CLK() - c2;
          if (!buf_ok) break;
        }
        tmem_st_32x32b_x32(t_lane + wb * Cfg::WBUF_COLS + half * 32, v);
      }
      if (!buf_ok) { give_up(p, abort, 12); break; }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_cluster(map_to_cta(smem_u32(&bars->wfull[wb]), 0));   // the leader's MMA warp counts both CTAs
        mbar_arrive(smem_u32(&bars->empty[st]));
      }
      d_work += W4A16_CLK() - c1;
    }
    if (warp == 0) { W4A16_BUCKET(4, d_full); W4A16_BUCKET(5, d_wempty); W4A16_BUCKET(6, d_work); }
    if (HELP) {
      // ---- help to finish the CTA's last tile if it is a split one (chunks 16*(1+set), +48, ... of this quadrant)
      int l_tile = 0, l_kb = 1, l_ke = 0, l_seg = -1;
      {
        Walk walk(p, pair);
        int t, kb, ke;
        while (walk.next(t, kb, ke)) l_tile = t, l_kb = kb, l_ke = ke, ++l_seg;
      }
      if (l_seg >= 0 && l_kb == 0 && l_ke < p.k_iters) {
        int l_n, l_m;
        tile_nm(p, l_tile, l_n, l_m);
        const int n0 = (2 * l_n + (int)rank) * TILE_N, m0 = l_m * TM;
        const int acc = l_seg & 1;
        const int last_pair = ((l_tile - p.sk_tile0 + 1) * p.k_iters - 1) / p.iters_per_cta;
        __half sch = __float2half(1.0f);
        if (!GROUPED) {
          const int c32 = row & 31;
          sch = p.s[n0 + row - c32 + 8 * ((c32 & 7) >> 1) + 2 * (c32 >> 3) + (c32 & 1)];
        }
        pdl_wait_prior_grid();
        bool ok = warp_wait(smem_u32(&bars->accfull[acc]), (l_seg >> 1) & 1, abort, p.wait_ns);
        tc_fence_after();
        const uint64_t t0 = globaltimer_ns();
        const uint32_t t_acc = tmem + ((uint32_t)(quad * 32) << 16) + acc * Cfg::ACC_STRIDE;
        const int width = tile_width<TM>(p, m0);
#pragma unroll 1
        for (int c0 = 16 * (1 + set); c0 < width && ok; c0 += 48) {
          uint32_t v[16];
          tmem_ld_32x32b_x16(t_acc + c0, v);
          tc_wait_ld();
          // contributors are the same-rank CTAs of the following pairs: slots 2 (pair + 1) + rank, + 2, ...
          ok = fold_partial_slices<2>(v, p.partials, TM, c0, row, 2 * (pair + 1) + (int)rank, 2, last_pair - pair, abort, t0, p.wait_ns);
          if (!ok) break;
#pragma unroll
          for (int i = 0; i < 16; ++i) {   // (never the gathering form: HELP is off there)
            const int mm = m0 + c0 + i;
            __half h = __float2half(__uint_as_float(v[i]));
            if (!GROUPED) h = __hmul(h, sch);  // per-channel scale after the fp16 convert (marlin_cute_trait.h:764-769)
            if (mm < p.m) p.C[(size_t)mm * p.n + n0 + row] = h;
          }
        }
        if (!ok) give_up(p, abort, 19);
      }
    }
  } else if (warp < NDQ + EPI_WARPS) {
    // =========================================================== epilogue warps: this CTA's 128 columns, all TM rows
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t t_lane = tmem + ((uint32_t)(quad * 32) << 16);
    pdl_wait_prior_grid();
    __half *slabs = reinterpret_cast<__half *>(reinterpret_cast<uint8_t *>(bars) + Cfg::BAR_BYTES);   // gathering form only
    int gcount = 0;
    Walk walk(p, pair);
    int tile, kb, ke;
    for (int seg = 0; walk.next(tile, kb, ke); ++seg) {
      int n_idx2, m_idx;
      tile_nm(p, tile, n_idx2, m_idx);
      const int n0 = (2 * n_idx2 + (int)rank) * TILE_N, m0 = m_idx * TM;
      const int acc = seg & 1;
      const bool finisher = (kb == 0);
      // contributors are the same-rank CTAs of the following pairs: slots blockIdx.x + 2, + 4, ...
      const int last_pair = (finisher && ke < p.k_iters) ? ((tile - p.sk_tile0 + 1) * p.k_iters - 1) / p.iters_per_cta : pair;
      const int ncontrib = last_pair - pair;
      __half sch = __float2half(1.0f);
      if (!GROUPED && finisher) {
        const int c32 = row & 31;
        sch = p.s[n0 + row - c32 + 8 * ((c32 & 7) >> 1) + 2 * (c32 >> 3) + (c32 & 1)];
      }
      if (!warp_wait(smem_u32(&bars->accfull[acc]), (seg >> 1) & 1, abort, p.wait_ns)) { give_up(p, abort, 13); break; }
      tc_fence_after();
      uint32_t *part = p.partials + ((size_t)blockIdx.x * TM) * TILE_N + row;
      bool ok = true;
      const uint64_t t0 = ncontrib > 0 ? globaltimer_ns() : 0ull;
      constexpr int FLY = 2;
      const int c_step = (HELP && finisher && ncontrib > 0) ? 48 : 16;   // the dequant warps take the other chunks
      const int width = tile_width<TM>(p, m0);
#pragma unroll 1
      for (int c0 = 0; c0 < width && ok; c0 += c_step) {
        uint32_t v[16];
        tmem_ld_32x32b_x16(t_lane + acc * Cfg::ACC_STRIDE + c0, v);
        tc_wait_ld();
        if (!finisher) {
#pragma unroll
          for (int i = 0; i < 16; ++i) st_slot(part + (size_t)(c0 + i) * TILE_N, v[i] == PARTIAL_IDLE ? 0x7fffffffu : v[i]);
        } else {
          if (ncontrib > 0) ok = fold_partial_slices<FLY>(v, p.partials, TM, c0, row, 2 * (pair + 1) + (int)rank, 2, ncontrib, abort, t0, p.wait_ns);
          if (!ok) break;
          if constexpr (GATHER) {
            if (!store_chunk_gather4<GROUPED>(p, v, sch, m0 + c0, n0, quad, lane, slabs, smem_u32(&bars->gfull[0]), gcount, abort)) {
              ok = false;
              break;
            }
          } else if constexpr (OUT == OUT_TMA) {
            if (!store_chunk_tma<GROUPED>(p, &tmC, v, sch, m0 + c0, n0, quad, lane, slabs, smem_u32(&bars->gfull[0]), gcount, abort)) {
              ok = false;
              break;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int mm = m0 + c0 + i;
              __half h = __float2half(__uint_as_float(v[i]));
              if (!GROUPED) h = __hmul(h, sch);  // per-channel scale after the fp16 convert (marlin_cute_trait.h:764-769)
              if (mm < p.m) p.C[(size_t)mm * p.n + n0 + row] = h;
            }
          }
        }
      }
      if (!ok) { give_up(p, abort, 14); break; }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bars->accempty[acc]), 0));
    }
    // the TMA stores of this thread have left shared memory and reached C before the CTA ends (also after a give-up)
    if (OUT == OUT_TMA && quad == 0 && lane == 0) tma_store_wait_all();
    if (OUT == OUT_GATHER) tma_store_wait_all();   // every lane issues row copies in the gathering form
  } else if (warp == PRODUCER_WARP) {
    // =========================================================== TMA producer (one per CTA, each for its own halves)
    const int first = min(S, nsteps);
    int step = 0;
    {  // weights of the first ring-full: parameters, requested before the previous kernel of the stream is known done
      Walk walk(p, pair);
      int tile, kb, ke, i = 0;
      while (i < first && walk.next(tile, kb, ke)) {
        int n_idx2, m_idx;
        tile_nm(p, tile, n_idx2, m_idx);
        for (int kk = kb; kk < ke && i < first; ++kk, ++i) {
          if (elect_one()) issue_weights(i, n_idx2, kk);
          __syncwarp();
        }
      }
    }
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    {
      Walk walk(p, pair);
      int tile, kb, ke;
      bool ok = true;
      while (ok && walk.next(tile, kb, ke)) {
        int n_idx2, m_idx;
        tile_nm(p, tile, n_idx2, m_idx);
        const int m0 = m_idx * TM;
        for (int kk = kb; kk < ke; ++kk, ++step) {
          const int st = step % S;
          if (step >= first) {
            if (!warp_wait(smem_u32(&bars->empty[st]), ((step / S) & 1) ^ 1, abort, p.wait_ns)) { give_up(p, abort, 15); ok = false; break; }
          }
          if (elect_one()) {
            if (step >= first) issue_weights(st, n_idx2, kk);
            issue_acts(st, m0, kk);
          }
          __syncwarp();
        }
      }
    }
    if (*abort) {   // unwinding: let this CTA's own weight copies land (activation bytes are counted in the leader)
      volatile int never = 0;
      const int issued = step < S ? step : S;
      for (int i = 0; i < issued; ++i) {
        const int sidx = step - 1 - i;
        mbar_wait(smem_u32(&bars->wsfull[sidx % S]), (sidx / S) & 1, &never, 200000000ull);
      }
    }
  } else if (rank == 0) {
    // =========================================================== MMA issuer: the leader's warp, for both CTAs
    int step = 0, seg = 0;
    bool ok = true;
    long long m_afull = 0, m_wfull = 0, m_issue = 0, m_acc = 0;
    const uint32_t sA_u = smem_u32(sA);
    Walk walk(p, pair);
    int tile, kb, ke;
    for (; ok && walk.next(tile, kb, ke); ++seg) {
      int n_idx2, m_idx;
      tile_nm(p, tile, n_idx2, m_idx);
      const uint32_t idesc = make_idesc_f16_f32(2 * TILE_N, tile_width<TM>(p, m_idx * TM));   // UMMA N = the tile's own rows
      const int acc = seg & 1;
      const long long ca = W4A16_CLK();
      if (!warp_wait(smem_u32(&bars->accempty[acc]), ((seg >> 1) & 1) ^ 1, abort, p.wait_ns)) { give_up(p, abort, 16); ok = false; break; }
      m_acc += W4A16_CLK() - ca;
      const uint32_t d_tmem = tmem + acc * Cfg::ACC_STRIDE;
      for (int kk = kb; kk < ke && ok; ++kk, ++step) {
        const int st = step % S, wb = step % Cfg::WBUFS;
        const long long c0 = W4A16_CLK();
        if (!warp_wait(smem_u32(&bars->afull[st]), (step / S) & 1, abort, p.wait_ns)) { give_up(p, abort, 17); ok = false; break; }
        const long long c1 = W4A16_CLK();
        if (!warp_wait(smem_u32(&bars->wfull[wb]), (step / Cfg::WBUFS) & 1, abort, p.wait_ns)) { give_up(p, abort, 18); ok = false; break; }
        tc_fence_after();
        const long long c2 = W4A16_CLK();
        m_afull += c1 - c0;
        m_wfull += c2 - c1;
        const uint32_t a_tmem = tmem + Cfg::WBUF_COL0 + wb * Cfg::WBUF_COLS;
        const uint64_t b_desc = make_smem_desc_sw128(sA_u + st * Cfg::A_BYTES);
        if (elect_one()) {
#pragma unroll
          for (int q = 0; q < KS / 16; ++q) {
            // per CTA the 64-k chunks are HALF_ROWS*128 bytes apart; 16 k inside a swizzle row are 32 bytes apart
            const uint64_t bd = b_desc + (uint64_t)(((q >> 2) * (Cfg::HALF_ROWS * 128) + (q & 3) * 32) >> 4);
            tc_mma_ts_pair(d_tmem, a_tmem + q * 8, bd, idesc, (kk > kb || q > 0) ? 1u : 0u);
          }
          tc_commit_pair(smem_u32(&bars->wempty[wb]));
          tc_commit_pair(smem_u32(&bars->empty[st]));
        }
        __syncwarp();
        m_issue += W4A16_CLK() - c2;
      }
      if (ok && elect_one()) tc_commit_pair(smem_u32(&bars->accfull[acc]));
      __syncwarp();
    }
    W4A16_BUCKET(8, m_afull); W4A16_BUCKET(9, m_wfull); W4A16_BUCKET(10, m_issue); W4A16_BUCKET(11, m_acc); W4A16_BUCKET(3, step);
    if (!ok || *abort) {   // unwinding: no MMA may still be running when tensor memory is freed
      volatile int never = 0;
      if (elect_one()) tc_commit_pair(smem_u32(&bars->drain));
      __syncwarp();
      mbar_wait(smem_u32(&bars->drain), 0, &never, 200000000ull);
    }
  }

  // ---- teardown: both CTAs meet (every wait above is bounded), so that no arrive can target a CTA that has left
  tc_fence_before();
  cluster_sync_all();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc_pair(tmem, Cfg::TMEM_COLS);
  }
}

}  // namespace w4a16
