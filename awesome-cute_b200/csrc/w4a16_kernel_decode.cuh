// The W4A16 GEMM for skinny batches (m <= 16): the HBM-bound case, where the kernel's job is to turn packed
// nibbles into tcgen05 operands as fast as HBM delivers them.
//
// Same formulation as w4a16_kernel.cuh (D[n, m] = sum_k W[n, k] * A[m, k]; weight columns are the 128 TMEM lanes,
// dequantised weights are the UMMA A operand in tensor memory, activations the B operand in shared memory; TMA ring,
// stream-K with sentinel slots, bounded waits, dependent launch).  What differs, and why:
//
//  * One packed word is converted ONCE, by one thread.  A word holds columns (n, n + 8) x k (2t, 2t+1, 2t+8, 2t+9) of
//    the lane-`4 (n % 8) + t` fragment the reference feeds to mma.sync (marlin_cute_trait.h:8-39,644-686).  The
//    tcgen05.st shape .16x128b stores register pairs (row T/4, row T/4 + 8) x column T%4 -- the same fragment -- so
//    the thread that loaded the word writes all four fp16 pairs it holds: 16 lanes x 8 columns per 16 k, in natural k
//    order, TMEM lane = weight column.  The 32x32b shape of the general kernel makes the owner of column n and the
//    owner of n + 8 both load the word and each throw half of it away (twice the shared-memory loads).
//  * The group scale leaves the dequant warps.  (q - 8) is exact in fp16, so the MMAs accumulate EXACT integer-weight
//    products per 128-k group into a small ring of TMEM accumulators, and the epilogue warps (idle otherwise) fold
//    each group in with one fp32 fma per output: acc += s[g][n] * P_g.  That removes a third of the dequant
//    instructions (the two hmul2 per word half).  The reference rounds (q - 8) * s to fp16 before its MMA
//    (marlin_cute_trait.h:656-664, marlin_test.py:31); applying s in fp32 afterwards differs from that by the
//    fp16 rounding of the dequantised operand (relative 2^-11 per weight), far inside the 1e-2 max-norm tolerance.
//  * Three dequant sets (12 warps) instead of two: each warp is latency-bound (shared load -> ALU chain -> TMEM store),
//    three per SM sub-partition keep its issue slot busy.  One TMEM operand buffer per set.
//
//  * One MMA issuer warp behind each dequant set.  An issuer's stream is serial (wait for the operand buffer, wait
//    for a free accumulator set, sixteen tcgen05.mma, three commits) and shares its sub-partition's issue slot with
//    three dequant warps; with a single issuer that chain, not the tensor pipe, set the pace.  Issuer i owns operand
//    buffer i and accumulator set i and takes the stages of set i, so every barrier has one waiter that sees each of
//    its phases (a parity wait must not skip a phase), and since every stage has its own accumulators the order in
//    which the issuers' MMAs reach the tensor pipe does not matter.
//
// Warp roles: [0,12) dequant (set = warp / 4, TMEM lane quadrant = warp % 4), [12,16) epilogue, 16 TMA producer,
// 17..19 MMA issuers (17 owns the TMEM allocation).
#pragma once
#include "w4a16_kernel.cuh"

namespace w4a16 {

template <int OUT = OUT_PLAIN, int CL = 1>
struct DecodeConfig {
  static_assert(CL == 1 || CL == 2 || CL == 4 || CL == 8, "cluster size along k");
  static_assert(CL == 1 || OUT != OUT_GATHER, "the gathering epilogue runs on the stream-K form");
  static constexpr int TM = 16;                              // batch tile = UMMA N
  static constexpr int KS = 256;                             // k per stage
  static constexpr int KCHUNKS = KS / 64;
  static constexpr int GROUPS = KS / 128;                    // 128-k groups per stage = accumulator hand-offs per stage
  static constexpr int W_BYTES = KS * TILE_N / 2;            // 16 KB of packed weights
  static constexpr int A_BYTES = TM * KS * 2;                // [KCHUNKS][TM][128 B]
  static constexpr int S_BYTES = GROUPS * TILE_N * 2;
  static constexpr int STAGE_BYTES = W_BYTES + A_BYTES + S_BYTES;
  static constexpr int NACC = 3;                             // accumulator sets (one accumulator per group), one per MMA issuer
  static constexpr int ACC_STRIDE = GROUPS * TM;             // TMEM columns per set
  static constexpr int WBUF_COL0 = NACC * ACC_STRIDE;
  static constexpr int WBUF_COLS = KS / 2;                   // fp16 pairs per lane per stage
  static constexpr int NSETS = 3;                            // dequant sets taking k-stages round-robin
  static constexpr int WBUFS = NSETS;                        // one TMEM operand buffer per set
  static constexpr int TMEM_COLS = 512;
  static_assert(WBUF_COL0 + WBUFS * WBUF_COLS <= TMEM_COLS, "TMEM budget");
  static constexpr int NDQ = 4 * NSETS;
  static constexpr int NMMA = NSETS;                         // MMA issuer warps, one behind each dequant set
  static_assert(NACC == NMMA && WBUFS == NMMA, "issuer i owns operand buffer i and accumulator set i");
  static constexpr int THREADS = (NDQ + EPI_WARPS + 1 + NMMA) * 32;
  static constexpr int BAR_BYTES = 1024;
  // output staging: two padded slabs for the gathering epilogue, one 4 KB slab for the TMA store (a tile is one chunk)
  static constexpr int GATHER_BYTES = OUT == OUT_GATHER ? GATHER_SLAB_BYTES : OUT == OUT_TMA ? 2 * 16 * TILE_N * 2 : 0;
  // cluster form: the other ranks' fp32 partial tiles land here, in rank 0's shared memory: [CL - 1][TM][128] fp32
  static constexpr int XSLAB_BYTES = (CL - 1) * TM * TILE_N * 4;
  static constexpr int SMEM_MAX = 227 * 1024;
  static constexpr int STAGES_RAW = (SMEM_MAX - BAR_BYTES - GATHER_BYTES - XSLAB_BYTES - 1024) / STAGE_BYTES;
  // a multiple of the number of dequant sets, so that a stage is always converted by the same set; in the cluster
  // form a CTA runs few stages and six are plenty
  static constexpr int STAGES = CL > 1 ? 6 : (STAGES_RAW > 12 ? 12 : STAGES_RAW);
  static_assert(STAGES <= STAGES_RAW, "shared memory budget");
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + GATHER_BYTES + XSLAB_BYTES + 1024 /*align slack*/;
};

struct DecodeBars {  // lives in shared memory
  uint64_t full[12];
  uint64_t empty[12];
  uint64_t wfull[4];
  uint64_t wempty[4];
  uint64_t accfull[4];
  uint64_t accempty[4];
  uint64_t drain[4];     // one per MMA issuer warp
  uint64_t gfull[2];
  uint32_t tmem_base;
  int abort;
};
static_assert(sizeof(DecodeBars) <= 1024, "barrier block");

// CL > 1: the cluster form for layers with few tiles.  A cluster of CL CTAs (launched with that cluster dimension) owns
// one tile and cuts its k-range CL ways; ranks 1.. send their fp32 partial tile straight into rank 0's shared memory
// (st.shared::cluster; the data is its own flag, as in the stream-K fix-up), and rank 0 adds them in rank order and writes C.  The stream-K
// form's fix-up goes through L2 instead, and when all CTAs of a tile finish together (which they do when a tile is cut
// evenly) that costs the finisher two L2 round trips after everybody else is done; inside a cluster it is one hop.
template <bool GROUPED, int OUT = OUT_PLAIN, int CL = 1>
__global__ void __launch_bounds__(DecodeConfig<>::THREADS, 1)
w4a16_decode_kernel(const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmA,
                    const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmC, const Params p) {
  using Cfg = DecodeConfig<OUT, CL>;
  constexpr bool GATHER = OUT == OUT_GATHER;
  using namespace sm100;
  constexpr int S = Cfg::STAGES, NDQ = Cfg::NDQ, TM = Cfg::TM, KS = Cfg::KS;
  constexpr int PRODUCER_WARP = NDQ + EPI_WARPS, MMA_WARP = NDQ + EPI_WARPS + 1;   // first of NMMA issuer warps
  constexpr uint32_t STAGE_TX = Cfg::W_BYTES + Cfg::A_BYTES + (GROUPED ? Cfg::S_BYTES : 0);
  constexpr int PRE = 3;           // stages requested before the CTA-wide sync of the prologue (one per dequant set)

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *sW = smem;                                   // [S][W_BYTES]   1024-aligned each
  uint8_t *sA = sW + S * Cfg::W_BYTES;                  // [S][A_BYTES]   1024-aligned each
  uint8_t *sS = sA + S * Cfg::A_BYTES;                  // [S][S_BYTES]
  DecodeBars *bars = reinterpret_cast<DecodeBars *>(sS + S * Cfg::S_BYTES);
  volatile int *abort = &bars->abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (warp == 0) W4A16_STAMP(0);   // kernel entry

  // this CTA's slice of the linearised (tile, k-stage) space: an equal contiguous range (stream-K), or in the cluster
  // form the rank's share of the cluster's tile
  int it_begin, it_end;
  uint32_t crank = 0;
  if constexpr (CL > 1) {
    crank = cluster_ctarank();
    const int tile = (int)blockIdx.x / CL;
    it_begin = tile * p.k_iters + (p.k_iters * (int)crank) / CL;
    it_end = tile * p.k_iters + (p.k_iters * ((int)crank + 1)) / CL;
  } else {
    it_begin = min(p.total_iters, (int)blockIdx.x * p.iters_per_cta);
    it_end = min(p.total_iters, it_begin + p.iters_per_cta);
  }
  const int nsteps = it_end - it_begin;

  auto issue_weights = [&](int st, int n_idx, int kk) {   // packed weights + group scales: immutable parameters
    const uint32_t full = smem_u32(&bars->full[st]);
    mbar_expect_tx(full, STAGE_TX);
    tma_load_3d(smem_u32(sW) + st * Cfg::W_BYTES, &tmB, 0, n_idx * 8, kk * (KS / 16), full);
    if (GROUPED) tma_load_2d(smem_u32(sS) + st * Cfg::S_BYTES, &tmS, n_idx * TILE_N, kk * Cfg::GROUPS, full);
  };
  auto issue_acts = [&](int st, int m0, int kk) {         // activations: may be the previous kernel's output
    const uint32_t full = smem_u32(&bars->full[st]);
    if (p.a_box3d) {
      tma_load_3d(smem_u32(sA) + st * Cfg::A_BYTES, &tmA, 0, m0, kk * Cfg::KCHUNKS, full);
    } else {
#pragma unroll
      for (int h = 0; h < Cfg::KCHUNKS; ++h)
        tma_load_2d(smem_u32(sA) + st * Cfg::A_BYTES + h * TM * 128, &tmA, kk * KS + h * 64, m0, full);
    }
  };

  // ---- prologue.  The producer initialises the barriers and requests the first ring-full of WEIGHTS at once
  // (parameters, never a kernel's output: legal before griddepcontrol.wait); the MMA warp allocates TMEM meanwhile and
  // then requests the first ring-full of activations, once the previous kernel of the stream has completed.
  int pro_step = 0, pro_kk = 0, pro_nidx = 0, pro_m0 = 0;
  if (warp == PRODUCER_WARP) {
    // one barrier (or two) per lane, so that the first TMA can go out a few hundred clocks earlier
    if (lane < S) {
      mbar_init(smem_u32(&bars->full[lane]), 1);
      // a stage is free when its dequant set has converted it, the MMAs that read its activations have completed
      // and (group scales) the epilogue warps have taken its scales
      mbar_init(smem_u32(&bars->empty[lane]), 4 + 1 + (GROUPED ? EPI_WARPS : 0));
    } else if (lane < S + Cfg::WBUFS) {
      mbar_init(smem_u32(&bars->wfull[lane - S]), 4);
      mbar_init(smem_u32(&bars->wempty[lane - S]), 1);
    } else if (lane < S + Cfg::WBUFS + Cfg::NACC) {
      mbar_init(smem_u32(&bars->accfull[lane - S - Cfg::WBUFS]), 1);
      mbar_init(smem_u32(&bars->accempty[lane - S - Cfg::WBUFS]), EPI_WARPS);
    } else if (lane < S + Cfg::WBUFS + Cfg::NACC + 2) {
      mbar_init(smem_u32(&bars->gfull[lane - S - Cfg::WBUFS - Cfg::NACC]), EPI_WARPS);
    } else if (lane == 31) {
      for (int i = 0; i < Cfg::NMMA; ++i) mbar_init(smem_u32(&bars->drain[i]), 1);
      bars->abort = 0;
      tma_prefetch_desc(&tmB);
      tma_prefetch_desc(&tmS);
    }
    static_assert(S + Cfg::WBUFS + Cfg::NACC + 2 < 32, "one lane per barrier group");
    mbar_fence_init();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    const int pro_tile = it_begin / p.k_iters;
    pro_kk = it_begin - pro_tile * p.k_iters;
    pro_nidx = pro_tile % p.n_tiles;
    pro_m0 = (pro_tile / p.n_tiles) * TM;
    bar_arrive(1, 64);             // barriers exist: the MMA warp may issue the activation loads (it waits, we do not)
    // Only the first PRE stages before the CTA-wide sync: issuing a TMA costs ~100 clocks, a whole ring-full would
    // hold the dequant warps at the sync for a microsecond, past the time the first stage lands.
    const int pre = min(PRE, nsteps);
    for (; pro_step < pre; ++pro_step) {
      if (elect_one()) issue_weights(pro_step, pro_nidx, pro_kk);
      __syncwarp();
      if (++pro_kk == p.k_iters) {
        pro_kk = 0;
        if (++pro_nidx == p.n_tiles) { pro_nidx = 0; pro_m0 += TM; }
      }
    }
  }
  if (warp == MMA_WARP) {          // the first MMA warp owns TMEM
    if (lane == 0) { tma_prefetch_desc(&tmA); }
    tmem_alloc(smem_u32(&bars->tmem_base), Cfg::TMEM_COLS);
    tmem_relinquish();
    bar_sync(1, 64);
    pdl_wait_prior_grid();
    int tile = it_begin / p.k_iters, kk = it_begin - tile * p.k_iters;
    int m0 = (tile / p.n_tiles) * TM, nidx = tile % p.n_tiles;
    const int pre = min(PRE, nsteps);
    for (int i = 0; i < pre; ++i) {   // the activations of the stages whose weights the producer has requested
      if (elect_one()) issue_acts(i, m0, kk);
      __syncwarp();
      if (++kk == p.k_iters) {
        kk = 0;
        if (++nidx == p.n_tiles) { nidx = 0; m0 += TM; }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // Cluster form: rank 0's slab must hold the idle pattern before another rank writes into it.  Every thread arrives
  // at the cluster barrier here and waits for it only where it needs the guarantee (the epilogue threads of ranks 1..
  // right before they send, everybody else at the end): waiting here held every warp for about a microsecond.
  bool cluster_waited = false;
  if (warp == 0) W4A16_STAMP(15);  // CTA-wide sync passed
  if constexpr (CL > 1) {
    if (crank == 0 && warp >= NDQ && warp < NDQ + EPI_WARPS) {
      // rank 0's epilogue warps, idle for the next microseconds, put the idle pattern into the slab; their arrive
      // releases it at cluster scope (that release is what costs ~1500 clocks: nobody else pays it)
      uint32_t *cell = reinterpret_cast<uint32_t *>(reinterpret_cast<uint8_t *>(bars) + Cfg::BAR_BYTES + Cfg::GATHER_BYTES) + (warp - NDQ) * 32 + lane;
#pragma unroll 4
      for (int i = 0; i < (CL - 1) * TM; ++i) cell[(size_t)i * TILE_N] = PARTIAL_IDLE;
      cluster_arrive();
    } else {
      cluster_arrive_relaxed();
    }
  }
  if (warp == 0) W4A16_STAMP(1);   // prologue done
  const uint32_t tmem = __shfl_sync(0xffffffffu, bars->tmem_base, 0);  // provably warp-uniform

  if (warp < NDQ) {
    // =========================================================== dequant warps
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may touch: weight columns [32 quad, +32)
    const int set = warp >> 2;                 // the sets take k-stages round-robin; set s owns operand buffer s
    const int blk = quad >> 1;                 // 64-column block of the packed layout
    // This lane is fragment lane `lane` of that block.  Its 16-byte chunk of a 16-k row holds the four words j = 0..3
    // (columns 16 j + lane/4 and + 8); this warp's quadrant covers j = 2 (quad & 1) and the next one: 8 bytes.
    // Byte offset inside a stage, 128-byte-swizzled as TMA wrote it: row r is 1024 bytes, the block's 512 bytes are
    // lines 4 blk .. 4 blk + 3 of 128 bytes, chunk (lane % 8) of line l sits at chunk (lane % 8) ^ (l % 8).
    const int line = 4 * blk + (lane >> 3);
    const uint32_t off = (uint32_t)(line * 128 + 16 * ((lane & 7) ^ line) + 8 * (quad & 1));
    const uint32_t sW_u = smem_u32(sW);
    const uint32_t t_dst = tmem + ((uint32_t)(quad * 32) << 16) + Cfg::WBUF_COL0 + set * Cfg::WBUF_COLS;
    const uint32_t wfull_bar = smem_u32(&bars->wfull[set]), wempty_bar = smem_u32(&bars->wempty[set]);

    long long d_full = 0, d_wempty = 0, d_work = 0;
    for (int g = set, use = 0; g < nsteps; g += Cfg::NSETS, ++use) {   // g: this CTA's running stage number
      const int st = g % S;
      const long long c0 = W4A16_CLK();
      if (!warp_wait(smem_u32(&bars->full[st]), (g / S) & 1, abort, p.wait_ns)) { give_up(p, abort, 1); break; }
      const long long c1 = W4A16_CLK();
      if (warp == 0 && g == 0) W4A16_STAMP(2);   // first stage landed
      d_full += c1 - c0;
      const uint32_t wbase = sW_u + st * Cfg::W_BYTES + off;
      bool buf_ok = true;
#pragma unroll
      for (int h = 0; h < 2; ++h) {              // 128-k halves of the stage
        uint32_t wx[8], wy[8];
#pragma unroll
        for (int rr = 0; rr < 8; ++rr)
          asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(wx[rr]), "=r"(wy[rr]) : "r"(wbase + (h * 8 + rr) * 1024));
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {         // the two 16-column groups of this quadrant
          uint32_t v[32];
          const __half2 unused = __half2();
#pragma unroll
          for (int rr = 0; rr < 8; ++rr) {
            const uint32_t w = jj ? wy[rr] : wx[rr];
            // registers (4 rr, +1, +2, +3) = (column n, k-pair t), (n + 8, t), (n, t + 4), (n + 8, t + 4) of 16-k row rr
            dequant_word<false>(w, unused, v[4 * rr], v[4 * rr + 2]);
            dequant_word<false>(w >> 8, unused, v[4 * rr + 1], v[4 * rr + 3]);
          }
          if (h == 0 && jj == 0) {
            // the operand buffer is needed only now: the first words were converted while the MMAs that last read
            // it were still running
            const long long c2 = W4A16_CLK();
            buf_ok = warp_wait(wempty_bar, (use & 1) ^ 1, abort, p.wait_ns);
            tc_fence_after();
            d_wempty += W4A16_CLK() - c2;
            if (!buf_ok) break;
          }
          tmem_st_16x128b_x16(t_dst + ((uint32_t)(16 * jj) << 16) + h * 64, v);
        }
        if (!buf_ok) break;
      }
      if (!buf_ok) { give_up(p, abort, 2); break; }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(wfull_bar);
        mbar_arrive(smem_u32(&bars->empty[st]));
      }
      d_work += W4A16_CLK() - c1;
      if (warp == 0 && g == 0) W4A16_STAMP(3);   // first operand tile in TMEM
    }
    if (warp == 0) {
      W4A16_STAMP(4);                               // last dequant of set 0
      W4A16_BUCKET(4, d_full); W4A16_BUCKET(5, d_wempty); W4A16_BUCKET(6, d_work);
    }
  } else if (warp < NDQ + EPI_WARPS) {
    // =========================================================== epilogue warps
    // Each warp serves its own TMEM lane quadrant = 32 weight columns, end to end: it folds every 128-k group's
    // accumulator into fp32 registers (times the group scale), and at the end of a tile's k-range stores a partial
    // slice or, as the tile's finisher, adds the other CTAs' slices and writes C.
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int nr = row & 63;
    const uint32_t s_off = (uint32_t)(2 * (64 * (row >> 6) + 8 * (nr & 7) + (nr >> 3)));  // this column's group-scale slot
    const uint32_t t_lane = tmem + ((uint32_t)(quad * 32) << 16);
    const uint32_t sS_u = smem_u32(sS);
    pdl_wait_prior_grid();   // C and the partial-tile scratch may still be in use by the previous kernel
    __half *slabs = reinterpret_cast<__half *>(reinterpret_cast<uint8_t *>(bars) + Cfg::BAR_BYTES);   // gathering form only
    float *xslab = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(bars) + Cfg::BAR_BYTES + Cfg::GATHER_BYTES);   // cluster form only
    int gcount = 0;
    int step = 0;
    bool ok = true;
    for (int it = it_begin; it < it_end && ok;) {
      const int tile = it / p.k_iters, kb = it - tile * p.k_iters;
      const int ke = min(p.k_iters, kb + (it_end - it));
      const int n0 = (tile % p.n_tiles) * TILE_N, m0 = (tile / p.n_tiles) * TM;
      const bool finisher = (kb == 0);
      // the tile's other k-ranges belong to the next CTAs; they reached this tile first thing
      const int last_contrib = (finisher && ke < p.k_iters) ? ((tile + 1) * p.k_iters - 1) / p.iters_per_cta : (int)blockIdx.x;
      const int ncontrib = last_contrib - (int)blockIdx.x;
      __half sch = __float2half(1.0f);
      if (!GROUPED && finisher) {
        const int c32 = row & 31;  // per-channel scales are permuted inside 32-column blocks (marlin.py:52-54)
        sch = p.s[n0 + row - c32 + 8 * ((c32 & 7) >> 1) + 2 * (c32 >> 3) + (c32 & 1)];
      }
      float f[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) f[i] = 0.f;
      for (int kk = kb; kk < ke && ok; ++kk, ++step) {
        const int st = step % S, a = step % Cfg::NACC;
        float sc[2] = {1.f, 1.f};
        if (GROUPED) {
          // the scales of this stage's two groups, as TMA wrote them
          if (!warp_wait(smem_u32(&bars->full[st]), (step / S) & 1, abort, p.wait_ns)) { give_up(p, abort, 10); ok = false; break; }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint16_t sv;
            asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sv) : "r"(sS_u + st * Cfg::S_BYTES + h * (TILE_N * 2) + s_off));
            sc[h] = __half2float(__ushort_as_half(sv));
          }
        }
        if (!warp_wait(smem_u32(&bars->accfull[a]), (step / Cfg::NACC) & 1, abort, p.wait_ns)) { give_up(p, abort, 3); ok = false; break; }
        tc_fence_after();
        uint32_t v0[16], v1[16];
        tmem_ld_32x32b_x16(t_lane + a * Cfg::ACC_STRIDE, v0);
        tmem_ld_32x32b_x16(t_lane + a * Cfg::ACC_STRIDE + TM, v1);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(smem_u32(&bars->accempty[a]));
          if (GROUPED) mbar_arrive(smem_u32(&bars->empty[st]));   // scales taken: the stage may be reused
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          if (GROUPED) {
            f[i] = fmaf(sc[0], __uint_as_float(v0[i]), f[i]);
            f[i] = fmaf(sc[1], __uint_as_float(v1[i]), f[i]);
          } else {
            f[i] += __uint_as_float(v0[i]) + __uint_as_float(v1[i]);
          }
        }
        if (warp == NDQ && step == 0) W4A16_STAMP(5);   // first accumulator folded
      }
      if (!ok) break;
      if (warp == NDQ) W4A16_STAMP(6);                 // (last value wins) last accumulator folded
      uint32_t v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(f[i]);
      if (CL > 1 && !finisher) {
        // cluster form, ranks 1..: the partial tile goes into rank 0's slab [rank - 1][16][128], one hop over the
        // cluster's shared-memory network.  As in the stream-K form the data is its own flag (a cell is written when
        // it no longer holds the idle pattern): a release at cluster scope would cost the sender ~1500 clocks.
        // (Slab rows are 128 consecutive columns, so a warp's 4-byte stores are one 128-byte packet; a column-major
        // slab written with 16-byte stores per thread was measured 4-7 % slower on every cluster shape.)
        const uint32_t dst = map_to_cta(smem_u32(xslab + ((size_t)(crank - 1) * TM) * TILE_N + row), 0);
        if (!cluster_waited) { cluster_wait(); cluster_waited = true; }
#pragma unroll
        for (int i = 0; i < 16; ++i) st_shared_cluster_u32(dst + (uint32_t)i * TILE_N * 4, v[i] == PARTIAL_IDLE ? 0x7fffffffu : v[i]);
      } else if (!finisher) {
        // the data is its own flag: anything but the idle pattern means "written"
        uint32_t *part = p.partials + ((size_t)blockIdx.x * TM) * TILE_N + row;
#pragma unroll
        for (int i = 0; i < 16; ++i) st_slot(part + (size_t)i * TILE_N, v[i] == PARTIAL_IDLE ? 0x7fffffffu : v[i]);
      } else {
        if constexpr (CL > 1) {
          // rank 0: re-read its own slab until no cell shows the idle pattern, then add in rank order
          const uint32_t cell0 = smem_u32(xslab) + (uint32_t)row * 4;
          const uint64_t t0 = globaltimer_ns();
          for (uint32_t spin = 0;; ++spin) {
            bool up = true;
#pragma unroll 1
            for (int r = 0; r < CL - 1; ++r)
#pragma unroll
              for (int i = 0; i < TM; ++i) up &= (ld_shared_relaxed_cluster(cell0 + (uint32_t)((r * TM + i) * TILE_N * 4)) != PARTIAL_IDLE);
            if (__all_sync(0xffffffffu, up)) break;
            if ((spin & 0x3f) == 0x3f && __any_sync(0xffffffffu, *abort || globaltimer_ns() - t0 > p.wait_ns)) { ok = false; break; }
          }
          if (!ok) { give_up(p, abort, 4); break; }
#pragma unroll 1
          for (int r = 0; r < CL - 1; ++r)
#pragma unroll
            for (int i = 0; i < 16; ++i) f[i] += __uint_as_float(ld_shared_relaxed_cluster(cell0 + (uint32_t)((r * TM + i) * TILE_N * 4)));
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(f[i]);
          if (warp == NDQ) W4A16_STAMP(7);             // partial tiles folded in
        } else if (ncontrib > 0) {
          const uint64_t t0 = globaltimer_ns();
          if (!fold_partial_slices_call<3>(v, p.partials, TM, 0, row, (int)blockIdx.x + 1, 1, ncontrib, abort, t0, p.wait_ns)) {
            give_up(p, abort, 4);
            ok = false;
            break;
          }
          if (warp == NDQ) W4A16_STAMP(7);             // partial tiles folded in
        }
        if constexpr (GATHER) {
          if (!store_chunk_gather4<GROUPED>(p, v, sch, m0, n0, quad, lane, slabs, smem_u32(&bars->gfull[0]), gcount, abort)) {
            give_up(p, abort, 4);
            ok = false;
            break;
          }
        } else if constexpr (OUT == OUT_TMA) {
          if (!store_chunk_tma<GROUPED>(p, &tmC, v, sch, m0, n0, quad, lane, slabs, smem_u32(&bars->gfull[0]), gcount, abort)) {
            give_up(p, abort, 4);
            ok = false;
            break;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int mm = m0 + i;
            __half hv = __float2half(__uint_as_float(v[i]));
            if (!GROUPED) hv = __hmul(hv, sch);  // per-channel scale after the fp16 convert (marlin_cute_trait.h:764-769)
            if (mm < p.m) p.C[(size_t)mm * p.n + n0 + row] = hv;
          }
        }
      }
      it += ke - kb;
      if (warp == NDQ) W4A16_STAMP(8);     // (last value wins) epilogue of the last segment done
    }
    // the TMA stores of this thread have left shared memory and reached C before the CTA ends (also after a give-up)
    if (OUT == OUT_TMA && quad == 0 && lane == 0) tma_store_wait_all();
    if (OUT == OUT_GATHER) tma_store_wait_all();   // every lane issues row copies in the gathering form
  } else if (warp == PRODUCER_WARP) {
    // =========================================================== TMA producer (rest of the ring)
    long long c_wait = 0, c_issue = 0;
    {
      // the rest of the first ring-full: weights and scales at once (parameters, never a kernel's output: legal before
      // griddepcontrol.wait), their activations once the previous kernel of the stream has completed
      const int first = min(S, nsteps), from = pro_step;
      const int kk0 = pro_kk, nidx0 = pro_nidx, m00 = pro_m0;
      for (; pro_step < first; ++pro_step) {
        if (elect_one()) issue_weights(pro_step, pro_nidx, pro_kk);
        __syncwarp();
        if (++pro_kk == p.k_iters) {
          pro_kk = 0;
          if (++pro_nidx == p.n_tiles) { pro_nidx = 0; pro_m0 += TM; }
        }
      }
      pdl_launch_dependents();       // the next kernel may start its own prologue as SMs free up
      pdl_wait_prior_grid();
      int kk = kk0, nidx = nidx0, m0 = m00;
      for (int i = from; i < first; ++i) {
        if (elect_one()) issue_acts(i, m0, kk);
        __syncwarp();
        if (++kk == p.k_iters) {
          kk = 0;
          if (++nidx == p.n_tiles) { nidx = 0; m0 += TM; }
        }
      }
      W4A16_STAMP(9);                // first ring-full issued
    }
    for (; pro_step < nsteps; ++pro_step) {
      const int st = pro_step % S;
      const long long c0 = W4A16_CLK();
      if (!warp_wait(smem_u32(&bars->empty[st]), ((pro_step / S) & 1) ^ 1, abort, p.wait_ns)) { give_up(p, abort, 5); break; }
      const long long c1 = W4A16_CLK();
      c_wait += c1 - c0;
      if (elect_one()) {
        issue_weights(st, pro_nidx, pro_kk);
        issue_acts(st, pro_m0, pro_kk);
      }
      __syncwarp();
      if (++pro_kk == p.k_iters) {
        pro_kk = 0;
        if (++pro_nidx == p.n_tiles) { pro_nidx = 0; pro_m0 += TM; }
      }
      c_issue += W4A16_CLK() - c1;
    }
    W4A16_STAMP(10);                       // last TMA issued
    W4A16_BUCKET(0, c_wait); W4A16_BUCKET(1, c_issue); W4A16_BUCKET(3, nsteps);
    if (*abort) {
      // unwinding: let the copies already issued land before the CTA gives its shared memory back
      volatile int never = 0;
      const int issued = pro_step < S ? pro_step : S;
      for (int i = 0; i < issued; ++i) {
        const int sidx = pro_step - 1 - i;
        mbar_wait(smem_u32(&bars->full[sidx % S]), (sidx / S) & 1, &never, 200000000ull);
      }
    }
  } else {
    // =========================================================== MMA issuer
    // Per stage: two groups of 8 MMAs (K = 16 each), each group into a fresh accumulator of the ring.
    constexpr uint32_t idesc = make_idesc_f16_f32(TILE_N, TM);
    bool ok = true;
    long long m_full = 0, m_wfull = 0, m_issue = 0, m_acc = 0;
    const uint32_t sA_u = smem_u32(sA);
    for (int step = warp - MMA_WARP; step < nsteps && ok; step += Cfg::NMMA) {
      const int st = step % S, wb = step % Cfg::WBUFS, a = step % Cfg::NACC;
      const long long c1 = W4A16_CLK();
      // The operand buffer is complete.  Its dequant warps waited for full[st] before they read the stage, so the
      // activations of the stage have landed too (the barrier counts weights, scales and activations together).
      if (!warp_wait(smem_u32(&bars->wfull[wb]), (step / Cfg::WBUFS) & 1, abort, p.wait_ns)) { give_up(p, abort, 8); ok = false; break; }
      const long long c2 = W4A16_CLK();
      m_wfull += c2 - c1;
      if (!warp_wait(smem_u32(&bars->accempty[a]), ((step / Cfg::NACC) & 1) ^ 1, abort, p.wait_ns)) { give_up(p, abort, 6); ok = false; break; }
      tc_fence_after();
      const long long c3 = W4A16_CLK();
      m_acc += c3 - c2;
      const uint64_t b_desc = make_smem_desc_sw128(sA_u + st * Cfg::A_BYTES);
      const uint32_t a_tmem = tmem + Cfg::WBUF_COL0 + wb * Cfg::WBUF_COLS;
      const uint32_t d_tmem = tmem + a * Cfg::ACC_STRIDE;
      if (elect_one()) {
#pragma unroll
        for (int qq = 0; qq < 16; ++qq) {
          // group qq / 8 has its own accumulator; 64-k chunks are TM*128 bytes apart, 16 k inside a 128-byte
          // swizzle row are 32 bytes apart
          const uint64_t bd = b_desc + (uint64_t)(((qq >> 2) * (TM * 128) + (qq & 3) * 32) >> 4);
          if ((qq & 7) == 0)
            tc_mma_ts_imm<0>(d_tmem + (qq >> 3) * TM, a_tmem + qq * 8, bd, idesc);
          else
            tc_mma_ts_imm<1>(d_tmem + (qq >> 3) * TM, a_tmem + qq * 8, bd, idesc);
        }
        tc_commit(smem_u32(&bars->accfull[a]));
        tc_commit(smem_u32(&bars->wempty[wb]));
        tc_commit(smem_u32(&bars->empty[st]));
      }
      __syncwarp();
      m_issue += W4A16_CLK() - c3;
      if (step == 0) W4A16_STAMP(11);    // first MMA issued
    }
    if (warp == MMA_WARP) {
      W4A16_STAMP(12);                     // last MMA issued
      W4A16_BUCKET(8, m_full); W4A16_BUCKET(9, m_wfull); W4A16_BUCKET(10, m_issue); W4A16_BUCKET(11, m_acc);
    }
    if (!ok || *abort) {
      // unwinding: no tcgen05.mma may still be running when TMEM is freed
      volatile int never = 0;
      if (elect_one()) tc_commit(smem_u32(&bars->drain[warp - MMA_WARP]));
      __syncwarp();
      mbar_wait(smem_u32(&bars->drain[warp - MMA_WARP]), 0, &never, 200000000ull);
    }
  }

  // ---- teardown: everyone meets here, also after an abort (every wait above is bounded)
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
    W4A16_STAMP(13);                       // TMEM freed
  }
  // cluster form: rank 0's shared memory must outlive every store the other ranks may still send into it (they send
  // only on the regular path, microseconds before this point; after a time-out nobody sends)
  if constexpr (CL > 1) {
    if (!cluster_waited) cluster_wait();
    cluster_sync_all();
  }
}

}  // namespace w4a16
