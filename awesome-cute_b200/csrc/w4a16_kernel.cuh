// The sm_100a W4A16 GEMM kernel:  C[m,n] (fp16) = A[m,k] (fp16) x dequant(B, s)[k,n],  fp32 accumulation.
//
// It takes the place of the reference's MarlinGemmTraits::operator()
// (gemm/marlin_gemm/marlin_cute_trait.h:306-970: cp.async ring, ldmatrix, mma.sync.m16n8k16, serial
// in-place fp16 fix-up) and reads the same operands, bit for bit.  Nothing of its structure is kept.
//
// Formulation.  The problem is run transposed, D[n, m] = sum_k W[n, k] * A[m, k], so that
//   * the 128 weight columns of a tile are the 128 rows (TMEM lanes) of a tcgen05.mma with M = 128,
//   * the batch tile (TM = 16 .. 192 rows of A) is the UMMA N dimension, read K-major straight from
//     the shared-memory tile TMA wrote (128-byte swizzle),
//   * the dequantised weights are the UMMA *A* operand and live in TENSOR MEMORY: each dequant thread
//     owns one weight column, turns its packed nibbles into fp16 pairs in registers and writes them
//     with one tcgen05.st per k-step; they never pass through shared memory as fp16.
// A packed word holds two columns (n, n+8) x four k (2t, 2t+1, 2t+8, 2t+9); the thread owning column n
// uses the word as it is and the thread owning n+8 uses word >> 8, so every nibble is converted once.
// k-pair (2t, 2t+1) lands in TMEM column t of its 16-k block and (2t+8, 2t+9) in column 4+t, which is
// natural k order, the order of the activation tile.
//
// Warp roles (one CTA per SM, persistent):
//   warps [0, 8)          dequant: smem nibbles -> registers -> TMEM operand ring; two sets of four
//                         warps (one per TMEM lane quadrant) take alternate k-stages
//   warps [8, 12)         epilogue: TMEM accumulator -> fix-up -> fp16 -> C
//   warp  12              TMA producer (warp-uniform loop, one elected lane issues)
//   warp  13              tcgen05.mma issuer (same); also owns the TMEM allocation
// Hand-offs are mbarriers; the accumulator is double buffered in TMEM so the epilogue of one tile
// overlaps the main loop of the next.
//
// Work split: stream-K.  The (tile, k-step) space is linearised tile-major, n fastest
// (marlin_cute_trait.h:278-286 uses the same order) and cut into equal contiguous ranges, one per CTA.
// A tile cut between CTAs is finished by the CTA that holds its k-step 0; the others store their fp32
// partial tile to library-owned scratch whose idle state is a sentinel bit pattern (an all-ones NaN that
// no accumulator is allowed to keep): the data is its own flag, so there is no fence and no separate flag
// round trip, and the finisher simply re-reads a slot until the sentinel is gone.  It then writes the
// sentinel back, so the scratch is in its idle state between launches (the contract the reference's lock
// array has, marlin_cute_trait.h:941-945) and a launch can be replayed from a CUDA graph.
// The finisher reaches that tile LAST in its own range while the contributors reach it FIRST in theirs,
// so in practice it never waits; contributors never wait at all (no serial chain as in
// marlin_cute_trait.h:935-950).  The finisher's wait is bounded like every other wait in the kernel.
#pragma once
#include "ptx_sm100.cuh"

namespace w4a16 {

constexpr int TILE_N = 128;                         // weight columns per tile = UMMA M
constexpr int EPI_WARPS = 4;
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;   // every device-side wait gives up after 2 s
constexpr int STATUS_TIMEOUT = 4;                   // == W4A16_ERR_TIMEOUT
constexpr uint32_t PARTIAL_IDLE = 0xffffffffu;      // idle state of a partial-tile slot (a NaN never stored as data)

// Optional phase trace (compile with -DW4A16_TRACE): [cta][16] globaltimer stamps.
#ifdef W4A16_TRACE
__device__ unsigned long long *g_trace = nullptr;
#define W4A16_STAMP(slot)                                                           \
  do {                                                                              \
    if (g_trace && lane == 0) g_trace[blockIdx.x * 16 + (slot)] = sm100::globaltimer_ns(); \
  } while (0)
// cycle buckets accumulated in registers and written once per role: [4096 + cta*16 + slot]
#define W4A16_CLK() clock64()
#define W4A16_BUCKET(slot, val)                                                        \
  do {                                                                                 \
    if (g_trace && lane == 0) g_trace[4096 + blockIdx.x * 16 + (slot)] = (unsigned long long)(val); \
  } while (0)
#else
#define W4A16_CLK() 0ll
#define W4A16_BUCKET(slot, val) \
  do {                          \
  } while (0)
#define W4A16_STAMP(slot) \
  do {                    \
  } while (0)
#endif

struct Params {
  int m, n, k;
  int n_tiles, m_tiles, k_iters;        // k_iters = k / KS
  int total_iters, iters_per_cta;
  int a_box3d;                          // 1: tmA is the 3-D view (one box per stage), 0: 2-D (one box per 64 k)
  // CTA-pair kernel only: data-parallel waves before the stream-K part.  Worker c of `workers` first runs the whole
  // tiles c, c + workers, ... below sk_tile0 = dp_waves * workers; total_iters / iters_per_cta then describe the
  // stream-K split of the tiles from sk_tile0 on.  m_fast: tile index runs over the batch tiles first.
  int dp_waves, sk_tile0, workers, m_fast;
  const __half *s;                      // scales (read directly by the epilogue when per-channel)
  __half *C;
  uint32_t *partials;                   // [gridDim.x][TM][128] fp32 partial tiles; PARTIAL_IDLE between launches
  int *status;                          // 0, or STATUS_TIMEOUT | (site << 8)
  uint64_t wait_ns;                     // every device-side wait gives up after this long (WAIT_LIMIT_NS by default)
  // gathering instantiations only: C is [m][c_ld], this GEMM's columns start at c_col0, and every finished tile also
  // goes to n_extra (0..7) further buffers of that shape, which may be peer GPUs' memory (plain stores only).  Their
  // addresses sit in a small table in device memory: with them inline, the kernel's parameters pass 512 bytes, and
  // past that size ptxas was seen to spill registers in every instantiation, the plain GEMM's included.
  int c_ld, c_col0, n_extra;
  __half *const *C_extra;
};
static_assert(sizeof(Params) <= 128, "the kernels take four tensor maps and this block: keep it small");

// How a finished tile reaches C (template parameter OUT of the kernels)
constexpr int OUT_PLAIN = 0;    // 2-byte global stores from registers, 64 contiguous bytes per warp and row
constexpr int OUT_GATHER = 1;   // staged in shared memory, written by rows to C and to the other ranks' buffers
constexpr int OUT_TMA = 2;      // staged in shared memory, one cp.async.bulk.tensor store per 16-row x 128-column chunk

// Gathering epilogue, cooperative form used by the epilogue warps.  A warp owns 32 weight columns (its TMEM lane
// quadrant), so on its own it can only write 64 contiguous bytes per output row, and peer stores of that size reach
// less than half of the NVLink rate.  The four epilogue warps therefore stage each 16-row chunk of the 128-column tile
// in shared memory and write it out by rows of 256 contiguous bytes, every destination.
// Two slabs alternate; a warp may refill slab b for chunk c+2 once it has passed gfull[(c+1)&1], because every warp
// reads chunk c before it arrives for chunk c+1.  Returns false when the (bounded) wait ran out.
constexpr int GATHER_LD = TILE_N + 8;                       // slab row pitch in fp16 (272 bytes)
constexpr int GATHER_SLAB_BYTES = 2 * 16 * GATHER_LD * 2 + 512;  // two 16-row slabs, padded to 9216
template <bool GROUPED>
__device__ __forceinline__ bool store_chunk_gather4(const Params &p, const uint32_t (&v)[16], __half sch, int mrow0, int n0,
                                                    int quad, int lane, __half *slabs, uint32_t gfull_bar, int &gcount,
                                                    volatile int *abort) {
  const int buf = gcount & 1;
  __half *sb = slabs + buf * 16 * GATHER_LD;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    __half h = __float2half(__uint_as_float(v[i]));
    if (!GROUPED) h = __hmul(h, sch);  // after the fp16 convert, as in the plain epilogue
    sb[i * GATHER_LD + quad * 32 + lane] = h;
  }
  // The rows leave through the copy engine (cp.async.bulk, shared -> global, 256 bytes each): one lane per (row,
  // destination) -- this warp's rows quad, quad + 4, quad + 8, quad + 12 times up to eight destinations -- so all of a
  // chunk's rows are in flight at once and no thread waits for a peer's acknowledgement.  (Stores from registers,
  // 8 or 16 bytes per lane, in any destination order, stayed at ~420 GB/s per GPU on eight GPUs.)
  sm100::fence_proxy_async_smem();          // this thread's slab writes, for the async proxy that will read them
  // every lane's earlier copies (previous chunk, other slab) have been read: passing this chunk's barrier frees that slab
  sm100::tma_store_wait_read();
  __syncwarp();
  if (lane == 0) sm100::mbar_arrive(gfull_bar + 8 * buf);
  const bool ok = sm100::mbar_wait(gfull_bar + 8 * buf, (gcount >> 1) & 1, abort, p.wait_ns);
  ++gcount;
  if (!__all_sync(0xffffffffu, ok)) return false;
  const int r = quad + 4 * (lane & 3), dest = lane >> 2, mm = mrow0 + r;
  if (dest <= p.n_extra && mm < p.m) {
    __half *base = dest == 0 ? p.C : p.C_extra[dest - 1];
    sm100::bulk_store(base + (size_t)mm * p.c_ld + p.c_col0 + n0, sm100::smem_u32(sb + r * GATHER_LD), TILE_N * 2);
  }
  sm100::tma_store_commit();
  return true;
}

// TMA-store epilogue (the reference stages its tile through shared memory and writes 16-byte rows,
// marlin_cute_trait.h:754-799; here the copy engine writes the rows).  The four epilogue warps stage a 16-row chunk
// of the 128-column tile as fp16 rows of 256 bytes -- the box of the tensor map over C, whose bounds clip the rows past
// m -- and one thread issues the store.  Two slabs alternate as in store_chunk_gather4; the slab of chunk c is free
// for chunk c + 2 once every warp has passed gfull[(c+1)&1], because the issuing thread arrives there only after the
// store of chunk c has finished reading shared memory.  Returns false when the (bounded) wait ran out.
template <bool GROUPED>
__device__ __forceinline__ bool store_chunk_tma(const Params &p, const CUtensorMap *tmC, const uint32_t (&v)[16], __half sch,
                                                int mrow0, int n0, int quad, int lane, __half *slabs, uint32_t gfull_bar,
                                                int &gcount, volatile int *abort) {
  const int buf = gcount & 1;
  __half *sb = slabs + buf * 16 * TILE_N;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    __half h = __float2half(__uint_as_float(v[i]));
    if (!GROUPED) h = __hmul(h, sch);  // after the fp16 convert, as in the plain epilogue
    sb[i * TILE_N + quad * 32 + lane] = h;
  }
  sm100::fence_proxy_async_smem();
  const bool issuer = (quad == 0 && lane == 0);
  if (issuer) sm100::tma_store_wait_read();
  __syncwarp();
  if (lane == 0) sm100::mbar_arrive(gfull_bar + 8 * buf);
  const bool ok = sm100::mbar_wait(gfull_bar + 8 * buf, (gcount >> 1) & 1, abort, p.wait_ns);
  ++gcount;
  if (!__all_sync(0xffffffffu, ok)) return false;
  if (issuer) {
    sm100::tma_store_2d(tmC, p.c_col0 + n0, mrow0, sm100::smem_u32(sb));
    sm100::tma_store_commit();
  }
  return true;
}

// Tile configuration.  TM = batch tile (UMMA N); KS = k per pipeline stage.  The stage is the unit of
// every hand-off; it is made large (256 k for small TM) because issuing a TMA costs the producer
// 100+ clocks whatever its size, so bytes per TMA instruction is what bounds the load rate.
template <int TM, int KS, int OUT = OUT_PLAIN>
struct Config {
  static_assert(TM == 16 || TM == 32 || TM == 64 || TM == 128 || TM == 192, "batch tile");
  static_assert(KS == 64 || KS == 128 || KS == 256, "k per stage");
  static constexpr int KCHUNKS = KS / 64;                    // 64-k swizzle atoms per stage
  static constexpr int GROUPS = KS >= 128 ? KS / 128 : 1;    // group-scale rows per stage
  static constexpr int W_BYTES = KS * TILE_N / 2;            // packed weights per stage
  static constexpr int A_BYTES = TM * KS * 2;                // activations per stage: [KCHUNKS][TM][128 B]
  static constexpr int S_BYTES = GROUPS * TILE_N * 2;        // group scales per stage
  static constexpr int STAGE_BYTES = W_BYTES + A_BYTES + S_BYTES;
  static constexpr int ACC_STRIDE = TM < 32 ? 32 : TM;       // TMEM columns between the two accumulators
  static constexpr int WBUF_COL0 = 2 * ACC_STRIDE;
  // The dequant -> MMA hand-off unit (sub-step) can be finer than the TMA stage; measured on B200 the two
  // dequant sets then collide on the same stage and decode runs ~10 % slower, so it is the whole stage.
  static constexpr int SUBK = KS;
  static constexpr int SUBS = KS / SUBK;                     // sub-steps per stage
  static constexpr int WBUF_COLS = SUBK / 2;                 // fp16 pairs per lane per sub-step
  static constexpr int TMEM_COLS = 512;
  static constexpr int WBUFS_RAW = (TMEM_COLS - WBUF_COL0) / WBUF_COLS;
  static constexpr int WBUFS = WBUFS_RAW > 8 ? 8 : WBUFS_RAW;  // TMEM operand ring depth
  static_assert(WBUFS >= 2, "TMEM budget");
  static constexpr int BAR_BYTES = 1024;
  static constexpr int GATHER_BYTES = OUT != OUT_PLAIN ? GATHER_SLAB_BYTES : 0;   // output staging of the gathering / TMA-store epilogue
  static constexpr int SMEM_MAX = 227 * 1024;
  static constexpr int STAGES_RAW = (SMEM_MAX - BAR_BYTES - GATHER_BYTES - 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 12 ? 12 : STAGES_RAW;
  static_assert(STAGES >= 3, "ring too shallow");
  // Two sets measured best on B200: a third adds eligible warps (+5 % on the largest decode shapes) but
  // costs registers (spills at TM = 128) and start-up time on small ones.
  static constexpr int NSETS = 2;                            // dequant sets taking k-stages round-robin
  static constexpr int NDQ = 4 * NSETS;                      // dequant warps: NSETS sets of four
  static constexpr int THREADS = (NDQ + EPI_WARPS + 2) * 32;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + GATHER_BYTES + 1024 /*align slack*/;
};

struct Bars {  // lives in shared memory
  uint64_t full[12];
  uint64_t empty[12];
  uint64_t wfull[8];
  uint64_t wempty[8];
  uint64_t accfull[2];
  uint64_t accempty[2];
  uint64_t drain;
  uint64_t gfull[2];     // gathering epilogue: all four epilogue warps have staged a 16-row chunk
  uint32_t tmem_base;
  int abort;
};
static_assert(sizeof(Bars) <= 1024, "barrier block");

// A wait whose verdict is the same in every lane of the warp (the tcgen05 ld/st that follow are
// warp-collective).
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int *abort, uint64_t limit_ns) {
  const bool ok = sm100::mbar_wait(bar, parity, abort, limit_ns);
  return __all_sync(0xffffffffu, ok);
}

__device__ __forceinline__ void give_up(const Params &p, volatile int *abort, int site) {
  *abort = 1;
  atomicCAS(p.status, 0, STATUS_TIMEOUT | (site << 8));
}

// Finisher of a split tile: add to v the sixteen rows at row c0 of the slices that `count` other CTAs left in the
// scratch (slots first_slot, first_slot + slot_stride, ...: ascending, so the sum is deterministic), FLY slices in
// flight together, re-reading until none shows the idle pattern, and put the idle pattern back so that the scratch is
// idle again for the next launch.  `rows` = rows per slot.  Returns false when the bounded wait ran out.
template <int FLY>
__device__ __forceinline__ bool fold_partial_slices(uint32_t (&v)[16], uint32_t *partials, int rows, int c0, int row,
                                                    int first_slot, int slot_stride, int count, volatile int *abort,
                                                    uint64_t t0, uint64_t wait_ns) {
  using namespace sm100;
  for (int j = 0; j < count; j += FLY) {
    uint32_t *src[FLY];
#pragma unroll
    for (int f = 0; f < FLY; ++f)
      src[f] = partials + ((size_t)(first_slot + min(j + f, count - 1) * slot_stride) * rows + c0) * TILE_N + row;
    uint32_t x[FLY][16];
    for (uint32_t spin = 0;; ++spin) {
#ifdef W4A16_TRACE
      if (g_trace && (threadIdx.x & 31) == 0 && (threadIdx.x >> 5) == 12) {
        g_trace[4096 + blockIdx.x * 16 + 12] = spin + 1;                                   // poll rounds
        if (spin == 1 && j == 0) g_trace[blockIdx.x * 16 + 14] = globaltimer_ns();         // first poll came back
      }
#endif
      bool up = true;
#pragma unroll
      for (int f = 0; f < FLY; ++f)
#pragma unroll
        for (int i = 0; i < 16; ++i) x[f][i] = ld_slot(src[f] + (size_t)i * TILE_N);
#pragma unroll
      for (int f = 0; f < FLY; ++f)
#pragma unroll
        for (int i = 0; i < 16; ++i) up &= (x[f][i] != PARTIAL_IDLE);
      if (__all_sync(0xffffffffu, up)) break;
      if ((spin & 0xf) == 0xf && __any_sync(0xffffffffu, *abort || globaltimer_ns() - t0 > wait_ns)) return false;
    }
#pragma unroll
    for (int f = 0; f < FLY; ++f) {
      if (j + f < count) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(x[f][i]));
          st_slot(src[f] + (size_t)i * TILE_N, PARTIAL_IDLE);   // back to idle for the next launch
        }
      }
    }
  }
  return true;
}
// The same as a real call: a kernel whose hot loops fill its register budget keeps the FLY x 16 loaded values out of
// them this way (the call happens once per split tile).
template <int FLY>
__device__ __noinline__ bool fold_partial_slices_call(uint32_t (&v)[16], uint32_t *partials, int rows, int c0, int row,
                                                      int first_slot, int slot_stride, int count, volatile int *abort,
                                                      uint64_t t0, uint64_t wait_ns) {
  return fold_partial_slices<FLY>(v, partials, rows, c0, row, first_slot, slot_stride, count, abort, t0, wait_ns);
}

// int4 -> fp16 exactly (zero point 8), two weights per instruction, as in the reference's dequant
// (marlin_cute_trait.h:8-39): OR the nibble into the mantissa of 1024.0 and subtract 1032; the high
// nibbles carry a factor 16 folded into one fma.
template <bool SCALE>
__device__ __forceinline__ void dequant_word(uint32_t w, __half2 scale, uint32_t &lo, uint32_t &hi) {
  const uint32_t l = sm100::lop3_and_or(w, 0x000f000fu, 0x64006400u);
  const uint32_t h = sm100::lop3_and_or(w, 0x00f000f0u, 0x64006400u);
  const uint32_t SUB = 0x64086408u, MUL = 0x2c002c00u, ADD = 0xd480d480u;
  __half2 a = __hsub2(*reinterpret_cast<const __half2 *>(&l), *reinterpret_cast<const __half2 *>(&SUB));
  __half2 b = __hfma2(*reinterpret_cast<const __half2 *>(&h), *reinterpret_cast<const __half2 *>(&MUL),
                      *reinterpret_cast<const __half2 *>(&ADD));
  if (SCALE) {  // group scale in fp16 before the MMA, as the reference does (marlin_cute_trait.h:656-664)
    a = __hmul2(a, scale);
    b = __hmul2(b, scale);
  }
  lo = *reinterpret_cast<uint32_t *>(&a);
  hi = *reinterpret_cast<uint32_t *>(&b);
}

template <int TM, int KS, bool GROUPED, int OUT = OUT_PLAIN>
__global__ void __launch_bounds__(Config<TM, KS>::THREADS, 1)
w4a16_tc_kernel(const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmA,
                const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmC, const Params p) {
  using Cfg = Config<TM, KS, OUT>;
  constexpr bool GATHER = OUT == OUT_GATHER;
  using namespace sm100;
  constexpr int S = Cfg::STAGES;
  constexpr int NDQ = Cfg::NDQ;
  // dequant warps help to finish a split tile (see the epilogue); not in the gathering form, whose four epilogue
  // warps write every chunk together
  constexpr bool HELP = TM >= 64 && OUT == OUT_PLAIN;
  constexpr int PRODUCER_WARP = NDQ + EPI_WARPS, MMA_WARP = NDQ + EPI_WARPS + 1;
  constexpr uint32_t STAGE_TX = Cfg::W_BYTES + Cfg::A_BYTES + (GROUPED ? Cfg::S_BYTES : 0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *sW = smem;                                   // [S][W_BYTES]   1024-aligned each
  uint8_t *sA = sW + S * Cfg::W_BYTES;                  // [S][A_BYTES]   1024-aligned each
  uint8_t *sS = sA + S * Cfg::A_BYTES;                  // [S][S_BYTES]
  Bars *bars = reinterpret_cast<Bars *>(sS + S * Cfg::S_BYTES);
  volatile int *abort = &bars->abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (warp == 0) W4A16_STAMP(0);   // kernel entry

  // ---- this CTA's slice of the linearised (tile, k-step) space
  const int it_begin = min(p.total_iters, (int)blockIdx.x * p.iters_per_cta);
  const int it_end = min(p.total_iters, it_begin + p.iters_per_cta);

  // One stage of loads.  Coordinates: weights are the 3-D view [k/16][2n/32][32 int32] (box KS/16 x 8 x 32
  // words); activations [k/64][m][64] (box KS/64 x TM x 64) or, as 2-D, one 64 x TM box per 64 k; scales
  // [k/128][n] (box GROUPS x 128).
  auto issue_weights = [&](int st, int n_idx, int kk) {   // packed weights + group scales: immutable parameters
    const uint32_t full = smem_u32(&bars->full[st]);
    mbar_expect_tx(full, STAGE_TX);
    tma_load_3d(smem_u32(sW) + st * Cfg::W_BYTES, &tmB, 0, n_idx * 8, kk * (KS / 16), full);
    if (GROUPED) tma_load_2d(smem_u32(sS) + st * Cfg::S_BYTES, &tmS, n_idx * TILE_N, (kk * KS) / 128, full);
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

  // ---- prologue.  The producer warp initialises the barriers and puts the first ring-full of loads in
  // flight BEFORE the CTA-wide sync, so HBM latency overlaps the TMEM allocation and the sync itself.
  // Under programmatic dependent launch this CTA may be running while the previous kernel of the stream is
  // still finishing: the weights and scales of the first ring-full (parameters, never a kernel's output) are
  // requested at once, everything else (activations, C, the partial-tile scratch) only after
  // pdl_wait_prior_grid().
  int pro_step = 0, pro_tile = 0, pro_kk = 0, pro_nidx = 0, pro_m0 = 0;
  if (warp == PRODUCER_WARP) {
    if (lane == 0) {
      for (int i = 0; i < S; ++i) {
        mbar_init(smem_u32(&bars->full[i]), 1);
        mbar_init(smem_u32(&bars->empty[i]), 4 * Cfg::SUBS + 1);  // 4 dequant warps per sub-step + the MMA commit
      }
      for (int i = 0; i < Cfg::WBUFS; ++i) {
        mbar_init(smem_u32(&bars->wfull[i]), 4);
        mbar_init(smem_u32(&bars->wempty[i]), 1);
      }
      for (int i = 0; i < 2; ++i) {
        mbar_init(smem_u32(&bars->accfull[i]), 1);
        mbar_init(smem_u32(&bars->accempty[i]), EPI_WARPS);
        mbar_init(smem_u32(&bars->gfull[i]), EPI_WARPS);
      }
      mbar_init(smem_u32(&bars->drain), 1);
      bars->abort = 0;
      mbar_fence_init();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    pro_tile = it_begin / p.k_iters;
    pro_kk = it_begin - pro_tile * p.k_iters;
    pro_nidx = pro_tile % p.n_tiles;
    pro_m0 = (pro_tile / p.n_tiles) * TM;
    bar_sync(1, 64);               // barriers are initialised: the MMA warp may issue the activation loads
    const int first = min(S, it_end - it_begin);
    for (; pro_step < first; ++pro_step) {
      if (elect_one()) issue_weights(pro_step, pro_nidx, pro_kk);
      __syncwarp();
      if (++pro_kk == p.k_iters) {
        pro_kk = 0;
        if (++pro_nidx == p.n_tiles) { pro_nidx = 0; pro_m0 += TM; }
      }
    }
    pdl_launch_dependents();       // the next kernel may start its own prologue as SMs free up
    pdl_wait_prior_grid();         // (the steady-state loop below issues activation loads too)
    W4A16_STAMP(9);                // first ring-full issued
  }
  if (warp == MMA_WARP) {          // the MMA warp owns TMEM
    tmem_alloc(smem_u32(&bars->tmem_base), Cfg::TMEM_COLS);
    tmem_relinquish();
    // ... and, idle until the first operand tile exists, issues the first ring-full of ACTIVATION loads next to
    // the producer's weight loads, once the previous kernel of the stream has finished
    bar_sync(1, 64);
    pdl_wait_prior_grid();
    int tile = it_begin / p.k_iters, kk = it_begin - tile * p.k_iters;
    int m0 = (tile / p.n_tiles) * TM, nidx = tile % p.n_tiles;
    const int first = min(S, it_end - it_begin);
    for (int i = 0; i < first; ++i) {
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
  if (warp == 0) W4A16_STAMP(1);   // prologue done
  const uint32_t tmem = __shfl_sync(0xffffffffu, bars->tmem_base, 0);  // provably warp-uniform

  if (warp < NDQ) {
    // =========================================================== dequant warps
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may touch
    const int set = warp >> 2;                 // the sets take k-stages round-robin
    const int row = quad * 32 + lane;          // weight column within the tile = TMEM lane
    const int nr = row & 63, blk = row >> 6;
    const int j = nr >> 4, r8 = nr & 7;
    const uint32_t shift = ((nr >> 3) & 1) ? 8u : 0u;
    // byte offset of word (r, t) inside a stage, 128-byte-swizzled as TMA wrote it:
    //   r*1024 + (4*blk + r8/2)*128 + 16*(4*((r8&1)^blk) + (t ^ (r8>>1))) + 4*j
    const uint32_t base_off = (uint32_t)((4 * blk + (r8 >> 1)) * 128 + 64 * ((r8 & 1) ^ blk) + 4 * j);
    uint32_t toff[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) toff[t] = base_off + 16u * (uint32_t)(t ^ (r8 >> 1));
    const uint32_t s_off = (uint32_t)(2 * (64 * blk + 8 * (nr & 7) + (nr >> 3)));  // group-scale slot of this column
    const uint32_t sW_u = smem_u32(sW), sS_u = smem_u32(sS);
    const uint32_t one2 = 0x3c003c00u;
    const uint32_t t_lane = tmem + ((uint32_t)(quad * 32) << 16) + Cfg::WBUF_COL0;

    long long d_full = 0, d_wempty = 0, d_work = 0;
    const int nsubs = (it_end - it_begin) * Cfg::SUBS;
    for (int g = set; g < nsubs; g += Cfg::NSETS) {      // g: this CTA's running sub-step number
      const int step = g / Cfg::SUBS, sub = g % Cfg::SUBS;
      const int st = step % S, wb = g % Cfg::WBUFS;
      const long long c0 = W4A16_CLK();
      if (!warp_wait(smem_u32(&bars->full[st]), (step / S) & 1, abort, p.wait_ns)) { give_up(p, abort, 1); break; }
      const long long c1 = W4A16_CLK();
      if (warp == 0 && g == 0) W4A16_STAMP(2);   // first stage landed
      d_full += c1 - c0;
      const uint32_t wbase = sW_u + st * Cfg::W_BYTES + sub * (Cfg::SUBK / 16) * 1024;
      __half2 sc = *reinterpret_cast<const __half2 *>(&one2);
      bool buf_ok = true;
#pragma unroll
      for (int half = 0; half < Cfg::SUBK / 64; ++half) {
        if (GROUPED && (half & 1) == 0) {   // a new 128-k group starts every second 64-k chunk
          const int grow = Cfg::SUBK >= 128 ? sub * (Cfg::SUBK / 128) + (half >> 1) : 0;
          uint16_t sv;
          asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sv) : "r"(sS_u + st * Cfg::S_BYTES + grow * (TILE_N * 2) + s_off));
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
          // the TMEM operand buffer is needed only now: the first chunk was converted while the MMA that
          // last read this buffer was still running
          const long long c2 = W4A16_CLK();
          buf_ok = warp_wait(smem_u32(&bars->wempty[wb]), ((g / Cfg::WBUFS) & 1) ^ 1, abort, p.wait_ns);
          tc_fence_after();
          d_wempty += W4A16_CLK() - c2;
          if (!buf_ok) break;
        }
        tmem_st_32x32b_x32(t_lane + wb * Cfg::WBUF_COLS + half * 32, v);
      }
      if (!buf_ok) { give_up(p, abort, 2); break; }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&bars->wfull[wb]));
        mbar_arrive(smem_u32(&bars->empty[st]));
      }
      d_work += W4A16_CLK() - c1;
      if (warp == 0 && g == 0) W4A16_STAMP(3);   // first operand tile in TMEM
    }
    if (warp == 0) {
      W4A16_STAMP(4);                               // last dequant of set 0
      W4A16_BUCKET(4, d_full); W4A16_BUCKET(5, d_wempty); W4A16_BUCKET(6, d_work);
    }
    if (HELP) {
      // ---- help to finish the CTA's last tile if it is a split one (chunks 16*(1+set), +48, ... of this quadrant)
      int seg = 0, l_tile = 0, l_kb = 1, l_ke = 0, l_seg = 0;
      for (int it = it_begin; it < it_end; ++seg) {
        l_tile = it / p.k_iters;
        l_kb = it - l_tile * p.k_iters;
        l_ke = min(p.k_iters, l_kb + (it_end - it));
        l_seg = seg;
        it += l_ke - l_kb;
      }
      if (it_end > it_begin && l_kb == 0 && l_ke < p.k_iters) {
        const int n0 = (l_tile % p.n_tiles) * TILE_N, m0 = (l_tile / p.n_tiles) * TM;
        const int acc = l_seg & 1;
        const int last_contrib = ((l_tile + 1) * p.k_iters - 1) / p.iters_per_cta;
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
#pragma unroll 1
        for (int c0 = 16 * (1 + set); c0 < TM && ok; c0 += 48) {
          uint32_t v[16];
          tmem_ld_32x32b_x16(t_acc + c0, v);
          tc_wait_ld();
          ok = fold_partial_slices<2>(v, p.partials, TM, c0, row, (int)blockIdx.x + 1, 1, last_contrib - (int)blockIdx.x, abort, t0, p.wait_ns);
          if (!ok) break;
#pragma unroll
          for (int i = 0; i < 16; ++i) {   // (never the gathering form: HELP is off there)
            const int mm = m0 + c0 + i;
            __half h = __float2half(__uint_as_float(v[i]));
            if (!GROUPED) h = __hmul(h, sch);  // per-channel scale after the fp16 convert (marlin_cute_trait.h:764-769)
            if (mm < p.m) p.C[(size_t)mm * p.n + n0 + row] = h;
          }
        }
        if (!ok) give_up(p, abort, 9);
      }
    }
  } else if (warp < NDQ + EPI_WARPS) {
    // =========================================================== epilogue warps
    // Each warp serves its own TMEM lane quadrant = 32 weight columns, end to end (its partial-tile slots
    // carry their own flags), so the four warps never have to meet.
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t t_lane = tmem + ((uint32_t)(quad * 32) << 16);
    pdl_wait_prior_grid();   // C and the partial-tile scratch may still be in use by the previous kernel
    __half *slabs = reinterpret_cast<__half *>(reinterpret_cast<uint8_t *>(bars) + Cfg::BAR_BYTES);   // gathering form only
    int gcount = 0;
    int seg = 0;
    for (int it = it_begin; it < it_end; ++seg) {
      const int tile = it / p.k_iters, kb = it - tile * p.k_iters;
      const int ke = min(p.k_iters, kb + (it_end - it));
      const int n0 = (tile % p.n_tiles) * TILE_N, m0 = (tile / p.n_tiles) * TM;
      const int acc = seg & 1;
      const bool finisher = (kb == 0);
      // the tile's other k-ranges belong to the next CTAs; they reached this tile first thing
      const int last_contrib = (finisher && ke < p.k_iters) ? ((tile + 1) * p.k_iters - 1) / p.iters_per_cta : (int)blockIdx.x;
      const int ncontrib = last_contrib - (int)blockIdx.x;
      __half sch = __float2half(1.0f);
      if (!GROUPED && finisher) {
        const int c32 = row & 31;  // per-channel scales are permuted inside 32-column blocks (marlin.py:52-54)
        sch = p.s[n0 + row - c32 + 8 * ((c32 & 7) >> 1) + 2 * (c32 >> 3) + (c32 & 1)];
      }
      if (!warp_wait(smem_u32(&bars->accfull[acc]), (seg >> 1) & 1, abort, p.wait_ns)) { give_up(p, abort, 3); break; }
      tc_fence_after();
      if (warp == NDQ) { if (seg == 0) W4A16_STAMP(5); W4A16_STAMP(6); }   // first / last accumulator ready
      uint32_t *part = p.partials + ((size_t)blockIdx.x * TM) * TILE_N + row;
      bool ok = true;
      const uint64_t t0 = ncontrib > 0 ? globaltimer_ns() : 0ull;
      constexpr int FLY = TM <= 32 ? 4 : 2;   // contributors whose slices are in flight together
      // A split tile of 64+ rows is the last thing its finisher does, and folding the contributors' slices in is a
      // chain of L2 round trips per 16 columns: the CTA's dequant warps, idle by now, take two thirds of the chunks.
      const int c_step = (HELP && finisher && ncontrib > 0) ? 48 : 16;
#pragma unroll 1
      for (int c0 = 0; c0 < TM && ok; c0 += c_step) {
        uint32_t v[16];
        tmem_ld_32x32b_x16(t_lane + acc * Cfg::ACC_STRIDE + c0, v);
        tc_wait_ld();
        if (!finisher) {
          // the data is its own flag: anything but the idle pattern means "written"
#pragma unroll
          for (int i = 0; i < 16; ++i) st_slot(part + (size_t)(c0 + i) * TILE_N, v[i] == PARTIAL_IDLE ? 0x7fffffffu : v[i]);
        } else {
          // fixed summation order (ascending contributor) keeps the result deterministic
          // (narrow tiles take four slices at a time through a real call: inlined, their 64 loaded values spilled
          // registers of the main loops)
          if (ncontrib > 0)
            ok = TM <= 32 ? fold_partial_slices_call<FLY>(v, p.partials, TM, c0, row, (int)blockIdx.x + 1, 1, ncontrib, abort, t0, p.wait_ns)
                          : fold_partial_slices<FLY>(v, p.partials, TM, c0, row, (int)blockIdx.x + 1, 1, ncontrib, abort, t0, p.wait_ns);
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
      if (!ok) { give_up(p, abort, 4); break; }
      if (warp == NDQ && ncontrib > 0) W4A16_STAMP(7);   // partial tiles folded in
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->accempty[acc]));
      it += ke - kb;
      if (warp == NDQ) W4A16_STAMP(8);     // (last value wins) epilogue of the last segment done
    }
    // the TMA stores of this thread have left shared memory and reached C before the CTA ends (also after a give-up)
    if (OUT == OUT_TMA && quad == 0 && lane == 0) tma_store_wait_all();
    if (OUT == OUT_GATHER) tma_store_wait_all();   // every lane issues row copies in the gathering form
  } else if (warp == PRODUCER_WARP) {
    // =========================================================== TMA producer (rest of the ring)
    // The whole warp runs the loop (warp-uniform operands); one elected lane issues.
    long long c_wait = 0, c_issue = 0;
    const int nsteps = it_end - it_begin;
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
    // The whole warp runs the loop (warp-uniform descriptors); one elected lane issues.
    constexpr uint32_t idesc = make_idesc_f16_f32(TILE_N, TM);
    int step = 0, seg = 0;
    bool ok = true;
    long long m_full = 0, m_wfull = 0, m_issue = 0, m_acc = 0;
    const uint32_t sA_u = smem_u32(sA);
    for (int it = it_begin; it < it_end && ok; ++seg) {
      const int tile = it / p.k_iters, kb = it - tile * p.k_iters;
      const int ke = min(p.k_iters, kb + (it_end - it));
      const int acc = seg & 1;
      const long long ca = W4A16_CLK();
      if (!warp_wait(smem_u32(&bars->accempty[acc]), ((seg >> 1) & 1) ^ 1, abort, p.wait_ns)) { give_up(p, abort, 6); ok = false; break; }
      m_acc += W4A16_CLK() - ca;
      const uint32_t d_tmem = tmem + acc * Cfg::ACC_STRIDE;
      for (int kk = kb; kk < ke && ok; ++kk, ++step) {
        const int st = step % S;
        const long long c0 = W4A16_CLK();
        if (!warp_wait(smem_u32(&bars->full[st]), (step / S) & 1, abort, p.wait_ns)) { give_up(p, abort, 7); ok = false; break; }
        m_full += W4A16_CLK() - c0;
        const uint64_t b_desc = make_smem_desc_sw128(sA_u + st * Cfg::A_BYTES);
#pragma unroll
        for (int sub = 0; sub < Cfg::SUBS; ++sub) {
          const int g = step * Cfg::SUBS + sub, wb = g % Cfg::WBUFS;
          const long long c1 = W4A16_CLK();
          if (!warp_wait(smem_u32(&bars->wfull[wb]), (g / Cfg::WBUFS) & 1, abort, p.wait_ns)) { give_up(p, abort, 8); ok = false; break; }
          tc_fence_after();
          const long long c2 = W4A16_CLK();
          m_wfull += c2 - c1;
          const uint32_t a_tmem = tmem + Cfg::WBUF_COL0 + wb * Cfg::WBUF_COLS;
          if (elect_one()) {
#pragma unroll
            for (int q = 0; q < Cfg::SUBK / 16; ++q) {
              // 64-k chunks are TM*128 bytes apart; 16 k inside a 128-byte swizzle row are 32 bytes apart
              const int qq = sub * (Cfg::SUBK / 16) + q;
              const uint64_t bd = b_desc + (uint64_t)(((qq >> 2) * (TM * 128) + (qq & 3) * 32) >> 4);
              tc_mma_ts(d_tmem, a_tmem + q * 8, bd, idesc, (kk > kb || qq > 0) ? 1u : 0u);
            }
            tc_commit(smem_u32(&bars->wempty[wb]));
            if (sub == Cfg::SUBS - 1) tc_commit(smem_u32(&bars->empty[st]));
          }
          __syncwarp();
          m_issue += W4A16_CLK() - c2;
        }
        if (step == 0) W4A16_STAMP(11);    // first MMA issued
      }
      if (ok && elect_one()) tc_commit(smem_u32(&bars->accfull[acc]));
      __syncwarp();
      it += ke - kb;
    }
    W4A16_STAMP(12);                       // last MMA issued
    W4A16_BUCKET(8, m_full); W4A16_BUCKET(9, m_wfull); W4A16_BUCKET(10, m_issue); W4A16_BUCKET(11, m_acc);
    if (!ok || *abort) {
      // unwinding: no tcgen05.mma may still be running when TMEM is freed
      volatile int never = 0;
      if (elect_one()) tc_commit(smem_u32(&bars->drain));
      __syncwarp();
      mbar_wait(smem_u32(&bars->drain), 0, &never, 200000000ull);
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
}

}  // namespace w4a16
