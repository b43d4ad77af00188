// Host launcher + C ABI of the sm_100a W4A16 GEMM (declarations: include/w4a16.h, include/marlin_cute.h).
//
// Takes the place of the reference's launcher marlin_cute (gemm/marlin_gemm/marlin_cute_kernel.cu:28-115):
// same arguments, same shape checks and return codes, but ONE launch for any m (the reference loops
// over 64-row chunks and re-streams the weights per chunk, :71-111), tensor maps instead of raw pointer
// arithmetic, and per-(device, stream) cached state instead of per-call attribute queries (:18,35,38).
// There is no CPU path and no fallback: if the device is not sm_100 the launch fails with a CUDA error.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <array>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <tuple>
#include <utility>
#include <vector>

#include "../../include/marlin_cute.h"
#include "../../include/w4a16.h"
#include "w4a16_kernel.cuh"
#include "w4a16_kernel_2sm.cuh"
#include "w4a16_kernel_decode.cuh"

namespace {

thread_local std::string g_last_error;

// W4A16_PDL=0 in the environment turns programmatic dependent launch off (debugging aid)
const bool g_use_pdl = [] {
  const char *e = std::getenv("W4A16_PDL");
  return !(e && e[0] == '0');
}();

// W4A16_WAIT_MS in the environment shortens (or lengthens, up to 5000) the limit of every device-side wait (debugging aid)
const uint64_t g_wait_ns = [] {
  const char *e = std::getenv("W4A16_WAIT_MS");
  const long v = e ? std::atol(e) : 0;
  return (v >= 1 && v <= 5000) ? (uint64_t)v * 1000000ull : w4a16::WAIT_LIMIT_NS;
}();

bool cuda_ok(cudaError_t e, const char *what) {
  if (e == cudaSuccess) return true;
  g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
  return false;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, fetched through the runtime so the library needs no link against libcuda.
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void *f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

bool encode(CUtensorMap *map, CUtensorMapDataType dt, int rank, const void *base, const cuuint64_t *dims,
            const cuuint64_t *strides_bytes, const cuuint32_t *box, CUtensorMapSwizzle swz, const char *what) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) {
    g_last_error = "cuTensorMapEncodeTiled entry point not available";
    return false;
  }
  const cuuint32_t ones[3] = {1, 1, 1};
  CUresult r = fn(map, dt, (cuuint32_t)rank, const_cast<void *>(base), dims, strides_bytes, box, ones,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_error = std::string("cuTensorMapEncodeTiled(") + what + ") failed with CUresult " + std::to_string((int)r);
    return false;
  }
  return true;
}

// Per (device, stream) state: scratch of the stream-K fix-up, the status word.
struct StreamCtx {
  uint32_t *partials = nullptr;  // fp32 partial-tile slots, all PARTIAL_IDLE (0xff bytes) between launches
  size_t partial_slots = 0;
  int *status = nullptr;
  // Earlier, smaller scratch blocks.  They stay allocated (idle pattern intact) until w4a16_release_stream: a launch
  // captured in a CUDA graph keeps pointing at the block it was captured with.
  std::vector<std::pair<uint32_t *, size_t>> retired;
};
constexpr int MAX_GRID = 256;

std::mutex g_mu;
std::map<std::pair<int, cudaStream_t>, StreamCtx> g_ctx;
int g_sm_count[64] = {0};

int sm_count(int dev) {
  if (dev < 0 || dev >= 64) return -1;
  if (g_sm_count[dev] == 0) {
    int v = 0;
    if (!cuda_ok(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev), "cudaDeviceGetAttribute")) return -1;
    g_sm_count[dev] = v;
  }
  return g_sm_count[dev];
}

int g_l2_bytes[64] = {0};

int l2_bytes(int dev) {
  if (dev < 0 || dev >= 64) return -1;
  if (g_l2_bytes[dev] == 0) {
    int v = 0;
    if (!cuda_ok(cudaDeviceGetAttribute(&v, cudaDevAttrL2CacheSize, dev), "cudaDeviceGetAttribute")) return -1;
    g_l2_bytes[dev] = v > 0 ? v : 1;
  }
  return g_l2_bytes[dev];
}

// Must be called with g_mu held.  The scratch is sized by need: the first block covers every launch of up to 64 batch
// rows on this device (one slot row per CTA row: SMs x 64 x 128 fp32, 4.8 MB on a 148-SM part), larger batch tiles
// grow it (SMs x 192 x 128 fp32 = 14.5 MB at most).  Growing allocates, which CUDA refuses while a stream is being
// captured: run a problem of the size once before capturing it.
StreamCtx *get_ctx(int dev, cudaStream_t stream, size_t need_slots) {
  StreamCtx &c = g_ctx[{dev, stream}];
  if (!c.status) {
    if (!cuda_ok(cudaMalloc(&c.status, sizeof(int)), "cudaMalloc(status)")) return nullptr;
    if (!cuda_ok(cudaMemset(c.status, 0, sizeof(int)), "cudaMemset(status)")) return nullptr;
  }
  if (c.partial_slots < need_slots) {
    const int nsm = sm_count(dev);
    const size_t floor_slots = (size_t)(nsm > 0 ? nsm : MAX_GRID) * 64 * w4a16::TILE_N;
    const size_t slots = std::max(need_slots, floor_slots);
    uint32_t *blk = nullptr;
    if (!cuda_ok(cudaMalloc(&blk, sizeof(uint32_t) * slots), "cudaMalloc(partials)")) return nullptr;
    if (!cuda_ok(cudaMemset(blk, 0xff, sizeof(uint32_t) * slots), "cudaMemset(partials)")) {
      cudaFree(blk);
      return nullptr;
    }
    if (c.partials) c.retired.emplace_back(c.partials, c.partial_slots);
    c.partials = blk;
    c.partial_slots = slots;
  }
  return &c;
}

struct Problem {
  const void *A, *B, *s;
  void *C;
  int m, n, k, groupsize, dev, sms;
  cudaStream_t stream;
  // set only by the allocation-free entry point: caller-independent scratch that already exists
  uint32_t *fixed_partials = nullptr;
  int *fixed_status = nullptr;
  size_t fixed_slots = 0;
  // set only by the bounded-wait self-test: launch CTA 0 alone, so that it waits for partial tiles nobody writes
  bool orphan_finisher = false;
  uint64_t wait_ns = g_wait_ns;
  // set only by the gathering entry point: C is [m][c_ld], this GEMM's columns start at c_col0, and every finished
  // tile also goes to the same place of n_extra further buffers
  int c_ld = 0, c_col0 = 0, n_extra = 0;
  void *const *C_extra = nullptr;   // device table of the n_extra further buffers
  // set only by w4a16_plan: describe the launch instead of making it (no CUDA call on that path)
  w4a16_plan_t *plan = nullptr;
  int plan_sms = 0;                 // SMs of the device the plan is for
};

// SMs of the problem's device: asked of CUDA, or given by the caller of w4a16_plan
int problem_sm_count(const Problem &pr);

int problem_sm_count(const Problem &pr) { return pr.plan ? pr.plan_sms : sm_count(pr.dev); }

void set_output(w4a16::Params &p, const Problem &pr) {
  p.C = static_cast<__half *>(pr.C);
  p.c_ld = pr.c_ld > 0 ? pr.c_ld : pr.n;
  p.c_col0 = pr.c_col0;
  p.n_extra = pr.n_extra;
  p.C_extra = reinterpret_cast<__half *const *>(pr.C_extra);
}

// ---- tensor maps.  They depend only on the operands' addresses, the shape and the kernel's box sizes, and encoding
// them is most of a launch's host time, so they are kept: key (B, A, s, m, n, k, k per stage, activation rows per box).
struct Maps {
  CUtensorMap b, a, s, c;
  int a_box3d;
};
struct MapKey {
  const void *B, *A, *s, *C;   // C only for the TMA-store epilogue (else null: the maps do not depend on it)
  int m, n, k, ks, a_rows, grouped;
  bool operator<(const MapKey &o) const {
    return std::tie(B, A, s, C, m, n, k, ks, a_rows, grouped) < std::tie(o.B, o.A, o.s, o.C, o.m, o.n, o.k, o.ks, o.a_rows, o.grouped);
  }
};
std::map<MapKey, Maps> g_maps;   // guarded by g_mu

bool build_maps(const Problem &pr, int ks, int a_rows, bool grouped, bool tma_store, Maps &mp) {
  {  // weights: int32 [k/16][2n] viewed as [k/16][2n/32][32] so a 128-byte inner box can be swizzled
    const cuuint64_t dims[3] = {32, (cuuint64_t)(2 * pr.n / 32), (cuuint64_t)(pr.k / 16)};
    const cuuint64_t strides[2] = {128, (cuuint64_t)pr.n * 8};
    const cuuint32_t box[3] = {32, 8, (cuuint32_t)(ks / 16)};
    if (!encode(&mp.b, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, pr.B, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "B"))
      return false;
  }
  {  // activations: fp16 [m][k]; rows past m read as zero.  Preferred: the 3-D view [k/64][m][64] so that one
     // box brings a whole stage as ks/64 swizzle atoms; if the driver refuses that stride order, 2-D boxes.
    const cuuint64_t dims3[3] = {64, (cuuint64_t)pr.m, (cuuint64_t)(pr.k / 64)};
    const cuuint64_t strides3[2] = {(cuuint64_t)pr.k * 2, 128};
    const cuuint32_t box3[3] = {64, (cuuint32_t)a_rows, (cuuint32_t)(ks / 64)};
    mp.a_box3d = 1;
    if (ks == 64 ||
        !encode(&mp.a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, pr.A, dims3, strides3, box3, CU_TENSOR_MAP_SWIZZLE_128B, "A3")) {
      const cuuint64_t dims[2] = {(cuuint64_t)pr.k, (cuuint64_t)pr.m};
      const cuuint64_t strides[1] = {(cuuint64_t)pr.k * 2};
      const cuuint32_t box[2] = {64, (cuuint32_t)a_rows};
      mp.a_box3d = 0;
      if (!encode(&mp.a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, pr.A, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "A"))
        return false;
    }
  }
  if (grouped) {  // scales: fp16 [k/128][n]
    const cuuint64_t dims[2] = {(cuuint64_t)pr.n, (cuuint64_t)(pr.k / 128)};
    const cuuint64_t strides[1] = {(cuuint64_t)pr.n * 2};
    const cuuint32_t box[2] = {(cuuint32_t)w4a16::TILE_N, (cuuint32_t)(ks >= 128 ? ks / 128 : 1)};
    if (!encode(&mp.s, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, pr.s, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE, "s"))
      return false;
  } else {
    mp.s = mp.a;  // never read
  }
  if (tma_store) {  // output: fp16 [m][n]; the epilogue stores boxes of 16 rows x 128 columns, rows past m are clipped
    const cuuint64_t dims[2] = {(cuuint64_t)pr.n, (cuuint64_t)pr.m};
    const cuuint64_t strides[1] = {(cuuint64_t)pr.n * 2};
    const cuuint32_t box[2] = {(cuuint32_t)w4a16::TILE_N, 16};
    if (!encode(&mp.c, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, pr.C, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE, "C"))
      return false;
  } else {
    mp.c = mp.a;  // never read
  }
  return true;
}

// Takes g_mu for the lookup only.
bool get_maps(const Problem &pr, int ks, int a_rows, bool grouped, bool tma_store, Maps &out) {
  if (pr.fixed_partials) return build_maps(pr, ks, a_rows, grouped, tma_store, out);  // the allocation-free entry point keeps nothing, on the host either
  const MapKey key{pr.B, pr.A, pr.s, tma_store ? pr.C : nullptr, pr.m, pr.n, pr.k, ks, a_rows, grouped ? 1 : 0};
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_maps.find(key);
  if (it == g_maps.end()) {
    Maps mp;
    if (!build_maps(pr, ks, a_rows, grouped, tma_store, mp)) return false;
    if (g_maps.size() >= 1024) g_maps.clear();
    it = g_maps.emplace(key, mp).first;
  }
  out = it->second;
  return true;
}

// scratch + status word of this launch (library-owned per (device, stream), or the built-in array)
bool get_scratch(const Problem &pr, size_t need_slots, w4a16::Params &p) {
  if (pr.fixed_partials) {
    if (need_slots > pr.fixed_slots) {
      g_last_error = "problem needs " + std::to_string(need_slots) + " partial-tile slots, the built-in scratch holds " +
                     std::to_string(pr.fixed_slots);
      return false;
    }
    p.partials = pr.fixed_partials;
    p.status = pr.fixed_status;
    return true;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  StreamCtx *ctx = get_ctx(pr.dev, pr.stream, need_slots);
  if (!ctx) return false;
  p.partials = ctx->partials;
  p.status = ctx->status;
  return true;
}

// the kernels behind launch_single, as traits
template <int TM_, int KS_, bool GROUPED_, int OUT_>
struct GeneralKernel {
  using Cfg = w4a16::Config<TM_, KS_, OUT_>;
  static constexpr int TM = TM_, KS = KS_, THREADS = Cfg::THREADS, SMEM = Cfg::SMEM_BYTES, OUT = OUT_;
  static constexpr bool GROUPED = GROUPED_;
  static constexpr bool IS_DECODE = false;
  static auto kernel() { return w4a16::w4a16_tc_kernel<TM_, KS_, GROUPED_, OUT_>; }
};
template <bool GROUPED_, int OUT_>
struct DecodeKernel {
  using Cfg = w4a16::DecodeConfig<OUT_>;
  static constexpr int TM = Cfg::TM, KS = Cfg::KS, THREADS = Cfg::THREADS, SMEM = Cfg::SMEM_BYTES, OUT = OUT_;
  static constexpr bool GROUPED = GROUPED_;
  static constexpr bool IS_DECODE = true;
  static auto kernel() { return w4a16::w4a16_decode_kernel<GROUPED_, OUT_>; }
};

// W4A16_ALIGNED_CUT=0 in the environment keeps every kernel on the even cut over all workers (A/B timing)
const bool g_aligned_cut = [] {
  const char *e = std::getenv("W4A16_ALIGNED_CUT");
  return !(e && e[0] == '0');
}();

// How many workers (CTAs, or CTA pairs) a problem of `tiles` tiles x `k_iters` stages gets when it has fewer tiles than
// workers.  The even cut over all workers makes most of them straddle two tiles (contributor to one, finisher of the
// other) and cuts a tile workers / tiles ways, and the finisher of a tile folds every other piece's fp32 partial tile
// through L2; fewer, longer ranges trade stages per worker against partial tiles to fold.  The candidates are priced
// in microseconds, t_stage per stage and t_fix per partial tile folded, and the cheapest wins.  Measured at m = 128,
// us per launch: 4096 x 4096 17.5 on the even cut, 13.4 cut 2 ways; 1024 x 4096 27.8 on the even cut (every tile
// 16 ways), 12.8 cut 2 ways.  The prices for 128+ rows (0.45, 2.2) were fitted on CTA pairs at m = 128: 2048 x 8192 cut
// 2 / 4 / 8 ways 19.2 / 16.5 / 19.3, 1024 x 28672 cut 4 / 7 / 8 / 16 ways 31.6 / 26.3 / 26.9 / 33.3, 4096 x 4096 cut 2 / 4
// ways 13.5 / 14.3, 12288 x 4096 whole tiles on 48 pairs 20.7 against 18.8 on the even cut over 74.
int pick_workers(int tiles, int k_iters, int max_workers, double t_stage, double t_fix) {
  // Every range length `per` up to a whole tile is a candidate (the even cut over all workers is one of them): the
  // workers then number ceil(total / per), a tile is cut into ceil(k_iters / per) pieces, and unless `per` divides
  // k_iters (or there is one tile only) the ranges drift against the tile edges, which costs about one more partial
  // tile to fold.
  const long total = (long)tiles * k_iters;
  double best = 0.0;
  int workers = max_workers;
  for (int per = 1; per <= k_iters; ++per) {
    const long w = (total + per - 1) / per;
    if (w > max_workers) continue;
    const int pieces = (k_iters + per - 1) / per;
    const bool lined_up = k_iters % per == 0 || tiles == 1;
    const double cost = per * t_stage + (pieces - 1 + (lined_up ? 0 : 1)) * t_fix;
    if (best == 0.0 || cost < best) best = cost, workers = (int)w;
  }
  return workers;
}

// One CTA per SM, persistent, stream-K over (128-column tile, k-stage).
template <class K>
int launch_single(const Problem &pr) {
  auto kern = K::kernel();
  // at least 116 KiB so that two CTAs can never share an SM (each one allocates all of TMEM)
  constexpr int smem = K::SMEM > 116 * 1024 ? K::SMEM : 116 * 1024;
  static bool attr_done[64] = {false};

  const int nsm = problem_sm_count(pr);
  if (nsm <= 0) return W4A16_ERR_CUDA;

  w4a16::Params p{};
  p.m = pr.m, p.n = pr.n, p.k = pr.k;
  p.n_tiles = pr.n / w4a16::TILE_N;
  p.m_tiles = (pr.m + K::TM - 1) / K::TM;
  p.k_iters = pr.k / K::KS;
  const long total = (long)p.n_tiles * p.m_tiles * p.k_iters;
  if (total > 0x7fffffffL) return W4A16_ERR_ARG;
  p.total_iters = (int)total;
  int grid = pr.sms > 0 ? pr.sms : nsm;
  if (grid > nsm) grid = nsm;  // the finisher of a split tile needs its contributors co-resident
  if (grid > MAX_GRID) grid = MAX_GRID;
  // Skinny batches whose tiles number between ~0.58 and 1 x the SMs: one whole tile per CTA and no fix-up at all beats
  // cutting the tiles to occupy the remaining SMs (12288 x 4096 at m = 16: 9.6 us on 96 CTAs, 10.3 us on 140; the
  // launch is latency- and HBM-bound, not SM-bound).
  const int tiles = p.n_tiles * p.m_tiles;
  if (pr.sms <= 0 && K::TM <= 16 && !pr.orphan_finisher && tiles <= grid && 100 * tiles >= 58 * grid) grid = tiles;
  if (grid > p.total_iters) grid = p.total_iters;
  // wider batch tiles, fewer tiles than SMs: see pick_workers (a partial tile of 128+ rows costs ~2.2 us to fold, one
  // of 32-64 rows ~0.5 us)
  if (pr.sms <= 0 && K::TM > 16 && g_aligned_cut && !pr.orphan_finisher && tiles <= grid)
    grid = pick_workers(tiles, p.k_iters, grid, 0.45, K::TM >= 128 ? 2.2 : 0.5);
  // 16-row tiles outside the whole-tile rule above (very narrow layers: a 128-column layer of 28672 k would be one tile
  // cut 112 ways, its finisher folding 111 slices three at a time): the same pricing, a stage at 0.36 us and a 16-row
  // slice at 0.35 us (2048 x 28672 cut 7 / 8 / 9.25 ways: 14.1 / 14.6 / 14.9 us)
  if (pr.sms <= 0 && K::TM <= 16 && g_aligned_cut && !pr.orphan_finisher && tiles <= grid && grid != tiles)
    grid = pick_workers(tiles, p.k_iters, grid, 0.36, 0.35);
  p.iters_per_cta = (p.total_iters + grid - 1) / grid;
  grid = (p.total_iters + p.iters_per_cta - 1) / p.iters_per_cta;
  p.s = static_cast<const __half *>(pr.s);
  set_output(p, pr);
  p.wait_ns = pr.wait_ns;
  if (pr.orphan_finisher) {
    if (p.k_iters < 2) return W4A16_ERR_ARG;
    p.iters_per_cta = p.k_iters / 2;   // tile 0 is cut in two ...
    grid = 1;                          // ... and only the CTA that finishes it is launched
  }

  if (pr.plan) {
    *pr.plan = w4a16_plan_t{K::IS_DECODE ? W4A16_KERNEL_DECODE : W4A16_KERNEL_SINGLE, K::TM, K::KS, grid, 1, 0, p.iters_per_cta};
    return W4A16_OK;
  }
  Maps mp;
  if (!get_maps(pr, K::KS, K::TM, K::GROUPED, K::OUT == w4a16::OUT_TMA, mp)) return W4A16_ERR_CUDA;
  p.a_box3d = mp.a_box3d;
  if (!get_scratch(pr, (size_t)grid * K::TM * w4a16::TILE_N, p)) return pr.fixed_partials ? W4A16_ERR_ARG : W4A16_ERR_CUDA;
  if (!attr_done[pr.dev]) {   // (idempotent: a race between two host threads sets the same value twice)
    if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "cudaFuncSetAttribute"))
      return W4A16_ERR_CUDA;
    attr_done[pr.dev] = true;
  }
  // Programmatic dependent launch: this kernel may begin (prologue, weight prefetch) while the previous kernel of
  // the stream is finishing; it orders itself behind that kernel with griddepcontrol.wait before it reads
  // activations or writes anything.  Only this library's kernels signal early, so behind any other kernel the
  // launch is an ordinary stream-ordered one.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)K::THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = pr.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_use_pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (!cuda_ok(cudaLaunchKernelEx(&cfg, kern, mp.b, mp.a, mp.s, mp.c, p), "kernel launch")) return W4A16_ERR_CUDA;
  return W4A16_OK;
}

template <int TM, int KS, bool GROUPED, int OUT>
int launch_tc(const Problem &pr) {
  return launch_single<GeneralKernel<TM, KS, GROUPED, OUT>>(pr);
}

// ---- m <= 16, few tiles: one cluster of CL CTAs per tile, partial tiles reduced over the cluster's shared memory
// W4A16_CLUSTER=0 in the environment keeps these problems on the stream-K form (debugging aid, A/B timing)
const bool g_use_cluster = [] {
  const char *e = std::getenv("W4A16_CLUSTER");
  return !(e && e[0] == '0');
}();

// Cluster size for a layer of n_tiles 128-column tiles and k_iters stages per tile: the one that fills most of the
// SMs, if that is at least 0.6 of them and every rank gets between 2 and 32 stages; 0 = stay on stream-K.  (With
// more stages per rank the problem is long enough for stream-K's use of every SM and its deeper ring to win:
// 8192 x 28672 at m = 16 runs 26.6 us on stream-K, 27.3 us on 64 clusters of two.)
int pick_cluster_size(int n_tiles, int k_iters, int nsm) {
  int best = 0;
  for (int cl = 2; cl <= 8; cl *= 2)
    if (n_tiles * cl <= nsm && k_iters >= 2 * cl) best = cl;
  if (!best || k_iters > 32 * best) return 0;
  if (10 * n_tiles * best >= 6 * nsm) return best;
  // Very few tiles (a narrow column shard of a deep layer: 1024 x 28672 is 8 tiles of 112 stages): even clusters of 8
  // leave SMs idle, but stream-K would cut every tile 16 ways and its finisher would then fold fifteen slices
  // through L2, five polls one after the other.  Measured at m = 16: 1024 x 28672 11.5 us on 8 clusters of 8 against
  // 14.7 us on stream-K, 1024 x 8192 7.5 against 12.2 us.
  return (best == 8 && 4 * n_tiles * best >= nsm) ? best : 0;
}

// Returns -2 when the clusters cannot all be resident at once on this device (the caller takes the stream-K form).
template <bool GROUPED, int OUT, int CL>
int launch_decode_cluster(const Problem &pr) {
  using Cfg = w4a16::DecodeConfig<OUT, CL>;
  auto kern = w4a16::w4a16_decode_kernel<GROUPED, OUT, CL>;
  constexpr int smem = Cfg::SMEM_BYTES > 116 * 1024 ? Cfg::SMEM_BYTES : 116 * 1024;
  static bool attr_done[64] = {false};
  static int max_clusters[64] = {0};

  const int nsm = problem_sm_count(pr);
  if (nsm <= 0) return W4A16_ERR_CUDA;
  if (pr.plan) {   // (as if every cluster of this size could be resident: a cluster lives inside one GPC)
    if (nsm / CL < pr.n / w4a16::TILE_N) return -2;
    *pr.plan = w4a16_plan_t{W4A16_KERNEL_DECODE_CLUSTER, Cfg::TM, Cfg::KS, pr.n / w4a16::TILE_N * CL, CL, 0, pr.k / Cfg::KS / CL};
    return W4A16_OK;
  }
  w4a16::Params p{};
  p.m = pr.m, p.n = pr.n, p.k = pr.k;
  p.n_tiles = pr.n / w4a16::TILE_N;
  p.m_tiles = 1;
  p.k_iters = pr.k / Cfg::KS;
  p.total_iters = p.n_tiles * p.k_iters;
  p.iters_per_cta = 1;                 // not used by the cluster form: rank r of a tile's cluster takes k_iters * [r, r + 1) / CL
  p.s = static_cast<const __half *>(pr.s);
  set_output(p, pr);
  p.wait_ns = pr.wait_ns;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(p.n_tiles * CL));
  cfg.blockDim = dim3((unsigned)Cfg::THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = pr.stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = g_use_pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    if (!attr_done[pr.dev]) {
      if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "cudaFuncSetAttribute"))
        return W4A16_ERR_CUDA;
      if (CL > 8 && !cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1), "cudaFuncSetAttribute"))
        return W4A16_ERR_CUDA;
      // rank 0 of a cluster waits for its other ranks, so the ranks must be co-resident: that is what a cluster
      // guarantees; clusters beyond the resident ones simply run later
      cudaLaunchConfig_t probe = cfg;
      probe.gridDim = dim3((unsigned)(nsm / CL * CL));
      int clusters = 0;
      if (!cuda_ok(cudaOccupancyMaxActiveClusters(&clusters, kern, &probe), "cudaOccupancyMaxActiveClusters")) return W4A16_ERR_CUDA;
      max_clusters[pr.dev] = clusters;
      attr_done[pr.dev] = true;
    }
  }
  if (max_clusters[pr.dev] < p.n_tiles) return -2;   // a second wave of clusters would double the time: stream-K instead
  Maps mp;
  if (!get_maps(pr, Cfg::KS, Cfg::TM, GROUPED, OUT == w4a16::OUT_TMA, mp)) return W4A16_ERR_CUDA;
  p.a_box3d = mp.a_box3d;
  if (!get_scratch(pr, 0, p)) return W4A16_ERR_CUDA;   // the status word only: the partial tiles never leave the cluster
  if (!cuda_ok(cudaLaunchKernelEx(&cfg, kern, mp.b, mp.a, mp.s, mp.c, p), "kernel launch (clusters)")) return W4A16_ERR_CUDA;
  return W4A16_OK;
}

// W4A16_TMA_STORE=0 / 1 in the environment picks how finished tiles of the plain GEMM reach C: 2-byte stores from
// registers, or staged in shared memory and stored by the copy engine (cp.async.bulk.tensor).  Both are compiled
// and tested; the default is the one measured faster (see tma_store_default).
const int g_tma_store = [] {
  const char *e = std::getenv("W4A16_TMA_STORE");
  return (e && (e[0] == '0' || e[0] == '1')) ? e[0] - '0' : -1;
}();
bool tma_store_default(const Problem &pr) {
  (void)pr;
  return false;
}
bool use_tma_store(const Problem &pr) { return g_tma_store >= 0 ? g_tma_store == 1 : tma_store_default(pr); }

template <int OUT>
int launch_decode_cluster_o(const Problem &pr, int cl) {
  const bool g = pr.groupsize == 128;
  switch (cl) {
    case 2: return g ? launch_decode_cluster<true, OUT, 2>(pr) : launch_decode_cluster<false, OUT, 2>(pr);
    case 4: return g ? launch_decode_cluster<true, OUT, 4>(pr) : launch_decode_cluster<false, OUT, 4>(pr);
    case 8: return g ? launch_decode_cluster<true, OUT, 8>(pr) : launch_decode_cluster<false, OUT, 8>(pr);
  }
  return -2;
}
int launch_decode_cluster_g(const Problem &pr, int cl) {
  return use_tma_store(pr) ? launch_decode_cluster_o<w4a16::OUT_TMA>(pr, cl) : launch_decode_cluster_o<w4a16::OUT_PLAIN>(pr, cl);
}

// ---- large batches on CTA pairs (cta_group::2): see w4a16_kernel_2sm.cuh
// W4A16_WAVES=0 in the environment keeps the CTA-pair kernel on contiguous stream-K ranges only (debugging aid)
const bool g_use_waves = [] {
  const char *e = std::getenv("W4A16_WAVES");
  return !(e && e[0] == '0');
}();
// W4A16_MFAST=0 / 1 fixes the tile order of the whole-tile waves (1: the tile index runs over the batch tiles first);
// unset, the launcher picks the order with the smaller estimated HBM traffic
const int g_m_fast = [] {
  const char *e = std::getenv("W4A16_MFAST");
  return (e && (e[0] == '0' || e[0] == '1')) ? e[0] - '0' : -1;
}();

// One wave of whole tiles is `pairs` consecutive tile indices.  With the weight-column index running first
// (the reference's order, marlin_cute_trait.h:278-282) a wave shares few batch tiles and sweeps all weight columns:
// activations are read once, weights once per wave unless L2 keeps them.  With the batch index running first it is
// the other way round.  Whatever exceeds ~5/8 of L2 is taken to miss in proportion.  Returns 1 for batch-first.
int pick_tile_order(int dev, double act_bytes, double weight_bytes, int n_tiles, int m_tiles, int pairs) {
  if (g_m_fast >= 0) return g_m_fast;
  const double cap = 0.625 * (dev < 0 ? 126.0 * 1024 * 1024 : (double)l2_bytes(dev));   // (dev < 0: w4a16_plan, a B200's L2)
  const double waves = (double)n_tiles * m_tiles / pairs;
  auto traffic = [&](double bytes, double passes) {
    const double miss = bytes <= cap ? 0.0 : 1.0 - cap / bytes;
    return bytes * (1.0 + (passes - 1.0) * miss);
  };
  const double n_first = act_bytes + traffic(weight_bytes, std::min((double)m_tiles, waves));
  const double m_first = weight_bytes + traffic(act_bytes, std::min((double)n_tiles, waves));
  return m_first < 0.9 * n_first ? 1 : 0;
}

template <int TM, int KS, bool GROUPED, int OUT>
int launch_tc2(const Problem &pr) {
  using Cfg = w4a16::Config2<TM, KS, OUT>;
  auto kern = w4a16::w4a16_tc2_kernel<TM, KS, GROUPED, OUT>;
  constexpr int smem = Cfg::SMEM_BYTES > 116 * 1024 ? Cfg::SMEM_BYTES : 116 * 1024;
  static bool attr_done[64] = {false};
  static int max_pairs[64] = {0};

  const int nsm = problem_sm_count(pr);
  if (nsm <= 0) return W4A16_ERR_CUDA;

  w4a16::Params p{};
  p.m = pr.m, p.n = pr.n, p.k = pr.k;
  p.n_tiles = pr.n / (2 * w4a16::TILE_N);            // 256-column tiles of the pair
  p.m_tiles = (pr.m + TM - 1) / TM;
  p.k_iters = pr.k / Cfg::KS;
  const long total = (long)p.n_tiles * p.m_tiles * p.k_iters;
  if (total > 0x7fffffffL) return W4A16_ERR_ARG;
  p.total_iters = (int)total;
  p.s = static_cast<const __half *>(pr.s);
  set_output(p, pr);
  p.wait_ns = pr.wait_ns;
  p.a_box3d = 1;

  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3((unsigned)Cfg::THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = pr.stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = g_use_pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;

  if (!pr.plan) {
    std::lock_guard<std::mutex> lock(g_mu);
    if (!attr_done[pr.dev]) {
      if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "cudaFuncSetAttribute"))
        return W4A16_ERR_CUDA;
      // the finisher of a split tile needs its contributors co-resident: never launch more pairs than fit at once
      cfg.gridDim = dim3((unsigned)(nsm & ~1));
      int clusters = 0;
      if (!cuda_ok(cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg), "cudaOccupancyMaxActiveClusters")) return W4A16_ERR_CUDA;
      max_pairs[pr.dev] = clusters;
      attr_done[pr.dev] = true;
    }
  }
  const int fit_pairs = pr.plan ? nsm / 2 : max_pairs[pr.dev];
  if (fit_pairs < 1) return -2;   // no CTA pair can be scheduled here: the caller takes the single-CTA kernel
  int pairs = pr.sms > 0 ? pr.sms / 2 : nsm / 2;
  if (pairs < 1) pairs = 1;
  if (pairs > fit_pairs) pairs = fit_pairs;
  if (pairs > MAX_GRID / 2) pairs = MAX_GRID / 2;
  if (pairs > p.total_iters) pairs = p.total_iters;
  // With two or more tiles per pair, all but the last one or two are taken whole and round-robin (tiles in flight at
  // one time are neighbours and share their operands in L2); the rest is split by k-stages as before.
  const int tiles = p.n_tiles * p.m_tiles;
  // A slightly smaller number of pairs that divides the tile count leaves no stream-K part at all (no partial tiles,
  // no straddling): taken when its waves cost fewer stages than the waves plus the stream-K share plus about eight
  // stages' worth of fix-up (12288 x 4096 at m = 1024: 288 tiles = 4 waves of 72 pairs, 81.2 -> 77.1 us).
  if (g_use_waves && g_aligned_cut && pr.sms <= 0 && tiles >= 2 * pairs && tiles % pairs != 0) {
    const int waves = tiles / pairs - 1;
    const long with_sk = (long)waves * p.k_iters + ((long)(tiles - waves * pairs) * p.k_iters + pairs - 1) / pairs + 8;
    for (int c = pairs - 1; 100 * c >= 93 * pairs; --c)
      if (tiles % c == 0 && (long)(tiles / c) * p.k_iters < with_sk) {
        pairs = c;
        break;
      }
  }
  if (g_use_waves && tiles >= 2 * pairs) {
    p.dp_waves = tiles % pairs == 0 ? tiles / pairs : tiles / pairs - 1;
    p.sk_tile0 = p.dp_waves * pairs;
    p.total_iters = (tiles - p.sk_tile0) * p.k_iters;
    p.m_fast = pick_tile_order(pr.plan ? -1 : pr.dev, 2.0 * pr.m * pr.k, 0.5 * pr.n * pr.k, p.n_tiles, p.m_tiles, pairs);
  }
  // No whole-tile waves (fewer than two tiles per pair).  Fewer tiles than pairs: as in the single-CTA kernel
  // (pick_workers).  More: a cut in which every pair takes a whole number of half tiles (cuts at tile edges and
  // midpoints only) beats the even cut over all pairs when it costs a pair at most about eight more stages
  // (4096 x 4096 at m = 1024 on 64 pairs of one and a half tiles each: 34.5 -> 32.7 us).
  if (p.dp_waves == 0 && g_aligned_cut && pr.sms <= 0 && p.total_iters > 0) {
    if (tiles <= pairs) {
      pairs = pick_workers(tiles, p.k_iters, pairs, 0.45, TM >= 128 ? 2.2 : 0.5);
    } else if (p.k_iters % 2 == 0) {
      const int even = (p.total_iters + pairs - 1) / pairs;
      for (int c = pairs; c >= 1 && 5 * c >= 3 * pairs; --c) {
        if (p.total_iters % c || (p.total_iters / c) % (p.k_iters / 2)) continue;
        if (p.total_iters / c - even <= 8) pairs = c;
        break;
      }
    }
  }
  p.iters_per_cta = p.total_iters > 0 ? (p.total_iters + pairs - 1) / pairs : 1;     // per PAIR
  if (p.dp_waves == 0) pairs = (p.total_iters + p.iters_per_cta - 1) / p.iters_per_cta;
  p.workers = pairs;
  if (pr.plan) {
    *pr.plan = w4a16_plan_t{W4A16_KERNEL_PAIRS, TM, Cfg::KS, pairs, 2, p.dp_waves, p.total_iters > 0 ? p.iters_per_cta : 0};
    return W4A16_OK;
  }
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  Maps mp;   // each CTA of the pair loads half of the tile's activation rows
  if (!get_maps(pr, Cfg::KS, Cfg::HALF_ROWS, GROUPED, OUT == w4a16::OUT_TMA, mp)) return W4A16_ERR_CUDA;
  if (!mp.a_box3d) {
    g_last_error = "the CTA-pair kernel needs the 3-D activation view";
    return W4A16_ERR_CUDA;
  }
  if (!get_scratch(pr, (size_t)2 * pairs * TM * w4a16::TILE_N, p)) return W4A16_ERR_CUDA;
  if (!cuda_ok(cudaLaunchKernelEx(&cfg, kern, mp.b, mp.a, mp.s, mp.c, p), "kernel launch (CTA pairs)")) return W4A16_ERR_CUDA;
  return W4A16_OK;
}

// W4A16_PAIRS=0 in the environment keeps large batches on the single-CTA kernel (debugging aid)
const bool g_use_pairs = [] {
  const char *e = std::getenv("W4A16_PAIRS");
  return !(e && e[0] == '0');
}();
// W4A16_DECODE=0 in the environment keeps batches of up to 16 rows on the general kernel (debugging aid, A/B timing)
const bool g_use_decode = [] {
  const char *e = std::getenv("W4A16_DECODE");
  return !(e && e[0] == '0');
}();

// the gathering epilogue is a separate instantiation, so the plain GEMM's code is untouched by it
template <int TM, int KS>
int launch_tc_g(const Problem &pr) {
  using namespace w4a16;
  const bool g = pr.groupsize == 128;
  if (pr.c_ld > 0) return g ? launch_tc<TM, KS, true, OUT_GATHER>(pr) : launch_tc<TM, KS, false, OUT_GATHER>(pr);
  if (use_tma_store(pr)) return g ? launch_tc<TM, KS, true, OUT_TMA>(pr) : launch_tc<TM, KS, false, OUT_TMA>(pr);
  return g ? launch_tc<TM, KS, true, OUT_PLAIN>(pr) : launch_tc<TM, KS, false, OUT_PLAIN>(pr);
}

template <int TM, int KS>
int launch_tc2_g(const Problem &pr) {
  using namespace w4a16;
  const bool g = pr.groupsize == 128;
  if (pr.c_ld > 0) return g ? launch_tc2<TM, KS, true, OUT_GATHER>(pr) : launch_tc2<TM, KS, false, OUT_GATHER>(pr);
  if (use_tma_store(pr)) return g ? launch_tc2<TM, KS, true, OUT_TMA>(pr) : launch_tc2<TM, KS, false, OUT_TMA>(pr);
  return g ? launch_tc2<TM, KS, true, OUT_PLAIN>(pr) : launch_tc2<TM, KS, false, OUT_PLAIN>(pr);
}

int launch_decode_g(const Problem &pr) {
  using namespace w4a16;
  const bool g = pr.groupsize == 128;
  if (pr.c_ld > 0) return g ? launch_single<DecodeKernel<true, OUT_GATHER>>(pr) : launch_single<DecodeKernel<false, OUT_GATHER>>(pr);
  if (use_tma_store(pr)) return g ? launch_single<DecodeKernel<true, OUT_TMA>>(pr) : launch_single<DecodeKernel<false, OUT_TMA>>(pr);
  return g ? launch_single<DecodeKernel<true, OUT_PLAIN>>(pr) : launch_single<DecodeKernel<false, OUT_PLAIN>>(pr);
}

int dispatch_tc(const Problem &pr) {
  // batch tile = UMMA N; the k per stage is as deep as the activation tile allows (fewer, larger TMAs)
  const bool k256 = (pr.k % 256) == 0, k128 = (pr.k % 128) == 0;
  if (pr.m <= 16 && k256 && g_use_decode) {   // the HBM-bound case has a kernel of its own
    // few tiles and no split count from the caller: one cluster per tile
    if (g_use_cluster && pr.sms <= 0 && pr.c_ld == 0 && !pr.orphan_finisher) {
      const int n_tiles = pr.n / w4a16::TILE_N, nsm = problem_sm_count(pr);
      // the size that fills most SMs; if that many clusters of that size cannot be resident together (a cluster
      // lives inside one GPC), half the size, as long as a quarter of the SMs still gets work and a rank no more than
      // 16 stages (2048 x 8192 at m = 16: 7.5 us on 16 clusters of 4 against 9.7 us on stream-K; 2048 x 28672 with 28
      // stages per rank: 15.7 against 14.8 us, so that one stays on stream-K)
      for (int cl = pick_cluster_size(n_tiles, pr.k / 256, nsm); cl >= 2; cl /= 2) {
        const int rc = launch_decode_cluster_g(pr, cl);
        if (rc != -2) return rc;
        if (4 * n_tiles * (cl / 2) < nsm || pr.k / 256 > 16 * (cl / 2)) break;
      }
    }
    return launch_decode_g(pr);
  }
  if (pr.m <= 16) return k256 ? launch_tc_g<16, 256>(pr) : k128 ? launch_tc_g<16, 128>(pr) : launch_tc_g<16, 64>(pr);
  // 17..32 rows on CTA pairs as well (+12-16 % over the general kernel).  The decode kernel widened to 32- and 64-row
  // tiles (two dequant sets: the accumulator sets need the third operand buffer's tensor-memory columns) was measured
  // 5 % slower than the pairs at 32 rows and 50-90 % slower at 64 (4096 x 4096: 9.6 / 17.9 us against 9.1 / 10.0 us):
  // at N = 64 its sixteen MMAs per stage take 1024 tensor clocks on ONE SM, the pair spreads them over two.
  if (g_use_pairs && pr.m > 16 && pr.m <= 32 && k256 && pr.n % 256 == 0 && !pr.fixed_partials && !pr.orphan_finisher) {
    const int rc = launch_tc2_g<32, 256>(pr);
    if (rc != -2) return rc;
  }
  if (pr.m <= 32) return k256 ? launch_tc_g<32, 256>(pr) : k128 ? launch_tc_g<32, 128>(pr) : launch_tc_g<32, 64>(pr);
  // 33..64 rows: the activation tile is already twice the weight bytes of a stage; a CTA pair halves it (+8-12 %)
  if (g_use_pairs && pr.m > 32 && pr.m <= 64 && k256 && pr.n % 256 == 0 && !pr.fixed_partials && !pr.orphan_finisher) {
    const int rc = launch_tc2_g<64, 256>(pr);
    if (rc != -2) return rc;
  }
  if (pr.m <= 64) return k256 ? launch_tc_g<64, 256>(pr) : k128 ? launch_tc_g<64, 128>(pr) : launch_tc_g<64, 64>(pr);
  // batches past 64 rows: 128- or 192-row tiles (192 is the widest that keeps two accumulators and two operand
  // buffers in TMEM)
  const long pad192 = (long)((pr.m + 191) / 192) * 192, pad128 = (long)((pr.m + 127) / 128) * 128;
  // Large batches run on CTA pairs (two SMs per 256-column tile, half the activation traffic per SM): +16 % to +43 %
  // over the single-CTA kernel on B200.  192-row tiles beat 128-row tiles by ~8 % there, 12 % on the single-CTA
  // kernel: take them unless their row padding costs more than that.
  // ... when each pair gets at least ~6 k-stages.  (With the even cut over all pairs the threshold was 32: a few
  // large tiles cut five ways with straddling pairs lost to the single-CTA kernel, 4096 x 4096 at m = 128 25.7 against
  // 17.5 us.  With the cut lined up with the tiles the pairs win down to here: the same problem 14.2 us on pairs,
  // 14.9 us on single CTAs; 4096 x 4096 at m = 96 12.2 against 14.8 us, at m = 256 15.0 against 16.3 us, 8192 x 8192 at
  // m = 128 21.5 against 24.8 us.)
  // The pair kernel runs a ragged last tile at its own width (UMMA N = its rows rounded up to 16), so padding costs
  // nothing there; what a narrow tile still costs is its dequantisation, about 0.55 of a full 192-row tile's time.
  // A full 128-row tile takes about 0.72 of a 192-row tile's time.
  // (a ragged tile of exactly 128 rows inside the 192-row kernel measured 1-2 % behind the 128-row kernel, which has
  // four operand buffers in tensor memory instead of two: its cost is taken as 0.73)
  auto pair_cost = [&](int t, double full_cost) {
    const int rem = pr.m % t, rows = (rem + 15) & ~15;
    const double ragged = rows <= 128 ? std::max(0.73 * rows / 128.0, 0.55) : 0.73 + 0.27 * (rows - 128) / 64.0;
    return (pr.m / t) * full_cost + (rem ? ragged : 0.0);
  };
  // W4A16_FORCE_TM=128 / 192 in the environment fixes the batch tile of the large-batch kernels (A/B timing)
  static const int force_tm = [] {
    const char *e = std::getenv("W4A16_FORCE_TM");
    const int v = e ? atoi(e) : 0;
    return (v == 128 || v == 192) ? v : 0;
  }();
  const long tm = force_tm ? force_tm : (pair_cost(192, 1.0) < pair_cost(128, 0.72) ? 192 : 128);   // (a tie: a batch below 128 rows is one ragged tile either way)
  // (an explicit split count from the caller stands in for the 74 pairs of a whole B200)
  // (fewer tiles than pairs: the pairs that pick_workers would put to work)
  const int pair_tiles = (int)((pr.n / 256) * ((pr.m + tm - 1) / tm));
  int pairs_at_work = pr.sms > 1 ? pr.sms / 2 : (pr.plan ? std::max(pr.plan_sms / 2, 1) : 74);
  if (pr.sms <= 0 && g_aligned_cut && pr.n % 256 == 0 && k128 && pair_tiles <= pairs_at_work)
    pairs_at_work = pick_workers(pair_tiles, pr.k / 128, pairs_at_work, 0.45, 2.2);
  const long pair_stages = (long)pair_tiles * (pr.k / 128) / pairs_at_work;
  // (W4A16_PAIR_MIN_STAGES in the environment moves the threshold: A/B timing)
  static const int pair_min = [] { const char *e = std::getenv("W4A16_PAIR_MIN_STAGES"); return e ? atoi(e) : 6; }();
  if (g_use_pairs && k128 && pr.n % 256 == 0 && pair_stages >= pair_min && !pr.fixed_partials && !pr.orphan_finisher) {
    int rc;
    if (tm == 192)
      rc = launch_tc2_g<192, 128>(pr);
    else
      rc = launch_tc2_g<128, 128>(pr);
    if (rc != -2) return rc;
  }
  if (k128 && pad192 * 100 <= pad128 * 113) return launch_tc_g<192, 128>(pr);
  return k128 ? launch_tc_g<128, 128>(pr) : launch_tc_g<128, 64>(pr);
}

// ---- diagnostic CUDA-core kernel: one thread per output, closed form of the packed layout
__global__ void w4a16_simt_kernel(const __half *A, const uint32_t *B, __half *C, const __half *s, int m, int n, int k,
                                  int groupsize) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)m * n) return;
  const int mm = (int)(idx / n), nn = (int)(idx % n);
  const int nr = nn % 64, j = nr / 16, hi = (nr % 16) / 8;
  const long cbase = 128L * (nn / 64) + j;
  float acc = 0.f;
  for (int kk = 0; kk < k; ++kk) {
    const int kr = kk % 16;
    const int lane = 4 * (nr % 8) + (kr % 8) / 2;
    const int nib = 4 * (kr % 2) + 2 * hi + kr / 8;
    const int code = (int)((B[(long)(kk / 16) * 2 * n + cbase + 4 * lane] >> (4 * nib)) & 0xfu);
    __half w = __int2half_rn(code - 8);
    if (groupsize != -1) w = __hmul(w, s[(long)(kk / groupsize) * n + 64 * (nn / 64) + 8 * (nr % 8) + nr / 8]);
    acc += __half2float(A[(long)mm * k + kk]) * __half2float(w);
  }
  __half h = __float2half(acc);
  if (groupsize == -1) {
    const int c32 = nn % 32;
    h = __hmul(h, s[nn - c32 + 8 * ((c32 % 8) / 2) + 2 * (c32 / 8) + c32 % 2]);
  }
  C[idx] = h;
}

int launch_simt(const Problem &pr) {
  const long total = (long)pr.m * pr.n;
  const int threads = 256;
  const long blocks = (total + threads - 1) / threads;
  if (blocks > 0x7fffffffL) return W4A16_ERR_ARG;
  w4a16_simt_kernel<<<(unsigned)blocks, threads, 0, pr.stream>>>(
      static_cast<const __half *>(pr.A), static_cast<const uint32_t *>(pr.B), static_cast<__half *>(pr.C),
      static_cast<const __half *>(pr.s), pr.m, pr.n, pr.k, pr.groupsize);
  if (!cuda_ok(cudaGetLastError(), "kernel launch")) return W4A16_ERR_CUDA;
  return W4A16_OK;
}

// Shape / dispatch checks with the reference's meaning and order (marlin_cute_kernel.cu:39-60,95-107).
int check_problem(int prob_m, int prob_n, int prob_k, int groupsize, int &thread_k, int &thread_n) {
  if (thread_k == -1 || thread_n == -1) {
    if (prob_m <= 16) {
      thread_k = 128, thread_n = 128;
    } else {
      thread_k = 64, thread_n = 256;
    }
  }
  if (thread_k <= 0 || thread_n <= 0) return W4A16_ERR_KERN_SHAPE;
  const int group_blocks = groupsize == -1 ? -1 : groupsize / 16;
  if (prob_n % thread_n != 0 || prob_k % thread_k != 0 || (group_blocks > 0 && prob_k % group_blocks != 0))
    return W4A16_ERR_PROB_SHAPE;
  if (prob_m == 0 || prob_n == 0 || prob_k == 0) return -1;  // nothing to do
  // the reference instantiates (thread_n, thread_k) = (128,128) for one 16-row block only and (256,64) for
  // one to four blocks per launch chunk, group size 128 or -1
  const bool t128 = (thread_n == 128 && thread_k == 128), t256 = (thread_n == 256 && thread_k == 64);
  if (!(t128 || t256)) return W4A16_ERR_KERN_SHAPE;
  if (t128 && prob_m > 16) return W4A16_ERR_KERN_SHAPE;
  if (groupsize != -1 && groupsize != 128) return W4A16_ERR_KERN_SHAPE;
  return W4A16_OK;
}

// The launch, the per-device kernel attributes and the built-in scratch all belong to the CURRENT device, which the
// caller must have made `dev` (the reference's launcher has the same rule: it never calls cudaSetDevice and uses
// `dev` only for the SM count, marlin_cute_kernel.cu:37-38).  Checked on every call: it is one thread-local read.
bool device_is_current(int dev) {
  int cur = -1;
  if (!cuda_ok(cudaGetDevice(&cur), "cudaGetDevice")) return false;
  if (cur != dev) {
    g_last_error = "device " + std::to_string(dev) + " must be the current device (current is " + std::to_string(cur) + ")";
    return false;
  }
  return true;
}

int gemm_entry(bool simt, const void *A, const void *B, void *C, const void *s, int prob_m, int prob_n, int prob_k,
               void *workspace, int groupsize, int dev, cudaStream_t stream, int thread_k, int thread_n, int sms,
               int max_par) {
  (void)max_par;
  (void)workspace;  // the caller's lock array is not needed by this kernel and is left untouched (all zero)
  if (prob_m < 0 || prob_n < 0 || prob_k < 0) return W4A16_ERR_ARG;
  const int chk = check_problem(prob_m, prob_n, prob_k, groupsize, thread_k, thread_n);
  if (chk == -1) return W4A16_OK;
  if (chk != W4A16_OK) return chk;
  if (!A || !B || !C || !s) return W4A16_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C) |
       reinterpret_cast<uintptr_t>(s)) & 15)
    return W4A16_ERR_ARG;
  if (dev < 0 || dev >= 64) return W4A16_ERR_ARG;
  if (!device_is_current(dev)) return W4A16_ERR_ARG;
  Problem pr{A, B, s, C, prob_m, prob_n, prob_k, groupsize, dev, sms, stream};
  return simt ? launch_simt(pr) : dispatch_tc(pr);
}

}  // namespace

int marlin_cute(const void *A, const void *B, void *C, void *s, int prob_m, int prob_n, int prob_k, void *workspace,
                int groupsize, int dev, cudaStream_t stream, int thread_k, int thread_n, int sms, int max_par) {
  return gemm_entry(false, A, B, C, s, prob_m, prob_n, prob_k, workspace, groupsize, dev, stream, thread_k, thread_n,
                    sms, max_par);
}

extern "C" int w4a16_marlin_gemm(const void *A, const void *B, void *C, const void *s, int prob_m, int prob_n,
                                 int prob_k, void *workspace, int groupsize, int dev, void *stream, int thread_k,
                                 int thread_n, int sms, int max_par) {
  return gemm_entry(false, A, B, C, s, prob_m, prob_n, prob_k, workspace, groupsize, dev,
                    static_cast<cudaStream_t>(stream), thread_k, thread_n, sms, max_par);
}

extern "C" int w4a16_plan(int prob_m, int prob_n, int prob_k, int groupsize, int sms, int device_sms, w4a16_plan_t *out) {
  if (!out || device_sms < 2 || device_sms > MAX_GRID || prob_m < 0 || prob_n < 0 || prob_k < 0) return W4A16_ERR_ARG;
  int thread_k = -1, thread_n = -1;
  const int chk = check_problem(prob_m, prob_n, prob_k, groupsize, thread_k, thread_n);
  *out = w4a16_plan_t{W4A16_KERNEL_NONE, 0, 0, 0, 0, 0, 0};
  if (chk == -1) return W4A16_OK;
  if (chk != W4A16_OK) return chk;
  Problem pr{nullptr, nullptr, nullptr, nullptr, prob_m, prob_n, prob_k, groupsize, 0, sms, nullptr};
  pr.plan = out;
  pr.plan_sms = device_sms;
  return dispatch_tc(pr);
}

// The GEMM with HOST activations and HOST output: copy in, multiply, copy out, all enqueued on `stream`.
//
// Small host<->device copies through the copy engines cost about ten microseconds each on the stream (set-up and
// completion, not bytes), which is more than a decode GEMM.  When both host buffers are page-locked (and therefore
// addressable from the device) and the batch is small, the copies are done by the SMs instead:
//   * a few CTAs read A_host over PCIe into A_stage; the kernel signals griddepcontrol.launch_dependents at once, so
//     the GEMM behind it starts its prologue and weight prefetch meanwhile and waits for the copy (griddepcontrol.wait)
//     only before it loads activations;
//   * the GEMM's epilogue writes C rows straight into C_host (posted PCIe writes): no second copy, no C_stage.
// That serves a caller who runs one layer after the other on ONE stream (measured: the four 7B layers at m = 16 in
// 121 us instead of 162 us); with several streams the copy engines overlap one layer's copies with another layer's
// kernel and the direct writes only lengthen the kernels (66 us against 59.5 us; copying only A with the SMs: 65 us), so it is opt-in:
// W4A16_HOST_DIRECT=1 in the environment.
namespace {
const bool g_host_direct = [] {
  const char *e = std::getenv("W4A16_HOST_DIRECT");
  return e && e[0] == '1';
}();

__global__ void __launch_bounds__(512) copy_in_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst, size_t n16) {
  sm100::pdl_launch_dependents();   // the GEMM behind this kernel orders itself with griddepcontrol.wait
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) dst[i] = src[i];
}

// device address of a page-locked host buffer, or null when the buffer is pageable (looked up once per pointer)
void *device_view_of_host(const void *host) {
  static std::map<const void *, void *> cache;   // guarded by g_mu
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = cache.find(host);
  if (it != cache.end()) return it->second;
  void *dptr = nullptr;
  cudaPointerAttributes attr{};
  if (cudaPointerGetAttributes(&attr, host) == cudaSuccess && attr.type == cudaMemoryTypeHost && attr.devicePointer)
    dptr = attr.devicePointer;
  else
    cudaGetLastError();   // a pageable pointer is not an error here
  if (cache.size() >= 4096) cache.clear();
  cache[host] = dptr;
  return dptr;
}
}  // namespace

extern "C" int w4a16_marlin_gemm_host(const void *A_host, const void *B, void *C_host, const void *s, int prob_m,
                                      int prob_n, int prob_k, void *workspace, int groupsize, int dev, void *stream,
                                      void *A_stage, void *C_stage) {
  const int sms = -1;
  if (prob_m < 0 || prob_n < 0 || prob_k < 0) return W4A16_ERR_ARG;
  int tk = -1, tn = -1;
  const int chk = check_problem(prob_m, prob_n, prob_k, groupsize, tk, tn);
  if (chk == -1) return W4A16_OK;
  if (chk != W4A16_OK) return chk;
  if (!A_host || !C_host || !A_stage || !C_stage) return W4A16_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t a_bytes = sizeof(__half) * (size_t)prob_m * prob_k;
  if (g_host_direct && prob_m <= 64 && (a_bytes & 15) == 0 && !(reinterpret_cast<uintptr_t>(A_stage) & 15)) {
    void *dA = device_view_of_host(A_host), *dC = device_view_of_host(C_host);
    if (dA && dC && !((reinterpret_cast<uintptr_t>(dA) | reinterpret_cast<uintptr_t>(dC)) & 15)) {
      if (!device_is_current(dev)) return W4A16_ERR_ARG;
      copy_in_kernel<<<4, 512, 0, st>>>(static_cast<const uint4 *>(dA), static_cast<uint4 *>(A_stage), a_bytes / 16);
      if (!cuda_ok(cudaGetLastError(), "copy-in launch")) return W4A16_ERR_CUDA;
      return gemm_entry(false, A_stage, B, dC, s, prob_m, prob_n, prob_k, workspace, groupsize, dev, st, -1, -1, sms, 16);
    }
  }
  if (!cuda_ok(cudaMemcpyAsync(A_stage, A_host, a_bytes, cudaMemcpyHostToDevice, st), "cudaMemcpyAsync(A)"))
    return W4A16_ERR_CUDA;
  const int rc = gemm_entry(false, A_stage, B, C_stage, s, prob_m, prob_n, prob_k, workspace, groupsize, dev, st, -1, -1,
                            sms, 16);
  if (rc != W4A16_OK) return rc;
  if (!cuda_ok(cudaMemcpyAsync(C_host, C_stage, sizeof(__half) * (size_t)prob_m * prob_n, cudaMemcpyDeviceToHost, st),
               "cudaMemcpyAsync(C)"))
    return W4A16_ERR_CUDA;
  return W4A16_OK;
}

extern "C" int w4a16_marlin_gemm_simt(const void *A, const void *B, void *C, const void *s, int prob_m, int prob_n,
                                      int prob_k, void *workspace, int groupsize, int dev, void *stream, int thread_k,
                                      int thread_n, int sms, int max_par) {
  return gemm_entry(true, A, B, C, s, prob_m, prob_n, prob_k, workspace, groupsize, dev,
                    static_cast<cudaStream_t>(stream), thread_k, thread_n, sms, max_par);
}

// ---- allocation-free variant ---------------------------------------------------------------------------------
// Scratch of the stream-K fix-up as a file-scope device array: it exists as soon as the library is loaded on a
// device (5 MiB of every GPU that loads it, until the process exits) and is shared by every call.
constexpr int BUILTIN_MAX_M = 64;                                    // batch rows (partial tiles are TM <= 64 wide)
constexpr size_t BUILTIN_SLOTS = (size_t)160 * BUILTIN_MAX_M * w4a16::TILE_N;   // up to 160 CTAs: 1 310 720 slots
static __device__ __align__(256) uint32_t g_builtin_partials[BUILTIN_SLOTS];
static __device__ __align__(256) int g_builtin_status;

namespace {
struct BuiltinScratch {
  uint32_t *partials = nullptr;   // DEVICE addresses of the two symbols above, per device
  int *status = nullptr;
  bool ready = false;
};
BuiltinScratch g_builtin[64];

// Once per device, with that device current.  In host code `g_builtin_partials` is only a stand-in for the
// symbol, not a device address: the address has to be asked for.  Called with g_mu held.
int builtin_setup(int dev, cudaStream_t stream) {
  BuiltinScratch &b = g_builtin[dev];
  if (b.ready) return W4A16_OK;
  void *pp = nullptr, *ps = nullptr;
  if (!cuda_ok(cudaGetSymbolAddress(&pp, g_builtin_partials), "cudaGetSymbolAddress(partials)")) return W4A16_ERR_CUDA;
  if (!cuda_ok(cudaGetSymbolAddress(&ps, g_builtin_status), "cudaGetSymbolAddress(status)")) return W4A16_ERR_CUDA;
  // idle pattern in every slot, status clear; finished before any kernel of any stream can touch them
  if (!cuda_ok(cudaMemsetAsync(pp, 0xff, sizeof(uint32_t) * BUILTIN_SLOTS, stream), "cudaMemsetAsync(partials)")) return W4A16_ERR_CUDA;
  if (!cuda_ok(cudaMemsetAsync(ps, 0, sizeof(int), stream), "cudaMemsetAsync(status)")) return W4A16_ERR_CUDA;
  if (!cuda_ok(cudaStreamSynchronize(stream), "cudaStreamSynchronize")) return W4A16_ERR_CUDA;
  b.partials = static_cast<uint32_t *>(pp);
  b.status = static_cast<int *>(ps);
  b.ready = true;
  return W4A16_OK;
}
}  // namespace

extern "C" int w4a16_marlin_gemm_builtin_scratch(const void *A, const void *B, void *C, const void *s, int prob_m,
                                                 int prob_n, int prob_k, void *workspace, int groupsize, int dev,
                                                 void *stream, int thread_k, int thread_n, int sms, int max_par) {
  (void)max_par;
  (void)workspace;
  if (prob_m < 0 || prob_n < 0 || prob_k < 0) return W4A16_ERR_ARG;
  const int chk = check_problem(prob_m, prob_n, prob_k, groupsize, thread_k, thread_n);
  if (chk == -1) return W4A16_OK;
  if (chk != W4A16_OK) return chk;
  if (prob_m > BUILTIN_MAX_M) {
    g_last_error = "m = " + std::to_string(prob_m) + " exceeds the built-in scratch limit of " + std::to_string(BUILTIN_MAX_M) +
                   " rows; use w4a16_marlin_gemm";
    return W4A16_ERR_ARG;
  }
  if (!A || !B || !C || !s) return W4A16_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C) |
       reinterpret_cast<uintptr_t>(s)) & 15)
    return W4A16_ERR_ARG;
  if (dev < 0 || dev >= 64) return W4A16_ERR_ARG;
  // every call, not only the first: the symbol addresses looked up for `dev` mean nothing on another device
  if (!device_is_current(dev)) return W4A16_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Problem pr{A, B, s, C, prob_m, prob_n, prob_k, groupsize, dev, sms, st};
  {
    std::lock_guard<std::mutex> lock(g_mu);
    const int rc = builtin_setup(dev, st);
    if (rc != W4A16_OK) return rc;
    pr.fixed_partials = g_builtin[dev].partials;
    pr.fixed_status = g_builtin[dev].status;
    pr.fixed_slots = BUILTIN_SLOTS;
  }
  return dispatch_tc(pr);
}

// Self-test of the bounded waits: the GEMM is set up so that the CTA finishing tile 0 expects a partial tile
// from a CTA that is never launched.  Nothing faults or spins on: after the limit the kernel records a status,
// unwinds and returns, and w4a16_device_status reports W4A16_ERR_TIMEOUT.  C is left undefined.
// limit_ms < 0 runs the same on the built-in scratch of w4a16_marlin_gemm_builtin_scratch for -limit_ms ms.
extern "C" int w4a16_selftest_unanswered_wait(const void *A, const void *B, void *C, const void *s, int prob_m,
                                              int prob_n, int prob_k, int groupsize, int dev, void *stream,
                                              int limit_ms) {
  int tk = -1, tn = -1;
  const bool builtin = limit_ms < 0;
  if (builtin) limit_ms = -limit_ms;
  if (prob_m <= 0 || prob_n <= 0 || prob_k <= 0 || limit_ms <= 0 || limit_ms > 5000) return W4A16_ERR_ARG;
  if (builtin && prob_m > BUILTIN_MAX_M) return W4A16_ERR_ARG;
  const int chk = check_problem(prob_m, prob_n, prob_k, groupsize, tk, tn);
  if (chk != W4A16_OK) return chk;
  if (!A || !B || !C || !s || dev < 0 || dev >= 64) return W4A16_ERR_ARG;
  if (!device_is_current(dev)) return W4A16_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Problem pr{A, B, s, C, prob_m, prob_n, prob_k, groupsize, dev, -1, st};
  pr.orphan_finisher = true;
  pr.wait_ns = (uint64_t)limit_ms * 1000000ull;
  if (builtin) {
    std::lock_guard<std::mutex> lock(g_mu);
    const int rc = builtin_setup(dev, st);
    if (rc != W4A16_OK) return rc;
    pr.fixed_partials = g_builtin[dev].partials;
    pr.fixed_status = g_builtin[dev].status;
    pr.fixed_slots = BUILTIN_SLOTS;
  }
  return dispatch_tc(pr);
}

extern "C" int w4a16_workspace_ints(int prob_n, int max_par) {
  if (prob_n < 0 || max_par < 0) return 0;
  return prob_n / 128 * max_par;
}

// status word of the allocation-free variant (shared by all streams of the device)
static int builtin_status(int dev) {
  uint32_t *partials = nullptr;
  int *status = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    if (dev < 0 || dev >= 64 || !g_builtin[dev].ready) return W4A16_OK;
    partials = g_builtin[dev].partials;
    status = g_builtin[dev].status;
  }
  int word = 0;
  if (!cuda_ok(cudaMemcpy(&word, status, sizeof(int), cudaMemcpyDeviceToHost), "cudaMemcpy(status)")) return W4A16_ERR_CUDA;
  if (word == 0) return W4A16_OK;
  if (!cuda_ok(cudaMemset(status, 0, sizeof(int)), "cudaMemset(status)")) return W4A16_ERR_CUDA;
  if (!cuda_ok(cudaMemset(partials, 0xff, sizeof(uint32_t) * BUILTIN_SLOTS), "cudaMemset(partials)")) return W4A16_ERR_CUDA;
  g_last_error = "device-side wait timed out at site " + std::to_string(word >> 8) + " (built-in scratch variant)";
  return W4A16_ERR_TIMEOUT;
}

extern "C" int w4a16_device_status(int dev, void *stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!cuda_ok(cudaStreamSynchronize(st), "cudaStreamSynchronize")) return W4A16_ERR_CUDA;
  int *status = nullptr;
  std::vector<std::pair<uint32_t *, size_t>> blocks;
  bool launched_here = false;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_ctx.find({dev, st});
    if (it != g_ctx.end()) {
      launched_here = true;
      status = it->second.status;
      blocks = it->second.retired;
      if (it->second.partials) blocks.emplace_back(it->second.partials, it->second.partial_slots);
    }
  }
  if (!launched_here) return builtin_status(dev);  // no library-allocated scratch on this (device, stream)
  int word = 0;
  if (!cuda_ok(cudaMemcpy(&word, status, sizeof(int), cudaMemcpyDeviceToHost), "cudaMemcpy(status)")) return W4A16_ERR_CUDA;
  if (word == 0) return builtin_status(dev);
  if (!cuda_ok(cudaMemset(status, 0, sizeof(int)), "cudaMemset(status)")) return W4A16_ERR_CUDA;
  // a kernel that gave up may have left partial-tile slots written
  for (auto &b : blocks)
    if (!cuda_ok(cudaMemset(b.first, 0xff, sizeof(uint32_t) * b.second), "cudaMemset(partials)")) return W4A16_ERR_CUDA;
  g_last_error = "device-side wait timed out at site " + std::to_string(word >> 8);
  return W4A16_ERR_TIMEOUT;
}

extern "C" int w4a16_release_stream(int dev, void *stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!cuda_ok(cudaStreamSynchronize(st), "cudaStreamSynchronize")) return W4A16_ERR_CUDA;
  StreamCtx c;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_ctx.find({dev, st});
    if (it == g_ctx.end()) return W4A16_OK;
    c = it->second;
    g_ctx.erase(it);
  }
  bool ok = true;
  for (auto &b : c.retired) ok &= cuda_ok(cudaFree(b.first), "cudaFree(partials)");
  if (c.partials) ok &= cuda_ok(cudaFree(c.partials), "cudaFree(partials)");
  if (c.status) ok &= cuda_ok(cudaFree(c.status), "cudaFree(status)");
  return ok ? W4A16_OK : W4A16_ERR_CUDA;
}

extern "C" const char *w4a16_last_cuda_error(void) { return g_last_error.c_str(); }

// ---------------------------------------------------------------------------------------------------------
// Column-sharded GEMM with a gathering epilogue, and the peer-memory plumbing it needs.  One process per GPU.

namespace {
std::map<std::array<uintptr_t, 9>, void *> g_dst_tables;   // (device, up to 7 destinations, 0-padded) -> device table
}

extern "C" int w4a16_marlin_gemm_gather(const void *A, const void *B, const void *s, int prob_m, int n_local, int prob_k,
                                        void *workspace, int groupsize, int dev, void *stream, void *const *dst,
                                        int world, int rank) {
  (void)workspace;
  if (prob_m < 0 || n_local < 0 || prob_k < 0) return W4A16_ERR_ARG;
  if (!dst || world < 1 || world > 8 || rank < 0 || rank >= world) {
    g_last_error = "gather: world must be 1..8 and 0 <= rank < world";
    return W4A16_ERR_ARG;
  }
  int thread_k = -1, thread_n = -1;
  const int chk = check_problem(prob_m, n_local, prob_k, groupsize, thread_k, thread_n);
  if (chk == -1) return W4A16_OK;
  if (chk != W4A16_OK) return chk;
  if (!A || !B || !s) return W4A16_ERR_ARG;
  uintptr_t bits = reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(s);
  for (int r = 0; r < world; ++r) {
    if (!dst[r]) return W4A16_ERR_ARG;
    bits |= reinterpret_cast<uintptr_t>(dst[r]);
  }
  if (bits & 15) return W4A16_ERR_ARG;
  if (dev < 0 || dev >= 64) return W4A16_ERR_ARG;
  if (!device_is_current(dev)) return W4A16_ERR_ARG;
  if ((long)n_local * world > 0x7fffffffL) return W4A16_ERR_ARG;
  Problem pr{A, B, s, dst[rank], prob_m, n_local, prob_k, groupsize, dev, -1, static_cast<cudaStream_t>(stream)};
  pr.c_ld = n_local * world;
  pr.c_col0 = n_local * rank;
  if (world > 1) {
    // the other ranks' buffers, as a table in device memory that is made once per distinct set of destinations.
    // Order: rank + 1, rank + 2, ... (mod world), so that at any moment the ranks' stores head for different GPUs
    // instead of all ranks writing to GPU 0 first, then to GPU 1, ...
    std::array<uintptr_t, 9> key{};
    key[0] = (uintptr_t)dev;
    for (int j = 1; j < world; ++j) key[1 + pr.n_extra++] = reinterpret_cast<uintptr_t>(dst[(rank + j) % world]);
    std::lock_guard<std::mutex> lock(g_mu);
    void *&tab = g_dst_tables[key];
    if (!tab) {
      if (!cuda_ok(cudaMalloc(&tab, 8 * sizeof(void *)), "cudaMalloc(destination table)")) return W4A16_ERR_CUDA;
      if (!cuda_ok(cudaMemcpy(tab, &key[1], 8 * sizeof(void *), cudaMemcpyHostToDevice), "cudaMemcpy(destination table)")) {
        cudaFree(tab);
        g_dst_tables.erase(key);
        return W4A16_ERR_CUDA;
      }
    }
    pr.C_extra = static_cast<void *const *>(tab);
  }
  return dispatch_tc(pr);
}

extern "C" int w4a16_peer_alloc(size_t bytes, void **dptr, void *handle64) {
  if (!dptr || !handle64 || bytes == 0) return W4A16_ERR_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the ABI");
  void *p = nullptr;
  if (!cuda_ok(cudaMalloc(&p, bytes), "cudaMalloc(peer buffer)")) return W4A16_ERR_CUDA;
  cudaIpcMemHandle_t h;
  if (!cuda_ok(cudaMemset(p, 0, bytes), "cudaMemset(peer buffer)") ||
      !cuda_ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize") ||
      !cuda_ok(cudaIpcGetMemHandle(&h, p), "cudaIpcGetMemHandle")) {
    cudaFree(p);
    return W4A16_ERR_CUDA;
  }
  std::memcpy(handle64, &h, sizeof(h));
  *dptr = p;
  return W4A16_OK;
}

extern "C" int w4a16_peer_open(const void *handle64, void **dptr) {
  if (!dptr || !handle64) return W4A16_ERR_ARG;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, sizeof(h));
  void *p = nullptr;
  if (!cuda_ok(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle")) return W4A16_ERR_CUDA;
  *dptr = p;
  return W4A16_OK;
}

extern "C" int w4a16_peer_close(void *dptr) {
  return cuda_ok(cudaIpcCloseMemHandle(dptr), "cudaIpcCloseMemHandle") ? W4A16_OK : W4A16_ERR_CUDA;
}

extern "C" int w4a16_peer_free(void *dptr) { return cuda_ok(cudaFree(dptr), "cudaFree") ? W4A16_OK : W4A16_ERR_CUDA; }

namespace {
struct PeerFlags {
  uint32_t *p[8];
};

// One warp.  Flag block of a rank: words 0..7 = the epoch last announced by rank r, word 8 = this rank's own epoch
// counter.  The epoch lives on the device, so a captured launch keeps working when it is replayed.
__global__ void peer_barrier_kernel(PeerFlags f, int world, int rank, uint64_t wait_ns, int *status) {
  const int lane = threadIdx.x;
  // launched with programmatic stream serialisation: let the next kernel of the stream begin its prologue now (it
  // orders itself behind this kernel with griddepcontrol.wait), then wait for the previous kernel to complete
  sm100::pdl_launch_dependents();
  sm100::pdl_wait_prior_grid();
  uint32_t *mine = f.p[rank];
  uint32_t e = 0;
  if (lane == 0) {
    e = mine[8] + 1;
    mine[8] = e;
  }
  e = __shfl_sync(0xffffffffu, e, 0);
  __threadfence_system();
  if (lane < world) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f.p[lane] + rank), "r"(e) : "memory");
    const uint64_t t0 = sm100::globaltimer_ns();
    for (;;) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine + lane) : "memory");
      if ((int32_t)(v - e) >= 0) break;
      if (sm100::globaltimer_ns() - t0 > wait_ns) {
        atomicCAS(status, 0, w4a16::STATUS_TIMEOUT | (30 << 8));
        break;
      }
    }
  }
}
}  // namespace

extern "C" int w4a16_peer_barrier(void *const *flags, int world, int rank, int dev, void *stream, int limit_ms) {
  if (!flags || world < 1 || world > 8 || rank < 0 || rank >= world || dev < 0 || dev >= 64) return W4A16_ERR_ARG;
  if (limit_ms < 1 || limit_ms > 5000) return W4A16_ERR_ARG;
  PeerFlags f{};
  for (int r = 0; r < world; ++r) {
    if (!flags[r] || (reinterpret_cast<uintptr_t>(flags[r]) & 63)) return W4A16_ERR_ARG;
    f.p[r] = static_cast<uint32_t *>(flags[r]);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int *status = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    StreamCtx *ctx = get_ctx(dev, st, 0);
    if (!ctx) return W4A16_ERR_CUDA;
    status = ctx->status;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(32);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_use_pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cuda_ok(cudaLaunchKernelEx(&cfg, peer_barrier_kernel, f, world, rank, (uint64_t)limit_ms * 1000000ull, status),
                 "barrier launch")
             ? W4A16_OK
             : W4A16_ERR_CUDA;
}

#ifdef W4A16_TRACE
// trace builds only: point the kernels at a [gridDim.x][16] uint64 buffer for phase time stamps
extern "C" int w4a16_debug_set_trace(void *buf) {
  unsigned long long *p = static_cast<unsigned long long *>(buf);
  return cuda_ok(cudaMemcpyToSymbol(w4a16::g_trace, &p, sizeof(p)), "cudaMemcpyToSymbol") ? W4A16_OK : W4A16_ERR_CUDA;
}
#endif
