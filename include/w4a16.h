/*
 * C ABI of the B200 (sm_100a) W4A16 GEMM library: fp16 activations x Marlin-packed int4 weights
 * with fp16 group (or per-channel) scales, fp32 accumulation, fp16 output.
 *
 * Plain pointers and sizes only; no framework types.  Device pointers are caller-owned.  Every
 * entry point replaces one interface of the reference project (cited as file:line within the
 * reference tree).  The C++ twin with the reference's exact launcher signature is declared in
 * marlin_cute.h.
 */
#ifndef W4A16_H_
#define W4A16_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Return codes.  1 and 2 are the reference's (gemm/marlin_gemm/marlin_cute_kernel.cu:4-5,
 * gemm/marlin_gemm/marlin_gemm.cpp:16-17); larger values are new failure kinds and never alias them. */
#define W4A16_OK 0
#define W4A16_ERR_PROB_SHAPE 1 /* n, k not divisible by the tile / group (marlin_cute_kernel.cu:56-58) */
#define W4A16_ERR_KERN_SHAPE 2 /* no kernel for (thread_k, thread_n, groupsize) (marlin_cute_kernel.cu:105-107) */
#define W4A16_ERR_CUDA 3       /* a CUDA runtime / driver call failed (see w4a16_last_cuda_error) */
#define W4A16_ERR_TIMEOUT 4    /* a bounded device-side wait ran out; reported by w4a16_device_status */
#define W4A16_ERR_ARG 5        /* null pointer, misaligned pointer or size out of range */

/*
 * The GEMM.  Replaces  int marlin_cute(...)  gemm/marlin_gemm/marlin_cute_kernel.cu:28-31 (and its
 * caller-side declaration gemm/marlin_gemm/marlin_gemm.cpp:6-9), argument for argument:
 *   A          fp16 [m, k] row-major, 16-byte aligned                      (device)
 *   B          int32 [k/16, 2n]  Marlin-packed 4-bit codes, zero-point 8   (device)
 *   C          fp16 [m, n] row-major, 16-byte aligned, overwritten         (device)
 *   s          fp16 [k/groupsize, n] (groupsize 128) or [1, n] (groupsize -1), Marlin-permuted (device)
 *   workspace  int32, >= w4a16_workspace_ints(n, max_par) entries, all zero on entry; left all zero
 *   groupsize  128 or -1 (one scale per output column)
 *   dev        ordinal of the CUDA device the pointers live on; must be the current device
 *   stream     cudaStream_t passed as void*
 *   thread_k, thread_n   -1 for automatic, else one of the reference's tile pairs (128,128) / (64,256):
 *              they keep the reference's divisibility and dispatch meaning (same error codes) although
 *              the sm_100a kernel picks its own tiling
 *   sms        CTAs to launch, -1 for one per SM (clamped to the SM count of the device)
 *   max_par    kept for workspace sizing compatibility
 * Enqueues on `stream` and returns; 0 at once when m, n or k is 0 (marlin_cute_kernel.cu:59-60).
 * Scratch beyond the caller's workspace (fp32 partial tiles of the stream-K fix-up) is owned by the
 * library and cached per (device, stream), sized by need: the first use on a (device, stream) calls cudaMalloc
 * for SMs x 64 x 128 fp32 (4.8 MB on a 148-SM B200), which covers every batch of up to 64 rows; batch tiles of
 * 128 / 192 rows grow it once to at most SMs x 192 x 128 fp32 (14.5 MB).  Growing allocates, which CUDA refuses
 * during stream capture: run a problem of each batch size once before capturing it.  A block that was outgrown
 * stays allocated (captured launches may point at it) until w4a16_release_stream.
 * Numerics: products are accumulated in fp32.  For m <= 16 with group scales the kernel accumulates the exact
 * integer weights (q - 8) per 128-k group and applies the fp16 group scale in fp32 afterwards; the reference
 * rounds (q - 8) * s to fp16 first (gemm/marlin_gemm/marlin_cute_trait.h:656-664), as this library does for larger m.
 * The two differ by that rounding only (relative 2^-11 per weight).
 * Stream order holds for A, C, workspace and the scratch.  B and s are treated as parameters: when the
 * previous kernel on `stream` is another GEMM of this library, this one may prefetch B and s while that
 * one is still finishing (programmatic dependent launch), so B and s must not be that GEMM's output.
 * W4A16_PDL=0 in the environment restores plain stream order for everything.
 */
int w4a16_marlin_gemm(const void *A, const void *B, void *C, const void *s, int prob_m, int prob_n, int prob_k,
                      void *workspace, int groupsize, int dev, void *stream, int thread_k, int thread_n, int sms,
                      int max_par);

/*
 * The same GEMM for callers that cannot let a library allocate device memory.  It has no counterpart in the
 * reference (whose launcher never needs scratch beyond the caller's workspace, because it keeps fp16 partial
 * sums in C).
 *
 * Who needs it: a process whose framework allocator has already reserved the whole device, so that a raw
 * cudaMalloc made by this library fails with out-of-memory or eats into memory the framework believes it
 * owns; a latency-critical loop, where cudaMalloc / cudaFree stall every stream of the device while they run;
 * and callers whose memory budget is audited, where a library-owned cache of 5 to 15 MB per stream is not acceptable.
 * w4a16_marlin_gemm allocates its fix-up scratch on the first call of every (device, stream) pair; this entry
 * point never calls cudaMalloc, cudaFree or any allocating routine.  Its scratch is a 5 MiB array compiled
 * into the library (every GPU that loads the library holds it until the process exits).
 *
 * Arguments, results and return codes are those of w4a16_marlin_gemm, with these differences:
 *   - prob_m <= 64 only, and at most 160 CTAs (any sm_100 part today); beyond that it returns W4A16_ERR_ARG and
 *     w4a16_last_cuda_error() says which limit was hit.  Larger batches must use w4a16_marlin_gemm.
 *   - The first call on a device looks up the device address of the built-in array (cudaGetSymbolAddress),
 *     puts the array into its idle state on `stream` and synchronises `stream`.  Make that first call before
 *     any stream capture begins.  On EVERY call `dev` must be the current device (checked: W4A16_ERR_ARG
 *     otherwise), because the array's address on one device means nothing on another.
 *   - All calls on one device share the one array.  Each call leaves it in the idle state, so back-to-back
 *     calls on ONE stream are fine; two calls that overlap on the GPU (different streams, or different host
 *     threads feeding different streams) race on it and produce garbage.  Serialise them.
 *   - A bounded wait that runs out is reported by w4a16_device_status(dev, stream), which then also restores
 *     the idle state.
 */
int w4a16_marlin_gemm_builtin_scratch(const void *A, const void *B, void *C, const void *s, int prob_m, int prob_n,
                                      int prob_k, void *workspace, int groupsize, int dev, void *stream, int thread_k,
                                      int thread_n, int sms, int max_par);

/*
 * w4a16_marlin_gemm for callers whose activations and outputs live in HOST memory (pinned, for the copies to
 * be asynchronous): enqueues on `stream` the copy of A_host [m, k] into the device staging buffer A_stage, the
 * GEMM (automatic tiles), and the copy of the result from the device staging buffer C_stage [m, n] into
 * C_host.  B, s, workspace, A_stage and C_stage are device pointers owned by the caller (the weights stay
 * resident, as the reference's Layer keeps them, gemm/marlin_gemm/marlin.py:82-85).  It is the host-tensor
 * form of the reference's  mul()  (gemm/marlin_gemm/marlin.py:11-24), which the reference only offers for
 * device tensors.  Returns like w4a16_marlin_gemm; the caller synchronises `stream` before reading C_host.
 * With W4A16_HOST_DIRECT=1 in the environment, page-locked host buffers and prob_m <= 64, the copies do not go through
 * the copy engines (about ten microseconds of stream time each, more than a decode GEMM): a small kernel reads A_host
 * over PCIe into A_stage while the GEMM behind it already prefetches its weights, and the GEMM writes its result rows
 * straight into C_host; C_stage is then not touched.  It pays on a single stream (layers run one after the other) and
 * costs where several streams already overlap copies with kernels, hence opt-in.
 */
int w4a16_marlin_gemm_host(const void *A_host, const void *B, void *C_host, const void *s, int prob_m, int prob_n,
                           int prob_k, void *workspace, int groupsize, int dev, void *stream, void *A_stage,
                           void *C_stage);


/* ---- column-sharded GEMM with a gathering epilogue (one process per GPU).  The reference is single-GPU and has
 * no counterpart; the shard rule follows from its layout (gemm/marlin_gemm/marlin.py:29-57: both permutations stay
 * inside 64-column blocks).
 *
 * Rank `rank` of `world` (<= 8) holds columns [rank*n_local, (rank+1)*n_local) of the layer (B, s as produced by
 * w4a16_shard_columns).  dst[r] is an fp16 [m, world*n_local] row-major buffer in GPU r's memory, as addressable
 * from THIS process: dst[rank] is local, the others come from w4a16_peer_open.  The kernel's epilogue writes every
 * finished tile into its columns of ALL world buffers with plain stores (peer memory is never read and never the
 * source of a TMA copy), so the transfer over NVLink overlaps the main loop tile by tile and no separate all-gather
 * runs.  A rank may read the other ranks' columns of its own buffer only after w4a16_peer_barrier on the same
 * stream, and must not start the next gathering GEMM into the same buffers before every rank has finished reading
 * (barrier again, or alternate two sets of buffers).  Return codes as w4a16_marlin_gemm (n_local plays prob_n). */
int w4a16_marlin_gemm_gather(const void *A, const void *B, const void *s, int prob_m, int n_local, int prob_k,
                             void *workspace, int groupsize, int dev, void *stream, void *const *dst, int world,
                             int rank);

/* Device memory that other processes of this machine can map.  w4a16_peer_alloc: cudaMalloc on the current device,
 * zero-filled, plus its 64-byte inter-process handle (pass it to the other ranks by any host channel).
 * w4a16_peer_open: maps another process's buffer for the current device and enables peer access to its GPU
 * (cudaIpcOpenMemHandle); never call it on a handle of the own process.  Close what was opened before the owner
 * frees it. */
int w4a16_peer_alloc(size_t bytes, void **dptr, void *handle64);
int w4a16_peer_open(const void *handle64, void **dptr);
int w4a16_peer_close(void *dptr);
int w4a16_peer_free(void *dptr);

/* Stream-ordered barrier over the ranks' GPUs: enqueues a one-warp kernel that announces this rank's next epoch in
 * every rank's flag block and waits (at most limit_ms, 1..5000) until every rank has announced it here.  flags[r]
 * = rank r's flag block: 64 bytes, 64-byte aligned, zero when first used (w4a16_peer_alloc zero-fills), mapped like
 * dst above.  Work enqueued on `stream` before the call is complete and visible on all ranks when the barrier
 * kernel of each rank ends.  The epoch counter lives in the flag block, so a captured barrier can be replayed.
 * Every rank must run its barrier kernel on its own GPU; never two ranks on one GPU.  A wait that runs out is
 * reported by w4a16_device_status(dev, stream) as W4A16_ERR_TIMEOUT; the flag blocks must then be zeroed again by
 * all ranks before further use. */
int w4a16_peer_barrier(void *const *flags, int world, int rank, int dev, void *stream, int limit_ms);

/* Size rule of the caller's lock array: n / 128 * max_par  (gemm/marlin_gemm/marlin_gemm.cpp:29-31,
 * gemm/marlin_gemm/marlin.py:85). */
int w4a16_workspace_ints(int prob_n, int max_par);

/* Synchronises `stream` and returns W4A16_OK, or W4A16_ERR_TIMEOUT when a kernel launched on
 * (dev, stream) since the last call gave up a bounded wait (its output is then undefined), or
 * W4A16_ERR_CUDA.  The reference has no counterpart: its fix-up spin is unbounded
 * (include/barrier.h:85-96). */
int w4a16_device_status(int dev, void *stream);

/* Which kernel a call of w4a16_marlin_gemm with these sizes would launch on a device of `device_sms` SMs, and how the
 * work would be cut.  Pure host arithmetic: no CUDA call, no device needed.  `sms` as in w4a16_marlin_gemm.  Returns
 * the code that call would return for the sizes (W4A16_OK, or the shape errors); for an empty problem `kernel` is
 * W4A16_KERNEL_NONE.  The cluster form is planned as if every cluster could be resident at once (the launch itself
 * asks cudaOccupancyMaxActiveClusters and falls back to smaller clusters or stream-K).  The reference's counterpart
 * is the dispatch table at the end of its launcher (gemm/marlin_gemm/marlin_cute_kernel.cu:62-115), which is not
 * callable by itself. */
#define W4A16_KERNEL_NONE 0
#define W4A16_KERNEL_SINGLE 1         /* one CTA per worker, stream-K */
#define W4A16_KERNEL_PAIRS 2          /* one CTA pair per worker (256 weight columns per tile) */
#define W4A16_KERNEL_DECODE 3         /* prob_m <= 16: one CTA per worker, stream-K or one whole tile each */
#define W4A16_KERNEL_DECODE_CLUSTER 4 /* prob_m <= 16: one cluster per 128-column tile */
typedef struct {
  int kernel;            /* W4A16_KERNEL_* */
  int tile_rows;         /* batch rows per tile */
  int k_per_stage;       /* k per pipeline stage */
  int workers;           /* CTAs (pairs: CTA pairs) launched */
  int ctas_per_worker;   /* 1, 2 for pairs; for the cluster form the cluster size, `workers` counting CTAs */
  int whole_tile_waves;  /* pairs: waves of whole tiles before the stream-K part */
  int stages_per_worker; /* k-stages per worker in the stream-K part (the cluster form: per CTA) */
} w4a16_plan_t;
int w4a16_plan(int prob_m, int prob_n, int prob_k, int groupsize, int sms, int device_sms, w4a16_plan_t *out);

/* Frees the scratch and status word the library keeps for (dev, stream), after synchronising `stream`.  No launch
 * captured in a CUDA graph on that stream may be replayed afterwards.  The reference has no counterpart (it owns
 * no memory).  Returns W4A16_OK also when nothing was kept. */
int w4a16_release_stream(int dev, void *stream);

/* Self-test of the bounded device-side waits (the reference has none: its fix-up spin is unbounded,
 * include/barrier.h:85-96).  Launches the GEMM so that one CTA waits for a partial tile that no CTA will ever
 * write; after limit_ms (1..5000) the kernel gives up, unwinds and returns.  The call itself returns W4A16_OK;
 * w4a16_device_status(dev, stream) then returns W4A16_ERR_TIMEOUT and restores the scratch, after which the
 * stream is usable as before.  C is left undefined.  Injects no GPU fault.  A negative limit_ms runs the same on the
 * built-in array of w4a16_marlin_gemm_builtin_scratch (prob_m <= 64) for -limit_ms milliseconds. */
int w4a16_selftest_unanswered_wait(const void *A, const void *B, void *C, const void *s, int prob_m, int prob_n,
                                   int prob_k, int groupsize, int dev, void *stream, int limit_ms);

/* Text of the last CUDA error seen by this library on the calling thread ("" if none). */
const char *w4a16_last_cuda_error(void);

/* Diagnostic twin of w4a16_marlin_gemm on plain CUDA cores (one thread per output element, reads the
 * packed layout through its closed form).  Same arguments and return codes.  Never selected
 * automatically; used by the tests to cross-check the tensor-core kernel on the device. */
int w4a16_marlin_gemm_simt(const void *A, const void *B, void *C, const void *s, int prob_m, int prob_n,
                           int prob_k, void *workspace, int groupsize, int dev, void *stream, int thread_k,
                           int thread_n, int sms, int max_par);

/* ---- host-side weight packer (all pointers are HOST memory) -------------------------------- */

/* codes q (uint8 0..15) [k, n] row-major -> B int32 [k/16, 2n].  Replaces the permute + nibble-pack half
 * of Layer.pack, gemm/marlin_gemm/marlin.py:119-129.  k % 16 == 0, n % 64 == 0. */
int w4a16_pack_weights(const uint8_t *q, int k, int n, int32_t *B);
/* Inverse of w4a16_pack_weights. */
int w4a16_unpack_weights(const int32_t *B, int k, int n, uint8_t *q);
/* fp16 scales [groups, n] natural column order -> kernel order.  groups > 1: 64-column blocks
 * (_scale_perm); groups == 1: 32-column blocks (_scale_perm_single).  marlin.py:49-54,111-118. */
int w4a16_permute_scales(const uint16_t *s, int groups, int n, uint16_t *s_packed);
int w4a16_unpermute_scales(const uint16_t *s_packed, int groups, int n, uint16_t *s);
/* All of Layer.pack (gemm/marlin_gemm/marlin.py:92-131): weight fp16 [n, k] (the nn.Linear layout),
 * scales fp16 [k/groupsize or 1, n]  ->  round(w/s)+8 clamped to 0..15, packed B and permuted s. */
int w4a16_quantize_pack(const uint16_t *weight_nk, const uint16_t *scales, int k, int n, int groupsize, int32_t *B,
                        uint16_t *s_packed);
/* Column shard `rank` of `world` of a packed layer: B_shard int32 [k/16, 2n/world], s_shard
 * [groups, n/world].  n/world must be a multiple of 128.  No counterpart in the reference (it is single
 * GPU); valid because both permutations are local to 64-column blocks. */
int w4a16_shard_columns(const int32_t *B, const uint16_t *s_packed, int k, int n, int groups, int rank, int world,
                        int32_t *B_shard, uint16_t *s_shard);

/* Layer.pack on the DEVICE (gemm/marlin_gemm/marlin.py:92-131 runs it with numpy on the host): weight fp16 [n, k]
 * and scales fp16 [k/groupsize or 1, n] in device memory -> B int32 [k/16, 2n] and s_packed in device memory,
 * enqueued on `stream`.  Bit-exact with w4a16_quantize_pack. */
int w4a16_quantize_pack_device(const void *weight_nk, const void *scales, int k, int n, int groupsize, void *B,
                               void *s_packed, void *stream);

/* ---- packed layers on disk (host pointers).  The reference keeps packed layers only as torch buffers
 * (gemm/marlin_gemm/marlin.py:82-83); these give them a file form: 64-byte header, B, s.  Reading takes column
 * shard `rank` of `world` straight from the file (1, 0 reads the whole layer). */
int w4a16_blob_write(const char *path, const int32_t *B, const uint16_t *s_packed, int k, int n, int groupsize);
int w4a16_blob_info(const char *path, int *k, int *n, int *groupsize, int *groups);
int w4a16_blob_read(const char *path, int rank, int world, int32_t *B_shard, uint16_t *s_shard);

#ifdef __cplusplus
}
#endif
#endif /* W4A16_H_ */
