/*
 * CPU oracle for the W4A16 (fp16 activation x Marlin-packed int4 weight) GEMM path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or calls
 * this file; it is the checker the parity tests, the smoke test and the bench's
 * CPU-baseline leg compare the CUDA path against.
 *
 * It restates, in plain C, the algorithm the reference spells in Python:
 *   - the Marlin permutation tables      gemm/marlin_gemm/marlin.py:29-57   (_get_perms)
 *   - quantise + permute + nibble pack   gemm/marlin_gemm/marlin.py:92-131  (Layer.pack)
 *   - dequantise  ref = (w - 8).half()*s gemm/marlin_gemm/marlin_test.py:22-31
 *   - GEMM        C_ref = A @ ref        gemm/marlin_gemm/marlin_test.py:64
 *     (accumulated in fp32, the accumulation type of the reference kernel,
 *      gemm/marlin_gemm/marlin_cute_trait.h:74)
 *
 * Parity pin: the reference holds no numeric fixtures for this path (its accuracy
 * assertion is commented out, marlin_test.py:75).  The pin is therefore made from the
 * reference's own Python packer run on CPU: tests/golden/make_golden.py imports
 * marlin.py, runs Layer.pack and torch matmul on seeded inputs and stores the outputs;
 * tests/test_oracle.py checks every function below against those vectors, bit-exact for
 * the integer work.
 *
 * fp16 values cross this interface as raw uint16_t bit patterns.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- fp16 <-> fp32, software, round-to-nearest-even (no dependence on F16C) ---- */
static inline float h2f(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else { /* subnormal: normalise */
      int e = -1;
      do { man <<= 1; e++; } while (!(man & 0x400u));
      man &= 0x3ffu;
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static inline uint16_t f2h(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  x &= 0x7fffffffu;
  if (x >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | ((x > 0x7f800000u) ? 0x200u : 0)); /* inf/nan */
  if (x >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);                                     /* overflow */
  if (x < 0x33000001u) return (uint16_t)sign;                                                  /* underflow to 0 */
  int32_t e = (int32_t)(x >> 23) - 127;
  uint32_t m = (x & 0x7fffffu) | 0x800000u;
  uint32_t shift, half;
  if (e < -14) { /* subnormal result */
    shift = (uint32_t)(13 + (-14 - e));
    uint32_t r = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    half = 1u << (shift - 1);
    if (rem > half || (rem == half && (r & 1u))) r++;
    return (uint16_t)(sign | r);
  }
  uint32_t r = ((uint32_t)(e + 15) << 10) | ((m >> 13) & 0x3ffu);
  uint32_t rem = m & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) r++;
  return (uint16_t)(sign | r);
}

void oracle_half_to_float(const uint16_t *h, float *f, long n) {
  for (long i = 0; i < n; i++) f[i] = h2f(h[i]);
}
void oracle_float_to_half(const float *f, uint16_t *h, long n) {
  for (long i = 0; i < n; i++) h[i] = f2h(f[i]);
}

/* ---- permutation tables: marlin.py:29-57 -------------------------------------- */
void oracle_get_perms(int *perm /*1024*/, int *scale_perm /*64*/, int *scale_perm_single /*32*/) {
  int tmp[1024];
  int cnt = 0;
  for (int i = 0; i < 32; i++) {           /* marlin.py:31 */
    int perm1[8];
    int c1 = 0;
    int col = i / 4;
    for (int block = 0; block < 2; block++) {
      int rows[4] = {2 * (i % 4), 2 * (i % 4) + 1, 2 * (i % 4 + 4), 2 * (i % 4 + 4) + 1};
      for (int r = 0; r < 4; r++) perm1[c1++] = 16 * rows[r] + col + 8 * block; /* :41 */
    }
    for (int j = 0; j < 4; j++)
      for (int p = 0; p < 8; p++) tmp[cnt++] = perm1[p] + 256 * j;              /* :42-43 */
  }
  static const int interleave[8] = {0, 2, 4, 6, 1, 3, 5, 7};                     /* :46 */
  for (int g = 0; g < 128; g++)
    for (int p = 0; p < 8; p++) perm[g * 8 + p] = tmp[g * 8 + interleave[p]];    /* :47 */
  cnt = 0;
  for (int i = 0; i < 8; i++)
    for (int j = 0; j < 8; j++) scale_perm[cnt++] = i + 8 * j;                   /* :49-51 */
  cnt = 0;
  static const int offs[8] = {0, 1, 8, 9, 16, 17, 24, 25};
  for (int i = 0; i < 4; i++)
    for (int j = 0; j < 8; j++) scale_perm_single[cnt++] = 2 * i + offs[j];      /* :52-54 */
}

/* ---- weight pack: marlin.py:119-129 -------------------------------------------
 * q: codes 0..15, row-major [k][n].  B: int32 row-major [k/16][2n].              */
int oracle_pack_weights(const uint8_t *q, int k, int n, int32_t *B) {
  if (k % 16 || n % 64) return 1;
  int perm[1024], sp[64], sps[32];
  oracle_get_perms(perm, sp, sps);
  const long rowlen = (long)n * 16; /* elements in one row of the 16x16-tiled matrix */
  int32_t *tiled = (int32_t *)malloc(sizeof(int32_t) * rowlen);
  int32_t *res = (int32_t *)malloc(sizeof(int32_t) * rowlen);
  if (!tiled || !res) { free(tiled); free(res); return 3; }
  for (int kt = 0; kt < k / 16; kt++) {
    /* w.reshape(k/16,16,n/16,16).permute(0,2,1,3).reshape(k/16, n*16)   (:119-121) */
    for (int nt = 0; nt < n / 16; nt++)
      for (int kr = 0; kr < 16; kr++)
        for (int nr = 0; nr < 16; nr++)
          tiled[(long)nt * 256 + kr * 16 + nr] = q[(long)(kt * 16 + kr) * n + nt * 16 + nr];
    /* res.reshape(-1, 1024)[:, perm]                                     (:123) */
    for (long blk = 0; blk < rowlen / 1024; blk++)
      for (int p = 0; p < 1024; p++) res[blk * 1024 + p] = tiled[blk * 1024 + perm[p]];
    /* q |= res[:, i::8] << 4*i                                           (:125-128) */
    for (long c = 0; c < rowlen / 8; c++) {
      uint32_t w = 0;
      for (int i = 0; i < 8; i++) w |= ((uint32_t)res[c * 8 + i] & 0xfu) << (4 * i);
      B[(long)kt * (rowlen / 8) + c] = (int32_t)w;
    }
  }
  free(tiled);
  free(res);
  return 0;
}

/* inverse of oracle_pack_weights (same tables, walked backwards) */
int oracle_unpack_weights(const int32_t *B, int k, int n, uint8_t *q) {
  if (k % 16 || n % 64) return 1;
  int perm[1024], sp[64], sps[32];
  oracle_get_perms(perm, sp, sps);
  const long rowlen = (long)n * 16;
  for (int kt = 0; kt < k / 16; kt++)
    for (long e = 0; e < rowlen; e++) {
      uint32_t w = (uint32_t)B[(long)kt * (rowlen / 8) + e / 8];
      uint8_t code = (w >> (4 * (e % 8))) & 0xfu;
      long blk = e / 1024;
      int src = perm[e % 1024];        /* position in the 16x16-tiled row */
      long t = blk * 1024 + src;
      int nt = (int)(t / 256), kr = (int)(t % 256) / 16, nr = (int)(t % 16);
      q[(long)(kt * 16 + kr) * n + nt * 16 + nr] = code;
    }
  return 0;
}

/* ---- scale permutation: marlin.py:111-118 --------------------------------------
 * s: fp16 [groups][n] in natural column order.  groups > 1 (grouped) uses
 * _scale_perm over 64-column blocks; groups == 1 (per-channel) uses
 * _scale_perm_single over 32-column blocks.                                     */
int oracle_permute_scales(const uint16_t *s, int groups, int n, uint16_t *out) {
  int perm[1024], sp[64], sps[32];
  oracle_get_perms(perm, sp, sps);
  const int *p = groups > 1 ? sp : sps;
  const int len = groups > 1 ? 64 : 32;
  if (n % len) return 1;
  for (long g = 0; g < groups; g++)
    for (int b = 0; b < n / len; b++)
      for (int i = 0; i < len; i++) out[g * n + b * len + i] = s[g * n + b * len + p[i]];
  return 0;
}
int oracle_unpermute_scales(const uint16_t *sp_in, int groups, int n, uint16_t *out) {
  int perm[1024], sp[64], sps[32];
  oracle_get_perms(perm, sp, sps);
  const int *p = groups > 1 ? sp : sps;
  const int len = groups > 1 ? 64 : 32;
  if (n % len) return 1;
  for (long g = 0; g < groups; g++)
    for (int b = 0; b < n / len; b++)
      for (int i = 0; i < len; i++) out[g * n + b * len + p[i]] = sp_in[g * n + b * len + i];
  return 0;
}

/* ---- quantiser: marlin.py:108-110 ----------------------------------------------
 * w: fp16 [k][n] (already transposed linear.weight), s: fp16 [groups][n] natural.
 * code = clamp(round_half_even(fp16(w / s)) + 8, 0, 15); the division is an fp16
 * division (torch computes half/half in fp32 and rounds to half).               */
static inline float rint_even(float x) {
  float r = (float)(long)x;
  float d = x - r;
  if (d > 0.5f || (d == 0.5f && ((long)r & 1))) r += 1.0f;
  else if (d < -0.5f || (d == -0.5f && ((long)r & 1))) r -= 1.0f;
  return r;
}
int oracle_quantize(const uint16_t *w, const uint16_t *s, int k, int n, int groupsize, uint8_t *q) {
  int g = groupsize == -1 ? k : groupsize;
  if (k % g) return 1;
  for (long kk = 0; kk < k; kk++)
    for (long nn = 0; nn < n; nn++) {
      float quo = h2f(f2h(h2f(w[kk * n + nn]) / h2f(s[(kk / g) * n + nn])));
      int c = (int)rint_even(quo) + 8;
      q[kk * n + nn] = (uint8_t)(c < 0 ? 0 : (c > 15 ? 15 : c));
    }
  return 0;
}

/* ---- dequantise: marlin_test.py:31  ref = (w - 8).half() * s  (fp16 product) ---- */
int oracle_dequant(const uint8_t *q, const uint16_t *s, int k, int n, int groupsize, uint16_t *ref) {
  int g = groupsize == -1 ? k : groupsize;
  if (k % g) return 1;
#pragma omp parallel for schedule(static)
  for (long kk = 0; kk < k; kk++)
    for (long nn = 0; nn < n; nn++) {
      float v = (float)((int)q[kk * n + nn] - 8) * h2f(s[(kk / g) * n + nn]);
      ref[kk * n + nn] = f2h(v); /* product of two fp16 values is exact in fp32; one rounding */
    }
  return 0;
}

/* ---- GEMM: marlin_test.py:64, fp32 accumulation --------------------------------
 * C[m][n] (fp32) = sum_k A[m][k] * ref[k][n]; runs over [n_begin, n_end) columns so the
 * tests can check a column window of a large problem.                           */
__attribute__((target_clones("avx512f", "avx2", "default")))
static void gemm_rows(const float *Af, const float *Wf, int m, int k, long ldw, long ncols, float *C, long ldc) {
  /* Wf: [k][ncols] window, C: [m][ncols] window.  Row blocks of 16 keep the C block in L1 while the
   * weight window streams through once per block. */
  for (int i0 = 0; i0 < m; i0 += 16) {
    const int i1 = i0 + 16 < m ? i0 + 16 : m;
    for (int i = i0; i < i1; i++) {
      float *c = C + (long)i * ldc;
      for (long j = 0; j < ncols; j++) c[j] = 0.0f;
    }
    for (int kk = 0; kk < k; kk++) {
      const float *w = Wf + (long)kk * ldw;
      for (int i = i0; i < i1; i++) {
        const float a = Af[(long)i * k + kk];
        float *c = C + (long)i * ldc;
        for (long j = 0; j < ncols; j++) c[j] += a * w[j];
      }
    }
  }
}

int oracle_gemm(const uint16_t *A, const uint8_t *q, const uint16_t *s, int m, int n, int k, int groupsize,
                float *C) {
  int g = groupsize == -1 ? k : groupsize;
  if (k % g) return 1;
  if (m == 0 || n == 0 || k == 0) return 0;
  float *Af = (float *)malloc(sizeof(float) * (size_t)m * k);
  if (!Af) return 3;
  for (long i = 0; i < (long)m * k; i++) Af[i] = h2f(A[i]);
  const long CB = 256; /* column block per task */
  const long nblk = (n + CB - 1) / CB;
#pragma omp parallel
  {
    float *Wf = (float *)malloc(sizeof(float) * (size_t)k * CB);
#pragma omp for schedule(dynamic)
    for (long b = 0; b < nblk; b++) {
      long n0 = b * CB, nc = (n0 + CB <= n) ? CB : (n - n0);
      for (long kk = 0; kk < k; kk++)
        for (long j = 0; j < nc; j++) {
          float v = (float)((int)q[kk * n + n0 + j] - 8) * h2f(s[(kk / g) * n + n0 + j]);
          Wf[kk * CB + j] = h2f(f2h(v));
        }
      gemm_rows(Af, Wf, m, k, CB, nc, C + n0, n);
    }
    free(Wf);
  }
  free(Af);
  return 0;
}

/* Same GEMM, but starting from the PACKED operands the kernel receives
 * (B Marlin-packed, s permuted): unpacks with the inverse tables, then calls oracle_gemm. */
int oracle_gemm_packed(const uint16_t *A, const int32_t *B, const uint16_t *s_packed, int m, int n, int k,
                       int groupsize, float *C) {
  int g = groupsize == -1 ? k : groupsize;
  if (k % g || k % 16 || n % 64) return 1;
  if (m == 0 || n == 0 || k == 0) return 0;
  int groups = k / g;
  uint8_t *q = (uint8_t *)malloc((size_t)k * n);
  uint16_t *s = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)groups * n);
  if (!q || !s) { free(q); free(s); return 3; }
  int rc = oracle_unpack_weights(B, k, n, q);
  if (!rc) rc = oracle_unpermute_scales(s_packed, groups, n, s);
  if (!rc) rc = oracle_gemm(A, q, s, m, n, k, groupsize, C);
  free(q);
  free(s);
  return rc;
}

/* Worker threads of the loops above.  A launcher may have exported OMP_NUM_THREADS=1 for its ranks (torchrun does);
 * the CPU-baseline leg calls this with the host's core count so that it is timed on the same cores at every
 * number of GPUs. */
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
