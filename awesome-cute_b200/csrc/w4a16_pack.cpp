// Host-side Marlin weight packer / unpacker / column shard slicer (C ABI in include/w4a16.h).
//
// The reference builds the layout from gather tables (gemm/marlin_gemm/marlin.py:29-57,119-129).
// This file uses the closed form of the same layout instead.  Packed word B[r][c] with
//   c = 128*blk + 4*lane + j          (blk: 64-column block, lane 0..31, j 0..3)
// holds in nibble i (bits 4i..4i+3) the code of weight W[kk][nn] with
//   nn = 64*blk + 16*j + lane/4 + 8*((i>>1)&1)
//   kk = 16*r + 2*(lane%4) + (i>>2) + 8*(i&1)
// i.e. lane/j/i address one mma.m16n8k16 B fragment; the sm_100a kernel reads the same words but
// assigns one weight column per thread (see w4a16_gemm.cu).
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#include "../../include/w4a16.h"

namespace {

inline float half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400u));
      bits = sign | ((uint32_t)(112 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

inline uint16_t float_to_half(float f) {  // round to nearest even
  uint32_t x;
  std::memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  x &= 0x7fffffffu;
  if (x >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (x > 0x7f800000u ? 0x200u : 0u));
  if (x >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);
  if (x < 0x33000001u) return (uint16_t)sign;
  int e = (int)(x >> 23) - 127;
  uint32_t m = (x & 0x7fffffu) | 0x800000u;
  if (e < -14) {
    uint32_t shift = (uint32_t)(13 + (-14 - e));
    uint32_t r = m >> shift, rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (r & 1u))) ++r;
    return (uint16_t)(sign | r);
  }
  uint32_t r = ((uint32_t)(e + 15) << 10) | ((m >> 13) & 0x3ffu), rem = m & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) ++r;
  return (uint16_t)(sign | r);
}

// position of natural column `col` inside its permuted block
inline int group_scale_pos(int c64) { return 8 * (c64 % 8) + c64 / 8; }                   // _scale_perm inverse
inline int single_scale_pos(int c32) { return 8 * ((c32 % 8) / 2) + 2 * (c32 / 8) + c32 % 2; }  // _scale_perm_single inverse

}  // namespace

extern "C" int w4a16_pack_weights(const uint8_t *q, int k, int n, int32_t *B) {
  if (!q || !B) return W4A16_ERR_ARG;
  if (k < 0 || n < 0 || k % 16 || n % 64) return W4A16_ERR_PROB_SHAPE;
  const long row_words = 2L * n;
  for (long r = 0; r < k / 16; ++r)
    for (long c = 0; c < row_words; ++c) {
      const long blk = c / 128;
      const int lane = (int)(c % 128) / 4, j = (int)(c % 4);
      uint32_t w = 0;
      for (int i = 0; i < 8; ++i) {
        const long nn = 64 * blk + 16 * j + lane / 4 + 8 * ((i >> 1) & 1);
        const long kk = 16 * r + 2 * (lane % 4) + (i >> 2) + 8 * (i & 1);
        w |= ((uint32_t)q[kk * n + nn] & 0xfu) << (4 * i);
      }
      B[r * row_words + c] = (int32_t)w;
    }
  return W4A16_OK;
}

extern "C" int w4a16_unpack_weights(const int32_t *B, int k, int n, uint8_t *q) {
  if (!q || !B) return W4A16_ERR_ARG;
  if (k < 0 || n < 0 || k % 16 || n % 64) return W4A16_ERR_PROB_SHAPE;
  for (long kk = 0; kk < k; ++kk)
    for (long nn = 0; nn < n; ++nn) {
      const int kr = (int)(kk % 16), nr = (int)(nn % 64);
      const int lane = 4 * (nr % 8) + (kr % 8) / 2, j = nr / 16;
      const long c = 128 * (nn / 64) + 4 * lane + j;
      const int i = 4 * (kr % 2) + 2 * ((nr % 16) / 8) + kr / 8;
      q[kk * n + nn] = (uint8_t)(((uint32_t)B[(kk / 16) * 2L * n + c] >> (4 * i)) & 0xfu);
    }
  return W4A16_OK;
}

extern "C" int w4a16_permute_scales(const uint16_t *s, int groups, int n, uint16_t *out) {
  if (!s || !out) return W4A16_ERR_ARG;
  const int len = groups > 1 ? 64 : 32;
  if (groups < 1 || n < 0 || n % len) return W4A16_ERR_PROB_SHAPE;
  for (long g = 0; g < groups; ++g)
    for (long col = 0; col < n; ++col) {
      const long base = col - col % len;
      const int pos = groups > 1 ? group_scale_pos((int)(col % 64)) : single_scale_pos((int)(col % 32));
      out[g * n + base + pos] = s[g * n + col];
    }
  return W4A16_OK;
}

extern "C" int w4a16_unpermute_scales(const uint16_t *sp, int groups, int n, uint16_t *out) {
  if (!sp || !out) return W4A16_ERR_ARG;
  const int len = groups > 1 ? 64 : 32;
  if (groups < 1 || n < 0 || n % len) return W4A16_ERR_PROB_SHAPE;
  for (long g = 0; g < groups; ++g)
    for (long col = 0; col < n; ++col) {
      const long base = col - col % len;
      const int pos = groups > 1 ? group_scale_pos((int)(col % 64)) : single_scale_pos((int)(col % 32));
      out[g * n + col] = sp[g * n + base + pos];
    }
  return W4A16_OK;
}

extern "C" int w4a16_quantize_pack(const uint16_t *weight_nk, const uint16_t *scales, int k, int n, int groupsize,
                                   int32_t *B, uint16_t *s_packed) {
  if (!weight_nk || !scales || !B || !s_packed) return W4A16_ERR_ARG;
  if (groupsize != -1 && groupsize != 128) return W4A16_ERR_KERN_SHAPE;          // marlin.py:70-71
  if (k <= 0 || n <= 0 || k % 128 || n % 256) return W4A16_ERR_PROB_SHAPE;       // marlin.py:72-73
  const int g = groupsize == -1 ? k : groupsize;
  const int groups = k / g;
  std::vector<uint8_t> q((size_t)k * n);
  for (long kk = 0; kk < k; ++kk)
    for (long nn = 0; nn < n; ++nn) {
      // fp16 division (computed in fp32, rounded to fp16), round half to even, +8, clamp: marlin.py:108-110
      const float quo = half_to_float(float_to_half(half_to_float(weight_nk[nn * k + kk]) /
                                                    half_to_float(scales[(kk / g) * n + nn])));
      int code = (int)std::nearbyintf(quo) + 8;
      q[kk * n + nn] = (uint8_t)(code < 0 ? 0 : (code > 15 ? 15 : code));
    }
  int rc = w4a16_pack_weights(q.data(), k, n, B);
  if (rc) return rc;
  return w4a16_permute_scales(scales, groups, n, s_packed);
}

extern "C" int w4a16_shard_columns(const int32_t *B, const uint16_t *s_packed, int k, int n, int groups, int rank,
                                   int world, int32_t *B_shard, uint16_t *s_shard) {
  if (!B || !s_packed || !B_shard || !s_shard) return W4A16_ERR_ARG;
  if (world < 1 || rank < 0 || rank >= world || groups < 1) return W4A16_ERR_ARG;
  if (k % 16 || n % world || (n / world) % 128) return W4A16_ERR_PROB_SHAPE;
  const long ns = n / world, n0 = ns * rank;
  for (long r = 0; r < k / 16; ++r)
    std::memcpy(B_shard + r * 2 * ns, B + r * 2L * n + 2 * n0, sizeof(int32_t) * 2 * ns);
  for (long g = 0; g < groups; ++g) std::memcpy(s_shard + g * ns, s_packed + g * (long)n + n0, sizeof(uint16_t) * ns);
  return W4A16_OK;
}
