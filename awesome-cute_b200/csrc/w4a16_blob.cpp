// On-disk form of a packed layer: one little-endian file = 64-byte header + B (int32 [k/16][2n]) + s (fp16
// [groups][n], kernel order).  Reading can take a column shard directly (rank r of G), which is a strided read:
// both Marlin permutations are local to 64-column blocks.  The reference keeps packed layers only as torch buffers
// (gemm/marlin_gemm/marlin.py:82-83); this is the file-level counterpart.
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "../../include/w4a16.h"

namespace {
struct Header {
  char magic[8];        // "W4A16MRL"
  uint32_t version;     // 1
  int32_t k, n, groupsize, groups;
  uint32_t reserved[9];
};
static_assert(sizeof(Header) == 64, "header is 64 bytes");

bool read_header(FILE *f, Header &h) {
  if (std::fread(&h, sizeof(h), 1, f) != 1) return false;
  if (std::memcmp(h.magic, "W4A16MRL", 8) != 0 || h.version != 1) return false;
  if (h.k <= 0 || h.n <= 0 || h.k % 16 || h.n % 64 || h.groups < 1) return false;
  return true;
}
}  // namespace

extern "C" int w4a16_blob_write(const char *path, const int32_t *B, const uint16_t *s_packed, int k, int n,
                                int groupsize) {
  if (!path || !B || !s_packed) return W4A16_ERR_ARG;
  if (groupsize != -1 && groupsize != 128) return W4A16_ERR_KERN_SHAPE;
  if (k <= 0 || n <= 0 || k % 16 || n % 64 || (groupsize == 128 && k % 128)) return W4A16_ERR_PROB_SHAPE;
  Header h{};
  std::memcpy(h.magic, "W4A16MRL", 8);
  h.version = 1;
  h.k = k, h.n = n, h.groupsize = groupsize, h.groups = groupsize == -1 ? 1 : k / groupsize;
  FILE *f = std::fopen(path, "wb");
  if (!f) return W4A16_ERR_ARG;
  const size_t nb = (size_t)(k / 16) * 2 * n, ns = (size_t)h.groups * n;
  const bool ok = std::fwrite(&h, sizeof(h), 1, f) == 1 && std::fwrite(B, sizeof(int32_t), nb, f) == nb &&
                  std::fwrite(s_packed, sizeof(uint16_t), ns, f) == ns;
  return (std::fclose(f) == 0 && ok) ? W4A16_OK : W4A16_ERR_ARG;
}

extern "C" int w4a16_blob_info(const char *path, int *k, int *n, int *groupsize, int *groups) {
  if (!path) return W4A16_ERR_ARG;
  FILE *f = std::fopen(path, "rb");
  if (!f) return W4A16_ERR_ARG;
  Header h;
  const bool ok = read_header(f, h);
  std::fclose(f);
  if (!ok) return W4A16_ERR_ARG;
  if (k) *k = h.k;
  if (n) *n = h.n;
  if (groupsize) *groupsize = h.groupsize;
  if (groups) *groups = h.groups;
  return W4A16_OK;
}

extern "C" int w4a16_blob_read(const char *path, int rank, int world, int32_t *B_shard, uint16_t *s_shard) {
  if (!path || !B_shard || !s_shard || world < 1 || rank < 0 || rank >= world) return W4A16_ERR_ARG;
  FILE *f = std::fopen(path, "rb");
  if (!f) return W4A16_ERR_ARG;
  Header h;
  if (!read_header(f, h)) { std::fclose(f); return W4A16_ERR_ARG; }
  if (h.n % world || (h.n / world) % 128) { std::fclose(f); return W4A16_ERR_PROB_SHAPE; }
  const long ns = h.n / world, n0 = ns * rank;
  bool ok = true;
  for (long r = 0; r < h.k / 16 && ok; ++r) {   // row r of B: 2n int32; the shard is columns [2 n0, 2 n0 + 2 ns)
    ok = std::fseek(f, (long)sizeof(Header) + (r * 2L * h.n + 2 * n0) * 4, SEEK_SET) == 0 &&
         std::fread(B_shard + r * 2 * ns, sizeof(int32_t), (size_t)(2 * ns), f) == (size_t)(2 * ns);
  }
  const long s_base = (long)sizeof(Header) + (long)(h.k / 16) * 2L * h.n * 4;
  for (long g = 0; g < h.groups && ok; ++g) {
    ok = std::fseek(f, s_base + (g * (long)h.n + n0) * 2, SEEK_SET) == 0 &&
         std::fread(s_shard + g * ns, sizeof(uint16_t), (size_t)ns, f) == (size_t)ns;
  }
  std::fclose(f);
  return ok ? W4A16_OK : W4A16_ERR_ARG;
}
