// Device-side Layer.pack: fake-quantised (or plain) fp16 weights + scales -> Marlin-packed int4 words and permuted
// scales, bit-exact with the host packer (w4a16_pack.cpp) and therefore with the reference's numpy packer
// (gemm/marlin_gemm/marlin.py:92-131).  One thread builds a packed word at a time: it gathers its eight weights
// through the closed form of the layout, quantises each as the reference does (fp16 division, round half to even,
// +8, clamp to 0..15; marlin.py:108-110) and ORs the nibbles together.  HBM-bound elementwise work: it reads 2 bytes
// and writes 0.5 byte per weight; nothing here is a GEMM.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/w4a16.h"

namespace {

// One block packs a tile of 128 k x 64 columns (one 64-column block of the layout, eight 16-k rows: 1024 words).
// The weights are [n][k] with k contiguous, so the tile is read as 64 rows of 256 contiguous bytes (16 bytes per
// thread and load, fully coalesced) into shared memory; the words are then gathered from there and written as eight
// runs of 512 contiguous bytes.  (Gathering the eight weights of a word straight from global memory touches sixteen
// different rows per warp, 32 bytes of each.)
constexpr int QT_K = 128, QT_N = 64, QT_LD = QT_K + 8;   // row pitch in halves: 272 bytes, keeps 16-byte alignment

__global__ void __launch_bounds__(256) quantize_pack_kernel(const __half *__restrict__ w_nk, const __half *__restrict__ scales,
                                                            int k, int n, int group, uint32_t *__restrict__ B) {
  __shared__ __align__(16) __half tile[QT_N * QT_LD];
  __shared__ __half sc[QT_N];
  const int k0 = blockIdx.x * QT_K, blk = blockIdx.y, n0 = blk * QT_N;
  // 64 rows x 16 chunks of 16 bytes = 1024 chunks, four per thread
  for (int q = threadIdx.x; q < QT_N * (QT_K / 8); q += 256) {
    const int row = q / (QT_K / 8), ch = q % (QT_K / 8);
    *reinterpret_cast<uint4 *>(&tile[row * QT_LD + ch * 8]) =
        *reinterpret_cast<const uint4 *>(&w_nk[(size_t)(n0 + row) * k + k0 + ch * 8]);
  }
  if (threadIdx.x < QT_N) sc[threadIdx.x] = scales[(size_t)(k0 / group) * n + n0 + threadIdx.x];   // group is 128 or k
  __syncthreads();
  // word (r, c): c = 4 * lane + j inside the block; nibble i holds column 16 j + lane / 4 + 8 ((i >> 1) & 1) at
  // k = 16 r + 2 (lane % 4) + (i >> 2) + 8 (i & 1)   (closed form of gemm/marlin_gemm/marlin.py:29-47)
  for (int wq = threadIdx.x; wq < (QT_K / 16) * 128; wq += 256) {
    const int r = wq / 128, c = wq % 128;
    const int lane = c / 4, j = c % 4;
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int nn = 16 * j + lane / 4 + 8 * ((i >> 1) & 1);
      const int kk = 16 * r + 2 * (lane % 4) + (i >> 2) + 8 * (i & 1);
      const float quo = __half2float(__float2half_rn(__half2float(tile[nn * QT_LD + kk]) / __half2float(sc[nn])));
      int code = (int)rintf(quo) + 8;
      code = code < 0 ? 0 : (code > 15 ? 15 : code);
      word |= (uint32_t)code << (4 * i);
    }
    B[(size_t)(k0 / 16 + r) * 2 * n + 128 * blk + c] = word;
  }
}

__global__ void permute_scales_kernel(const __half *__restrict__ s, int groups, int n, __half *__restrict__ out) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)groups * n) return;
  const long g = idx / n, col = idx % n;
  long pos;
  if (groups > 1) {
    const int c64 = (int)(col % 64);
    pos = col - c64 + 8 * (c64 % 8) + c64 / 8;
  } else {
    const int c32 = (int)(col % 32);
    pos = col - c32 + 8 * ((c32 % 8) / 2) + 2 * (c32 / 8) + c32 % 2;
  }
  out[g * n + pos] = s[idx];
}

}  // namespace

extern "C" int w4a16_quantize_pack_device(const void *weight_nk, const void *scales, int k, int n, int groupsize,
                                          void *B, void *s_packed, void *stream) {
  if (!weight_nk || !scales || !B || !s_packed) return W4A16_ERR_ARG;
  if (groupsize != -1 && groupsize != 128) return W4A16_ERR_KERN_SHAPE;      // marlin.py:70-71
  if (k <= 0 || n <= 0 || k % 128 || n % 256) return W4A16_ERR_PROB_SHAPE;   // marlin.py:72-73
  const int group = groupsize == -1 ? k : groupsize;
  const int groups = k / group;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (reinterpret_cast<uintptr_t>(weight_nk) & 15) return W4A16_ERR_ARG;   // rows are read 16 bytes at a time (k % 128 == 0)
  quantize_pack_kernel<<<dim3((unsigned)(k / QT_K), (unsigned)(n / QT_N)), 256, 0, st>>>(
      static_cast<const __half *>(weight_nk), static_cast<const __half *>(scales), k, n, group, static_cast<uint32_t *>(B));
  const long ns = (long)groups * n;
  permute_scales_kernel<<<(unsigned)((ns + 255) / 256), 256, 0, st>>>(static_cast<const __half *>(scales), groups, n,
                                                                     static_cast<__half *>(s_packed));
  return cudaGetLastError() == cudaSuccess ? W4A16_OK : W4A16_ERR_CUDA;
}
