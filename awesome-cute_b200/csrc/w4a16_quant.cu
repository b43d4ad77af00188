// Device-side Layer.pack: fake-quantised (or plain) fp16 weights + scales -> Marlin-packed int4 words and permuted
// scales, bit-exact with the host packer (w4a16_pack.cpp) and therefore with the reference's numpy packer
// (gemm/marlin_gemm/marlin.py:92-131).  One thread builds one packed word: it gathers its eight weights through
// the closed form of the layout, quantises each as the reference does (fp16 division, round half to even, +8,
// clamp to 0..15; marlin.py:108-110) and ORs the nibbles together.  HBM-bound elementwise work: it reads 2 bytes
// and writes 0.5 byte per weight; nothing here is a GEMM.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/w4a16.h"

namespace {

__global__ void quantize_pack_kernel(const __half *__restrict__ w_nk, const __half *__restrict__ scales, int k, int n,
                                     int group, uint32_t *__restrict__ B) {
  const long words = (long)(k / 16) * 2 * n;
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= words) return;
  const long r = idx / (2L * n), c = idx % (2L * n);
  const long blk = c / 128;
  const int lane = (int)(c % 128) / 4, j = (int)(c % 4);
  uint32_t word = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const long nn = 64 * blk + 16 * j + lane / 4 + 8 * ((i >> 1) & 1);
    const long kk = 16 * r + 2 * (lane % 4) + (i >> 2) + 8 * (i & 1);
    const float quo = __half2float(__float2half_rn(__half2float(w_nk[nn * k + kk]) / __half2float(scales[(kk / group) * n + nn])));
    int code = (int)rintf(quo) + 8;
    code = code < 0 ? 0 : (code > 15 ? 15 : code);
    word |= (uint32_t)code << (4 * i);
  }
  B[idx] = word;
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
  const long words = (long)(k / 16) * 2 * n;
  quantize_pack_kernel<<<(unsigned)((words + 255) / 256), 256, 0, st>>>(
      static_cast<const __half *>(weight_nk), static_cast<const __half *>(scales), k, n, group, static_cast<uint32_t *>(B));
  const long ns = (long)groups * n;
  permute_scales_kernel<<<(unsigned)((ns + 255) / 256), 256, 0, st>>>(static_cast<const __half *>(scales), groups, n,
                                                                     static_cast<__half *>(s_packed));
  return cudaGetLastError() == cudaSuccess ? W4A16_OK : W4A16_ERR_CUDA;
}
