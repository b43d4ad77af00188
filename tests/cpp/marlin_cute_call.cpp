// Calls the C++-linkage launcher the way the reference's binding does.
//
// The declaration below is the one the reference's caller carries (gemm/marlin_gemm/marlin_gemm.cpp:6-9): same name,
// parameter list and default arguments; the library under test must satisfy it unchanged.  Two calls are made:
//   1. with the defaults only (groupsize -1 is overridden when the fixture has group scales, the rest stays default:
//      dev 0, stream 0, automatic tiles, one CTA per SM, max_par 16);
//   2. spelled out as the binding spells it (marlin_gemm.cpp:36-39: groupsize, dev, a cudaStream_t, thread_k, thread_n,
//      sms, max_par), on a stream created here.
//
//   marlin_cute_call <in.bin> <out.bin>
//   in.bin : int32 m, n, k, groups, then A fp16 [m,k], B int32 [k/16, 2n], s fp16 [groups, n]  (B and s already packed)
//   out.bin: int32 rc1, rc2, then C fp16 [m,n] of call 1, C fp16 [m,n] of call 2
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

int marlin_cute(const void *A, const void *B, void *C, void *s, int prob_m,
                int prob_n, int prob_k, void *workspace, int groupsize = -1,
                int dev = 0, cudaStream_t stream = 0, int thread_k = -1,
                int thread_n = -1, int sms = -1, int max_par = 16);

#define CHECK(x)                                                                     \
  do {                                                                               \
    cudaError_t e_ = (x);                                                            \
    if (e_ != cudaSuccess) {                                                         \
      std::fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_));                  \
      return 2;                                                                      \
    }                                                                                \
  } while (0)

int main(int argc, char **argv) {
  if (argc != 3) return 64;
  std::FILE *f = std::fopen(argv[1], "rb");
  if (!f) return 65;
  int32_t hdr[4];
  if (std::fread(hdr, 4, 4, f) != 4) return 66;
  const int m = hdr[0], n = hdr[1], k = hdr[2], groups = hdr[3];
  std::vector<uint16_t> A((size_t)m * k), s((size_t)groups * n), C1((size_t)m * n), C2((size_t)m * n);
  std::vector<int32_t> B((size_t)k / 16 * 2 * n);
  if (std::fread(A.data(), 2, A.size(), f) != A.size() || std::fread(B.data(), 4, B.size(), f) != B.size() ||
      std::fread(s.data(), 2, s.size(), f) != s.size())
    return 67;
  std::fclose(f);
  const int groupsize = groups == 1 ? -1 : k / groups;        // as marlin_gemm.cpp:26 derives it

  CHECK(cudaSetDevice(0));
  void *dA, *dB, *ds, *dC, *dws;
  const size_t ws_ints = (size_t)n / 128 * 16;                 // marlin_gemm.cpp:29-31 with max_par = 16
  CHECK(cudaMalloc(&dA, A.size() * 2));
  CHECK(cudaMalloc(&dB, B.size() * 4));
  CHECK(cudaMalloc(&ds, s.size() * 2));
  CHECK(cudaMalloc(&dC, C1.size() * 2));
  CHECK(cudaMalloc(&dws, ws_ints * 4));
  CHECK(cudaMemcpy(dA, A.data(), A.size() * 2, cudaMemcpyHostToDevice));
  CHECK(cudaMemcpy(dB, B.data(), B.size() * 4, cudaMemcpyHostToDevice));
  CHECK(cudaMemcpy(ds, s.data(), s.size() * 2, cudaMemcpyHostToDevice));
  CHECK(cudaMemset(dws, 0, ws_ints * 4));

  // 1. default arguments
  CHECK(cudaMemset(dC, 0, C1.size() * 2));
  const int rc1 = groups == 1 ? marlin_cute(dA, dB, dC, ds, m, n, k, dws) : marlin_cute(dA, dB, dC, ds, m, n, k, dws, groupsize);
  CHECK(cudaDeviceSynchronize());
  CHECK(cudaMemcpy(C1.data(), dC, C1.size() * 2, cudaMemcpyDeviceToHost));

  // 2. every argument, as the binding passes them
  cudaStream_t stream;
  CHECK(cudaStreamCreate(&stream));
  CHECK(cudaMemsetAsync(dC, 0, C2.size() * 2, stream));
  const int dev = 0, thread_k = -1, thread_n = -1, sms = -1, max_par = 16;
  const int rc2 = marlin_cute(dA, dB, dC, ds, m, n, k, dws, groupsize, dev, stream, thread_k, thread_n, sms, max_par);
  CHECK(cudaStreamSynchronize(stream));
  CHECK(cudaMemcpy(C2.data(), dC, C2.size() * 2, cudaMemcpyDeviceToHost));

  // the lock array must still be all zero (gemm/marlin_gemm/marlin.py:17)
  std::vector<int32_t> ws(ws_ints);
  CHECK(cudaMemcpy(ws.data(), dws, ws_ints * 4, cudaMemcpyDeviceToHost));
  for (int32_t w : ws)
    if (w != 0) return 3;

  f = std::fopen(argv[2], "wb");
  if (!f) return 68;
  const int32_t rcs[2] = {rc1, rc2};
  std::fwrite(rcs, 4, 2, f);
  std::fwrite(C1.data(), 2, C1.size(), f);
  std::fwrite(C2.data(), 2, C2.size(), f);
  std::fclose(f);
  return 0;
}
