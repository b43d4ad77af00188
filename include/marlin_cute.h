/*
 * C++ launcher with the reference's exact name, parameter list and defaults, so the reference's
 * binding (gemm/marlin_gemm/marlin_gemm.cpp:6-9,36-39) links against this library unchanged.
 * Defined in the reference at gemm/marlin_gemm/marlin_cute_kernel.cu:28-31.  C++ linkage, as there.
 * Semantics and return codes: see w4a16_marlin_gemm in w4a16.h.
 */
#ifndef MARLIN_CUTE_H_
#define MARLIN_CUTE_H_

#include <cuda_runtime.h>

int marlin_cute(const void *A, const void *B, void *C, void *s, int prob_m, int prob_n, int prob_k,
                void *workspace, int groupsize = -1, int dev = 0, cudaStream_t stream = 0, int thread_k = -1,
                int thread_n = -1, int sms = -1, int max_par = 16);

#endif /* MARLIN_CUTE_H_ */
