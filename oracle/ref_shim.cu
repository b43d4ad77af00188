// C-ABI doorway onto the reference's own vendored Marlin launcher, compiled from the
// reference checkout where it lies (never copied).  TEST INFRASTRUCTURE ONLY: used by
// the GPU parity tests as a second opinion and by the bench as the legacy mma.sync
// comparator.  The declaration mirrors gemm/marlin_gemm/marlin_official_kernel.cu:782-798.
#include <cuda_runtime.h>

int marlin_official(const void *A, const void *B, void *C, void *s, int prob_m, int prob_n, int prob_k,
                    void *workspace, int groupsize, int dev, cudaStream_t stream, int thread_k,
                    int thread_n, int sms, int max_par);

extern "C" int ref_marlin_official(const void *A, const void *B, void *C, void *s, int prob_m, int prob_n,
                                   int prob_k, void *workspace, int groupsize, int dev, void *stream,
                                   int thread_k, int thread_n, int sms, int max_par) {
  return marlin_official(A, B, C, s, prob_m, prob_n, prob_k, workspace, groupsize, dev,
                         (cudaStream_t)stream, thread_k, thread_n, sms, max_par);
}
