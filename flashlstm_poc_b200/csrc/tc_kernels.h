// Host-side launchers of the tensor-core path kernels (tc_*.cu).
#pragma once

#include <cuda_runtime.h>

#include <cstddef>

namespace flstm_b200 {
namespace tc {

// D[M,N] (row pitch ldd, dtype out_dtype) = A B^T (+ bias[N]), fp32 accumulation in TMEM.
//   mn_major == false: A is (M,K) row-major with pitch lda, B is (N,K) row-major with pitch ldb.
//   mn_major == true : A is stored (K,M) with pitch lda, B is stored (K,N) with pitch ldb (fp32 out only).
// `err_word` is a device word the kernel sets to 1 if a bounded wait expired.
int gemm(int dtype, int out_dtype, size_t M, size_t N, size_t K, const void *A, size_t lda, const void *B, size_t ldb,
         void *D, size_t ldd, const float *bias, bool mn_major, unsigned int *err_word, int sms, cudaStream_t s);

int device_sm_count();

}  // namespace tc
}  // namespace flstm_b200
