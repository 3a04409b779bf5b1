// Stand-in for the CUDA-samples header of the same name, which the reference includes
// (cuda_bert/utils/common.h:13) but which is not part of the CUDA toolkit any more.  Written
// from scratch: only what the reference's sources use from it, i.e. checkCudaErrors() for
// cudaError_t and cublasStatus_t.  Used only to build oracle/_ref (the reference's own CUDA
// library, a test-time checker); the product never includes it.
#pragma once
#include <cstdio>
#include <cstdlib>
#include <cublas_v2.h>
#include <cuda_runtime.h>

inline void ref_shim_check(cudaError_t e, const char* expr, const char* file, int line) {
  if (e != cudaSuccess) {
    std::fprintf(stderr, "CUDA error %d (%s) in %s at %s:%d\n", static_cast<int>(e), cudaGetErrorString(e), expr, file,
                 line);
    std::exit(EXIT_FAILURE);
  }
}
inline void ref_shim_check(cublasStatus_t e, const char* expr, const char* file, int line) {
  if (e != CUBLAS_STATUS_SUCCESS) {
    std::fprintf(stderr, "cuBLAS error %d in %s at %s:%d\n", static_cast<int>(e), expr, file, line);
    std::exit(EXIT_FAILURE);
  }
}
#define checkCudaErrors(expr) ref_shim_check((expr), #expr, __FILE__, __LINE__)
