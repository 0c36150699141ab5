// Library matrix product of the bfloat16 path: C[M, N] = A[M, K] * W[N, K]^T
// with float accumulation, bfloat16 or float output.
//
// This is the one place where a library stands in the product path, exactly
// where 7QiC/ccInfer has one (cublasGemmEx with CUBLAS_COMPUTE_32F,
// src/backend/cuda/cuda_backend.cpp:82-108).  The row-major product is the
// column-major product C^T = W * A^T, as in that file (:72-80).
#include "common.cuh"
#include <cublas_v2.h>

CCB_API int ccb_cublas_create(void** handle_out) {
  cublasHandle_t h = nullptr;
  const cublasStatus_t st = cublasCreate(&h);
  if (st != CUBLAS_STATUS_SUCCESS) return 1000 + (int)st;
  *handle_out = (void*)h;
  return 0;
}

CCB_API int ccb_cublas_destroy(void* handle) {
  if (handle == nullptr) return 0;
  return (int)cublasDestroy((cublasHandle_t)handle);
}

// A caller-owned workspace keeps the library from allocating inside a step
// (and inside a stream capture).
CCB_API int ccb_cublas_set_workspace(void* handle, void* workspace, size_t bytes) {
  const cublasStatus_t st = cublasSetWorkspace((cublasHandle_t)handle, workspace, bytes);
  return st == CUBLAS_STATUS_SUCCESS ? 0 : 1000 + (int)st;
}

CCB_API int ccb_gemm_bf16(void* handle, void* C, const void* A, const void* W, int M, int N, int K, int lda,
                          int ldw, int ldc, int out_dtype, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || lda < K || ldw < K || ldc < N) return CCB_REFUSE_SIZE;
  if (out_dtype != CCB_F32 && out_dtype != CCB_BF16) return CCB_REFUSE_DTYPE;
  cublasHandle_t h = (cublasHandle_t)handle;
  cublasStatus_t st = cublasSetStream(h, stream);
  if (st != CUBLAS_STATUS_SUCCESS) return 1000 + (int)st;
  const float alpha = 1.f, beta = 0.f;
  st = cublasGemmEx(h, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &alpha, W, CUDA_R_16BF, ldw, A, CUDA_R_16BF, lda, &beta,
                    C, out_dtype == CCB_F32 ? CUDA_R_32F : CUDA_R_16BF, ldc, CUBLAS_COMPUTE_32F,
                    CUBLAS_GEMM_DEFAULT);
  return st == CUBLAS_STATUS_SUCCESS ? 0 : 1000 + (int)st;
}
