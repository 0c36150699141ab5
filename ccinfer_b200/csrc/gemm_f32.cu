// True 32-bit matrix product for the float path: C[M, N] = A[M, K] * W[N, K]^T.
//
// IEEE float fused multiply-adds on the CUDA cores: no tensor cores, no TF32,
// no reduced-precision mode of any library (7QiC/ccInfer runs this product in
// cuBLAS with float accumulation, src/backend/cuda/cuda_backend.cpp:82-108).
// Every output element is one accumulation chain over k = 0 .. K-1 in
// ascending order, whatever the tile shape, so a row's result does not depend
// on how many other rows are in the batch.  Any M, N, K.
#include "common.cuh"

constexpr int kBK = 8;
constexpr int kBN = 128;
constexpr int kTN = 8;

template <int TM>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(float* __restrict__ C, const float* __restrict__ A, const float* __restrict__ W, int M, int N,
                int K, int lda, int ldw, int ldc) {
  ccb::pdl_begin();
  constexpr int BM = 16 * TM;
  __shared__ __align__(16) float As[kBK][BM];
  __shared__ __align__(16) float Ws[kBK][kBN];
  const int tid = threadIdx.x;
  const int ty = tid >> 4, tx = tid & 15;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * kBN;
  const bool vec_a = (lda % 4 == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0);
  const bool vec_w = (ldw % 4 == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0);

  float acc[TM][kTN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < kTN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += kBK) {
    for (int idx = tid; idx < BM * kBK / 4; idx += 256) {
      const int row = idx >> 1, kq = (idx & 1) * 4;
      const int gm = m0 + row, gk = k0 + kq;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (gm < M) {
        const float* src = A + (size_t)gm * lda + gk;
        if (vec_a && gk + 3 < K) {
          const float4 f = *reinterpret_cast<const float4*>(src);
          v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (gk + e < K) v[e] = src[e];
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) As[kq + e][row] = v[e];
    }
    for (int idx = tid; idx < kBN * kBK / 4; idx += 256) {
      const int row = idx >> 1, kq = (idx & 1) * 4;
      const int gn = n0 + row, gk = k0 + kq;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (gn < N) {
        const float* src = W + (size_t)gn * ldw + gk;
        if (vec_w && gk + 3 < K) {
          const float4 f = *reinterpret_cast<const float4*>(src);
          v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (gk + e < K) v[e] = src[e];
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) Ws[kq + e][row] = v[e];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kBK; ++k) {
      float a[TM], b[kTN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < kTN; ++j) b[j] = Ws[k][tx * kTN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < kTN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < kTN; ++j) {
      const int gn = n0 + tx * kTN + j;
      if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j];
    }
  }
}

// Zero padding of the k range adds exact zeros at the end of a chain, which
// does not change a float sum, so ragged K is exact too.
CCB_API int ccb_gemm_f32(float* C, const float* A, const float* W, int M, int N, int K, int lda, int ldw, int ldc,
                         cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || lda < K || ldw < K || ldc < N) return CCB_REFUSE_SIZE;
  const int gx = (N + kBN - 1) / kBN;
  if (M <= 16)
    ccb_launch(gemm_f32_kernel<1>, dim3(gx, (M + 15) / 16), 256, 0, stream, C, A, W, M, N, K, lda, ldw, ldc);
  else if (M <= 32)
    ccb_launch(gemm_f32_kernel<2>, dim3(gx, (M + 31) / 32), 256, 0, stream, C, A, W, M, N, K, lda, ldw, ldc);
  else if (M <= 64)
    ccb_launch(gemm_f32_kernel<4>, dim3(gx, (M + 63) / 64), 256, 0, stream, C, A, W, M, N, K, lda, ldw, ldc);
  else
    ccb_launch(gemm_f32_kernel<8>, dim3(gx, (M + 127) / 128), 256, 0, stream, C, A, W, M, N, K, lda, ldw, ldc);
  return ccb_launch_status();
}
