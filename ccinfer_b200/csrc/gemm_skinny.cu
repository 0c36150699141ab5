// Matrix product for few rows (decode steps): C[M, N] = A[M, K] * W[N, K]^T, bfloat16 operands, M <= 32.
//
// With a handful of tokens the product is a stream of the weight matrix through the SMs: what matters is
// that every SM has enough 16-byte loads of W in flight, and the arithmetic must merely keep up.  So the
// roles are swapped against a large product: 16 rows of W (16 output features) are the M side of an
// m16n8k16 tensor-core tile, the tokens are its N side (8 per tile).  A block of 8 warps owns 16 features;
// each warp takes one eighth of K, streams its slice of the 16 weight rows straight from global memory
// into registers, and the eight partial sums are added through shared memory in a fixed order.
//
// No shared-memory staging of the operands is needed: a tensor-core product does not care in which order
// the k index is walked as long as both operands agree, so lane (gid, tig) loads 8 consecutive k of row
// gid (one 16-byte load) and feeds them to two mma instructions; the token operand is loaded with the same
// pattern.  (7QiC/ccInfer runs this product in cuBLAS, src/backend/cuda/cuda_backend.cpp:82-108, which at
// this shape leaves most of the memory bandwidth unused.)
#include "common.cuh"
#include "mma_common.cuh"

using namespace ccb;

namespace {

constexpr int kSkinnyWarps = 8;

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];\n"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

// NB: number of 8-token tiles (M <= 8 * NB).  TOut: float or bfloat16.
template <int NB, typename TOut>
__global__ void __launch_bounds__(kSkinnyWarps * 32)
gemm_skinny_kernel(TOut* __restrict__ C, const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                   int M, int N, int K, int lda, int ldw, int ldc) {
  __shared__ float red[kSkinnyWarps][16][8 * NB + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int n0 = blockIdx.x * 16;
  // rows beyond N are read from the last row and never written
  const int r0 = min(n0 + gid, N - 1), r1 = min(n0 + gid + 8, N - 1);
  const int kblocks = K >> 5;
  const int kb0 = (int)((long long)kblocks * warp / kSkinnyWarps);
  const int kb1 = (int)((long long)kblocks * (warp + 1) / kSkinnyWarps);
  const __nv_bfloat16* w0 = W + (size_t)r0 * ldw + tig * 8;
  const __nv_bfloat16* w1 = W + (size_t)r1 * ldw + tig * 8;
  const __nv_bfloat16* xa[NB];
  bool xv[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    const int tok = nb * 8 + gid;
    xv[nb] = tok < M;
    xa[nb] = A + (size_t)(xv[nb] ? tok : 0) * lda + tig * 8;
  }
  float c[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) c[nb][0] = c[nb][1] = c[nb][2] = c[nb][3] = 0.f;

  constexpr int U = 4;  // 32-wide k blocks in flight per warp
  // The weights do not depend on the kernel before this one: the loads of the first group of k blocks are
  // issued before waiting for it (programmatic dependent launch), the token operand after.
  int kb = kb0;
  uint4 a0[U], a1[U];
  const bool first_full = kb + U <= kb1;
  if (first_full) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      a0[u] = ld_stream16(w0 + ((kb + u) << 5));
      a1[u] = ld_stream16(w1 + ((kb + u) << 5));
    }
  }
  pdl_wait();
  pdl_trigger();
  for (; kb + U <= kb1; kb += U) {
    uint4 x[U][NB];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (kb + u) << 5;
      if (kb != kb0) {  // the first group is already on its way
        a0[u] = ld_stream16(w0 + k);
        a1[u] = ld_stream16(w1 + k);
      }
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
        x[u][nb] = xv[nb] ? *reinterpret_cast<const uint4*>(xa[nb] + k) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t fa[4] = {a0[u].x, a1[u].x, a0[u].y, a1[u].y};
      const uint32_t fb[4] = {a0[u].z, a1[u].z, a0[u].w, a1[u].w};
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        mma_bf16_16816(c[nb], fa, x[u][nb].x, x[u][nb].y);
        mma_bf16_16816(c[nb], fb, x[u][nb].z, x[u][nb].w);
      }
    }
  }
  for (; kb < kb1; ++kb) {
    const int k = kb << 5;
    const uint4 a0 = ld_stream16(w0 + k), a1 = ld_stream16(w1 + k);
    const uint32_t fa[4] = {a0.x, a1.x, a0.y, a1.y};
    const uint32_t fb[4] = {a0.z, a1.z, a0.w, a1.w};
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const uint4 x = xv[nb] ? *reinterpret_cast<const uint4*>(xa[nb] + k) : make_uint4(0u, 0u, 0u, 0u);
      mma_bf16_16816(c[nb], fa, x.x, x.y);
      mma_bf16_16816(c[nb], fb, x.z, x.w);
    }
  }
  // c[nb]: (feature gid, tokens 8 nb + 2 tig, + 1), (feature gid + 8, same tokens)
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    red[warp][gid][nb * 8 + 2 * tig] = c[nb][0];
    red[warp][gid][nb * 8 + 2 * tig + 1] = c[nb][1];
    red[warp][gid + 8][nb * 8 + 2 * tig] = c[nb][2];
    red[warp][gid + 8][nb * 8 + 2 * tig + 1] = c[nb][3];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < 16 * 8 * NB; idx += kSkinnyWarps * 32) {
    const int tok = idx >> 4, f = idx & 15;  // consecutive threads write consecutive features of a token
    if (tok < M && n0 + f < N) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kSkinnyWarps; ++w) s += red[w][f][tok];
      C[(size_t)tok * ldc + n0 + f] = from_f32<TOut>(s);
    }
  }
}

template <int NB>
int launch_skinny(void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldc,
                  int out_dtype, cudaStream_t stream) {
  const int blocks = (N + 15) / 16;
  if (out_dtype == CCB_F32)
    ccb_launch_ex(true, gemm_skinny_kernel<NB, float>, blocks, kSkinnyWarps * 32, 0, stream, 
        (float*)C, (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, M, N, K, lda, ldw, ldc);
  else
    ccb_launch_ex(true, gemm_skinny_kernel<NB, __nv_bfloat16>, blocks, kSkinnyWarps * 32, 0, stream, 
        (__nv_bfloat16*)C, (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, M, N, K, lda, ldw, ldc);
  return ccb_launch_status();
}

}  // namespace

// Takes M <= 32, K a multiple of 32, row strides that are multiples of 8 elements and 16-byte aligned
// bases; anything else is refused (CCB_REFUSE_SIZE) and belongs to the general product.
CCB_API int ccb_gemm_skinny_bf16(void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw,
                                 int ldc, int out_dtype, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (out_dtype != CCB_F32 && out_dtype != CCB_BF16) return CCB_REFUSE_DTYPE;
  if (M > 32 || K <= 0 || (K & 31) || lda < K || ldw < K || ldc < N || (lda & 7) || (ldw & 7) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
    return CCB_REFUSE_SIZE;
  if (M <= 8) return launch_skinny<1>(C, A, W, M, N, K, lda, ldw, ldc, out_dtype, stream);
  if (M <= 16) return launch_skinny<2>(C, A, W, M, N, K, lda, ldw, ldc, out_dtype, stream);
  return launch_skinny<4>(C, A, W, M, N, K, lda, ldw, ldc, out_dtype, stream);
}
