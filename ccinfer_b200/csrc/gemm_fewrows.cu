// Matrix product for few rows (decode steps), second form: C[M, N] = A[M, K] * W[N, K]^T, bfloat16, M <= 16.
//
// The product is a stream of W, and for the small matrices of a layer (q|k|v, o) what counts beside the
// bandwidth is what a block costs around its main loop.  So: small blocks, no tensor memory, no partial
// sums through global memory.
//   * A block owns 16 features (one m16n8k16 tile: the weights are the M side, the tokens the N side) and
//     walks the WHOLE K range, so there are N / 16 blocks that the hardware deals out as SMs fall free, and
//     nothing is added across blocks.
//   * A producer warp brings W (box 16 rows x 256 k, 8 KB) and the tokens (box 8 or 16 rows x 256 k) into a
//     ring of shared-memory stages by TMA, each stage with a full and an empty mbarrier.  The ring is as
//     deep as it can be with all blocks of the launch resident at once (two blocks of eight stages to seven
//     blocks of two stages per SM), so 100-130 KB of weights are in flight per SM from the first cycle and
//     there is no second wave.  The weight boxes of the first ring are requested before
//     griddepcontrol.wait (programmatic dependent launch), the token boxes after it.  Before the producer
//     refills a stage that the consumers have handed back it executes fence.proxy.async: they read the
//     stage through the generic proxy, the copy writes it through the async proxy.
//   * Eight consumer warps split each stage along k (32 k each): lane (gid, tig) reads 8 consecutive k of
//     weight rows gid and gid + 8 and of token gid with one 16-byte shared-memory load each and feeds two
//     mma instructions (a tensor-core product does not care in which order k is walked as long as both
//     operands agree).  The eight partial tiles are added through shared memory in a fixed order.
//   * Epilogues: C as bfloat16 or float; or silu(gate) * up for a weight matrix whose rows come in blocks
//     of 64 gate rows followed by the 64 up rows of the same channels: a block then takes 8 gate rows and
//     the 8 up rows of the same channels, which the fragment layout puts into the SAME thread (rows gid and
//     gid + 8), so the activation costs no exchange at all.
//   * Two more epilogues take the RMSNorm between two products apart, so that it needs no kernel of its own
//     (y = x * rsqrt(mean(x^2) + eps) * w is linear in x but for one factor per token, and a product commutes
//     with that factor).  "Into the residual stream": h[t, n] += C[t, n] in float, the block writes
//     bf16(h * w_norm) in place of C and the sum of h^2 over its 16 features to ssq_out[t][block].  "Row
//     scale": a product whose tokens are such rows multiplies token t of its result by
//     1 / sqrt(sum over blocks of ssq_in[t][block] / dim + eps) before anything else (before the activation).
//     The partial sums are added in the order of the blocks: nothing depends on which block ran first.
// (7QiC/ccInfer runs these products in cuBLAS, src/backend/cuda/cuda_backend.cpp:82-108, the activation
// as a kernel of its own, src/kernel/mlp/silu_mul.cu:24-28, and the sum and the norm as two more,
// src/kernel/norm/rms_norm.cu:24-60.)
//
// Every wait on an mbarrier is bounded: after kWaitLimit failed polls the thread records
// CCB_ST_WAIT_TIMEOUT in the status word and stops waiting; the block still reaches its barriers and returns.
#include "common.cuh"
#include <cuda.h>

#include "mma_common.cuh"
#include "tc_common.cuh"
#include "tma_host.h"

using namespace ccb;

namespace {

constexpr int FR_ROWS = 16;             // weight rows (features) per block
constexpr int FR_KC = 256;              // k elements per stage
constexpr int FR_WARPS = 8;             // consumer warps; warp FR_WARPS is the producer
constexpr int FR_THREADS = (FR_WARPS + 1) * 32;
constexpr int FR_W_BYTES = FR_ROWS * FR_KC * 2;

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 r;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
  return r;
}

__device__ __forceinline__ float silu_fr(float g) { return g / (1.f + __expf(-g)); }

}  // namespace

// the two halves of a norm that has no kernel of its own (see the head of this file); all null / 0 = off
struct CcbNormFuse {
  const float* ssq_in;   // [16][parts_in]: partial sums of squares of the token rows of A
  int parts_in;
  float dim, eps;        // of the norm whose factor is applied
  float* h;              // residual stream [M, ldh], float
  int ldh;
  const float* norm_w;   // [N]: weight of the norm that follows
  float* ssq_out;        // [16][blocks]
};

namespace {

// NB: 8-token tiles (M <= 8 NB).  tmW: box FR_KC x 16 rows (plain) or FR_KC x 8 rows (swiglu); tmX: box
// FR_KC x 8 NB rows.  Both without a swizzle: a box lies in shared memory as rows of 512 bytes.
template <int NB, int STAGES, typename TOut>
__global__ void __launch_bounds__(FR_THREADS)
gemm_fewrows_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                    TOut* __restrict__ C, int M, int N, int K, int ldc, int swiglu, const CcbNormFuse fuse, int* status) {
  __shared__ float s_scale[16];
  constexpr int X_BYTES = 8 * NB * FR_KC * 2;
  constexpr int RED_LD = 8 * NB + 1;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sW = smem;
  uint8_t* sX = smem + STAGES * FR_W_BYTES;
  float* red = reinterpret_cast<float*>(sX + STAGES * X_BYTES);  // [warp][16][RED_LD]
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + FR_WARPS * 16 * RED_LD + (FR_WARPS * 16 * RED_LD & 1));
  const uint32_t full0 = s32(bars), empty0 = s32(bars + STAGES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nstage = (K + FR_KC - 1) / FR_KC;
  // plain: features n0 .. n0 + 15.  swiglu: channels ch0 .. ch0 + 7, their gate rows at row_g .. + 7 and
  // their up rows 64 further on
  const int n0 = blockIdx.x * FR_ROWS;
  const int ch0 = blockIdx.x * 8;
  const int row_g = (ch0 >> 6) * 128 + (ch0 & 63);

  float h_old = 0.f, nw = 0.f;  // of the thread's (token, feature) of the "into the residual stream" epilogue
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, FR_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == FR_WARPS) {
    if (lane == 0) {  // ---- TMA producer ----
      auto load_w = [&](int i, int s) {
        const uint32_t dst = s32(sW + s * FR_W_BYTES), bar = full0 + 8 * s;
        if (swiglu) {
          tma_load_2d(dst, &tmW, i * FR_KC, row_g, bar);
          tma_load_2d(dst + FR_W_BYTES / 2, &tmW, i * FR_KC, row_g + 64, bar);
        } else {
          tma_load_2d(dst, &tmW, i * FR_KC, n0, bar);
        }
      };
      const int pre = min(nstage, STAGES);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(full0 + 8 * i, FR_W_BYTES + X_BYTES);
        load_w(i, i);
      }
      pdl_wait();
      pdl_trigger();
      for (int i = 0; i < pre; ++i) tma_load_2d(s32(sX + i * X_BYTES), &tmX, i * FR_KC, 0, full0 + 8 * i);
      for (int i = pre; i < nstage; ++i) {
        const int s = i % STAGES, ph = (i / STAGES) & 1;
        if (!mbar_wait(empty0 + 8 * s, ph ^ 1)) {
          set_status(status, CCB_ST_WAIT_TIMEOUT);
          break;
        }
        // The consumers read the stage through the generic proxy, the copy writes it through the async
        // proxy: the mbarrier orders the threads, this fence orders the proxies.  Without it the new tokens
        // landed under reads that were still in flight (wrong features in random blocks, seen once three
        // or more blocks shared an SM).
        fence_async_smem();
        mbar_expect_tx(full0 + 8 * s, FR_W_BYTES + X_BYTES);
        load_w(i, s);
        tma_load_2d(s32(sX + s * X_BYTES), &tmX, i * FR_KC, 0, full0 + 8 * s);
      }
    }
  } else {  // ---- consumers: warp w takes k 32 w .. 32 w + 31 of every stage ----
    if (fuse.ssq_in != nullptr || fuse.h != nullptr) {
      // what the epilogue needs of the kernels before this one is asked for now, while the first stages are
      // on their way, not after the last product
      pdl_wait();
      if (fuse.ssq_in != nullptr) {  // the factor of each token row: partial sums in the order of their blocks
        for (int tok = warp; tok < 8 * NB; tok += FR_WARPS) {
          const float ss = tok < M ? ccb::row_ssq(fuse.ssq_in + (size_t)tok * fuse.parts_in, fuse.parts_in, lane) : 0.f;
          if (lane == 0) s_scale[tok] = 1.0f / sqrtf(ss / fuse.dim + fuse.eps);
        }
      }
      if (fuse.h != nullptr && threadIdx.x < 16 * 8 * NB) {
        const int tok = threadIdx.x >> 4, f = threadIdx.x & 15;
        if (tok < M && n0 + f < N) {
          h_old = fuse.h[(size_t)tok * fuse.ldh + n0 + f];
          nw = fuse.norm_w[n0 + f];
        }
      }
    }
    const int gid = lane >> 2, tig = lane & 3;
    float c[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) c[nb][0] = c[nb][1] = c[nb][2] = c[nb][3] = 0.f;
    const uint32_t koff = (uint32_t)(warp * 32 + tig * 8) * 2;
    const uint32_t w_lo = s32(sW) + gid * (FR_KC * 2) + koff, w_hi = w_lo + 8 * (FR_KC * 2);
    const uint32_t x_lo = s32(sX) + gid * (FR_KC * 2) + koff;
    for (int i = 0; i < nstage; ++i) {
      const int s = i % STAGES, ph = (i / STAGES) & 1;
      if (!mbar_wait(full0 + 8 * s, ph)) {
        if (lane == 0) set_status(status, CCB_ST_WAIT_TIMEOUT);
        break;
      }
      const uint4 a0 = lds128(w_lo + s * FR_W_BYTES), a1 = lds128(w_hi + s * FR_W_BYTES);
      uint4 x[NB];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) x[nb] = lds128(x_lo + s * X_BYTES + nb * 8 * (FR_KC * 2));
      const uint32_t fa[4] = {a0.x, a1.x, a0.y, a1.y};
      const uint32_t fb[4] = {a0.z, a1.z, a0.w, a1.w};
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        mma_bf16_16816(c[nb], fa, x[nb].x, x[nb].y);
        mma_bf16_16816(c[nb], fb, x[nb].z, x[nb].w);
      }
      // the stage is handed back after the products have taken its registers
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * s);
    }
    // c[nb]: (row gid, tokens 8 nb + 2 tig, + 1), (row gid + 8, same tokens)
    float* mine = red + warp * 16 * RED_LD;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      mine[gid * RED_LD + nb * 8 + 2 * tig] = c[nb][0];
      mine[gid * RED_LD + nb * 8 + 2 * tig + 1] = c[nb][1];
      mine[(gid + 8) * RED_LD + nb * 8 + 2 * tig] = c[nb][2];
      mine[(gid + 8) * RED_LD + nb * 8 + 2 * tig + 1] = c[nb][3];
    }
  }
  __syncthreads();
  if (warp < FR_WARPS) {
    const bool scaled = fuse.ssq_in != nullptr;
    if (fuse.h != nullptr) {
      // into the residual stream: 16 consecutive threads hold the 16 features of a token
      const int idx = threadIdx.x;
      if (idx < 16 * 8 * NB) {  // whole warps: 128 NB of the 256 consumer threads
        const int tok = idx >> 4, f = idx & 15;
        float v = 0.f;
        if (tok < M && n0 + f < N) {
          float sum = 0.f;
#pragma unroll
          for (int w = 0; w < FR_WARPS; ++w) sum += red[(w * 16 + f) * RED_LD + tok];
          if (scaled) sum *= s_scale[tok];
          v = h_old + sum;
          fuse.h[(size_t)tok * fuse.ldh + n0 + f] = v;
          C[(size_t)tok * ldc + n0 + f] = from_f32<TOut>(v * nw);
        }
        float q = v * v;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
        if (f == 0) fuse.ssq_out[(size_t)tok * gridDim.x + blockIdx.x] = q;
      }
    } else if (swiglu) {
      for (int idx = threadIdx.x; idx < 8 * 8 * NB; idx += FR_WARPS * 32) {
        const int tok = idx >> 3, f = idx & 7;  // consecutive threads write consecutive channels of a token
        if (tok < M && 2 * (ch0 + f) < N) {
          float g = 0.f, u = 0.f;
#pragma unroll
          for (int w = 0; w < FR_WARPS; ++w) {
            g += red[(w * 16 + f) * RED_LD + tok];
            u += red[(w * 16 + f + 8) * RED_LD + tok];
          }
          if (scaled) g *= s_scale[tok], u *= s_scale[tok];
          C[(size_t)tok * ldc + ch0 + f] = from_f32<TOut>(silu_fr(g) * u);
        }
      }
    } else {
      for (int idx = threadIdx.x; idx < 16 * 8 * NB; idx += FR_WARPS * 32) {
        const int tok = idx >> 4, f = idx & 15;  // consecutive threads write consecutive features of a token
        if (tok < M && n0 + f < N) {
          float sum = 0.f;
#pragma unroll
          for (int w = 0; w < FR_WARPS; ++w) sum += red[(w * 16 + f) * RED_LD + tok];
          if (scaled) sum *= s_scale[tok];
          C[(size_t)tok * ldc + n0 + f] = from_f32<TOut>(sum);
        }
      }
    }
  }
}

int g_fr_stages = 0;  // 0: the default of the shape

template <int NB, int STAGES, typename TOut>
int launch_fewrows(const CUtensorMap& tmW, const CUtensorMap& tmX, void* C, int M, int N, int K, int ldc, int swiglu,
                   const CcbNormFuse& fuse, int* status, cudaStream_t stream) {
  constexpr int RED = FR_WARPS * 16 * (8 * NB + 1);
  constexpr size_t smem = (size_t)STAGES * (FR_W_BYTES + 8 * NB * FR_KC * 2) + (size_t)(RED + (RED & 1)) * 4 + 2 * STAGES * 8;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fewrows_kernel<NB, STAGES, TOut>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int blocks = swiglu ? (N / 2 + 7) / 8 : (N + FR_ROWS - 1) / FR_ROWS;
  ccb_launch_ex(true, gemm_fewrows_kernel<NB, STAGES, TOut>, dim3(blocks), FR_THREADS, smem, stream, tmW, tmX,
                (TOut*)C, M, N, K, ldc, swiglu, fuse, status);
  return ccb_launch_status();
}

// The ring is as deep as it can be with every block of the launch resident at once (148 SMs, 228 KB of
// shared memory each, 1 KB of it per block for the system): a single wave has no second ramp (measured: q|k|v
// of 10240 x 5120 at 8 tokens 20.1 us with three stages and five blocks per SM, 23.9 us with four stages and
// four).  With more blocks than fit at two stages, four (8 tokens) or three (16 tokens) blocks per SM.
template <int NB, typename TOut>
int pick_stages(const CUtensorMap& tmW, const CUtensorMap& tmX, void* C, int M, int N, int K, int ldc, int swiglu,
                const CcbNormFuse& fuse, int* status, cudaStream_t stream) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  const int blocks = (N + FR_ROWS - 1) / FR_ROWS;
  int st = g_fr_stages;
  if (st == 0) {
    const int per_sm = (blocks + sms - 1) / sms;  // blocks an SM must hold for a single wave
    if (NB == 1) st = per_sm <= 2 ? 8 : (per_sm == 3 ? 5 : (per_sm == 4 ? 4 : (per_sm == 5 ? 3 : (per_sm <= 7 ? 2 : 4))));
    else st = per_sm <= 2 ? 6 : (per_sm == 3 ? 4 : (per_sm <= 5 ? 2 : 4));
  }
#define CCB_FR_CASE(S) \
  if (st == S) return launch_fewrows<NB, S, TOut>(tmW, tmX, C, M, N, K, ldc, swiglu, fuse, status, stream);
  CCB_FR_CASE(8)
  CCB_FR_CASE(6)
  CCB_FR_CASE(5)
  CCB_FR_CASE(3)
  CCB_FR_CASE(2)
#undef CCB_FR_CASE
  return launch_fewrows<NB, 4, TOut>(tmW, tmX, C, M, N, K, ldc, swiglu, fuse, status, stream);
}

template <typename TOut>
int dispatch_fewrows(void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldc, int swiglu,
                     const CcbNormFuse& fuse, int* status, cudaStream_t stream) {
  CUtensorMap tmW, tmX;
  const int nb = M <= 8 ? 1 : 2;
  if (!ccb_tensor_map_2d_plain(W, N, K, ldw, FR_KC, swiglu ? 8 : FR_ROWS, &tmW) ||
      !ccb_tensor_map_2d_plain(A, M, K, lda, FR_KC, 8 * nb, &tmX))
    return CCB_REFUSE_ARG;
  if (nb == 1) return pick_stages<1, TOut>(tmW, tmX, C, M, N, K, ldc, swiglu, fuse, status, stream);
  return pick_stages<2, TOut>(tmW, tmX, C, M, N, K, ldc, swiglu, fuse, status, stream);
}

}  // namespace

CCB_API int ccb_gemm_fewrows_set_stages(int n) {
  g_fr_stages = n;
  return 0;
}

// C[M, N] = A[M, K] W[N, K]^T (swiglu = 0), or C[M, N / 2] = silu(A Wg^T) * (A Wu^T) for W [N, K] whose rows
// come in blocks of 64 gate rows followed by the 64 up rows of the same channels (swiglu = 1, N a multiple
// of 128).  M <= 16; K and the row strides multiples of 8 elements; A and W 16-byte aligned.
static int fewrows_checked(void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldc,
                           int out_dtype, int swiglu, const CcbNormFuse& fuse, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (out_dtype != CCB_F32 && out_dtype != CCB_BF16) return CCB_REFUSE_DTYPE;
  if (M > 16 || K <= 0 || (K & 7) || lda < K || ldw < K || (lda & 7) || (ldw & 7) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
    return CCB_REFUSE_SIZE;
  if (swiglu ? ((N & 127) || ldc < N / 2) : (ldc < N)) return CCB_REFUSE_SIZE;
  if (out_dtype == CCB_F32)
    return dispatch_fewrows<float>(C, A, W, M, N, K, lda, ldw, ldc, swiglu, fuse, status, stream);
  return dispatch_fewrows<__nv_bfloat16>(C, A, W, M, N, K, lda, ldw, ldc, swiglu, fuse, status, stream);
}

CCB_API int ccb_gemm_fewrows_bf16(void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw,
                                  int ldc, int out_dtype, int swiglu, int* status, cudaStream_t stream) {
  return fewrows_checked(C, A, W, M, N, K, lda, ldw, ldc, out_dtype, swiglu, CcbNormFuse{}, status, stream);
}

// Number of blocks of the plain product, which is the number of partial sums that the "into the residual
// stream" epilogue writes for every token.
CCB_API int ccb_gemm_fewrows_blocks(int N) { return (N + FR_ROWS - 1) / FR_ROWS; }

// The same product with the halves of a norm in its epilogue (see the head of this file).
//   ssq_in != null: token t of the result is multiplied by 1 / sqrt(sum_p ssq_in[t * parts_in + p] / dim + eps),
//     p < parts_in, before the activation if there is one.
//   h != null (plain product, bfloat16 result): h[t, n] += result, C[t, n] = bf16(h[t, n] * norm_w[n]) and
//     ssq_out[t * blocks + block] = sum over the block's 16 features of h[t, n]^2, blocks =
//     ccb_gemm_fewrows_blocks(N); ssq_out holds 16 * blocks floats.
CCB_API int ccb_gemm_fewrows_norm_bf16(void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw,
                                       int ldc, int out_dtype, int swiglu, const float* ssq_in, int parts_in,
                                       float dim, float eps, float* h, int ldh, const float* norm_w, float* ssq_out,
                                       int* status, cudaStream_t stream) {
  CcbNormFuse fuse{};
  if (ssq_in != nullptr) {
    if (parts_in <= 0 || !(dim > 0.f)) return CCB_REFUSE_ARG;
    fuse.ssq_in = ssq_in, fuse.parts_in = parts_in, fuse.dim = dim, fuse.eps = eps;
  }
  if (h != nullptr) {
    if (swiglu || out_dtype != CCB_BF16 || norm_w == nullptr || ssq_out == nullptr || ldh < N) return CCB_REFUSE_ARG;
    fuse.h = h, fuse.ldh = ldh, fuse.norm_w = norm_w, fuse.ssq_out = ssq_out;
  }
  return fewrows_checked(C, A, W, M, N, K, lda, ldw, ldc, out_dtype, swiglu, fuse, status, stream);
}
