// Embedding gather and SiLU-multiply.
//
// embed:    h[t, :] = float(table[ids[t], :])          (7QiC/ccInfer: src/kernel/elementwise/elementwise.cu:67-78)
// silu_mul: act[t, f] = silu(gu[t, f]) * gu[t, F + f]  (7QiC/ccInfer: src/kernel/mlp/silu_mul.cu:24-28)
// The gate and up projections are one merged matrix product here, so the
// kernel reads both halves of a [T, 2F] row.
#include "common.cuh"

using namespace ccb;

int g_ccb_pdl = 0;

// 1: launch every kernel of the library so that it may overlap the end of its predecessor (see common.cuh)
CCB_API int ccb_set_pdl(int on) {
  g_ccb_pdl = on < 0 ? 0 : (on > 2 ? 2 : on);  // 1: products only; 2: every kernel
  return 0;
}

template <typename T>
__global__ void embed_gather_kernel(float* __restrict__ h, const T* __restrict__ table,
                                    const int* __restrict__ ids, int D, int V, const int* __restrict__ pending,
                                    int n_pending, int* status) {
  ccb::pdl_begin();
  const int t = blockIdx.x;
  int id = ids[t];
  // id = -1 - s names the token that the sampling kernel last stored for request slot s: the host has
  // launched this step before it has read that token
  if (id < 0 && pending != nullptr && -1 - id < n_pending) id = pending[-1 - id];
  float* out = h + (size_t)t * D;
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) set_status(status, CCB_ST_BAD_TOKEN);
    for (int d = threadIdx.x; d < D; d += blockDim.x) out[d] = 0.f;
    return;
  }
  const T* row = table + (size_t)id * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) out[d] = to_f32(row[d]);
}

CCB_API int ccb_embed_gather(float* h, const void* table, const int* ids, int T_, int D, int V,
                             int dtype, const int* pending, int n_pending, int* status, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (D <= 0 || V <= 0) return CCB_REFUSE_SIZE;
  const int threads = D >= 1024 ? 256 : 128;
  if (dtype == CCB_F32)
    ccb_launch(embed_gather_kernel<float>, T_, threads, 0, stream, h, (const float*)table, ids, D, V, pending, n_pending, status);
  else if (dtype == CCB_BF16)
    ccb_launch(embed_gather_kernel<__nv_bfloat16>, T_, threads, 0, stream, h, (const __nv_bfloat16*)table, ids, D, V, pending,
               n_pending, status);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

// accurate variant for the 32-bit path, fast exponential for the bf16 path
template <typename T> __device__ __forceinline__ float silu(float g);
template <> __device__ __forceinline__ float silu<float>(float g) { return g / (1.f + expf(-g)); }
template <> __device__ __forceinline__ float silu<__nv_bfloat16>(float g) { return g / (1.f + __expf(-g)); }

template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ act, const T* __restrict__ gu, int F, int B, size_t total) {
  ccb::pdl_begin();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t t = i / F;
    const int f = (int)(i - t * F);
    const T* row = gu + t * 2 * (size_t)F;
    const int gi = (f / B) * 2 * B + f % B;  // B gate columns, then the B up columns of the same channels
    const float g = to_f32(row[gi]);
    const float u = to_f32(row[gi + B]);
    act[i] = from_f32<T>(silu<T>(g) * u);
  }
}

// bf16, F even: two elements per thread
__global__ void silu_mul_bf16x2_kernel(__nv_bfloat162* __restrict__ act, const __nv_bfloat162* __restrict__ gu,
                                       int F2, int B2, size_t total2) {
  ccb::pdl_begin();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total2; i += stride) {
    const size_t t = i / F2;
    const int f = (int)(i - t * F2);
    const __nv_bfloat162* row = gu + t * 2 * (size_t)F2;
    const int gi = (f / B2) * 2 * B2 + f % B2;
    const float2 g = __bfloat1622float2(row[gi]);
    const float2 u = __bfloat1622float2(row[gi + B2]);
    act[i] = __floats2bfloat162_rn(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y);
  }
}

// bf16, F a multiple of 8: eight elements (16 bytes) per thread and access
__global__ void silu_mul_bf16x8_kernel(uint4* __restrict__ act, const uint4* __restrict__ gu, int F8, int B8,
                                       size_t total8) {
  ccb::pdl_begin();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total8; i += stride) {
    const size_t t = i / F8;
    const int f = (int)(i - t * F8);
    const uint4* row = gu + t * 2 * (size_t)F8;
    const int gi = (f / B8) * 2 * B8 + f % B8;
    const uint4 g = row[gi], u = row[gi + B8];
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = __bfloat1622float2(gh[e]), b = __bfloat1622float2(uh[e]);
      oh[e] = __floats2bfloat162_rn(a.x / (1.f + __expf(-a.x)) * b.x, a.y / (1.f + __expf(-a.y)) * b.y);
    }
    act[i] = o;
  }
}

// gate_up[t, :] holds the 2F columns either as [all gate | all up] (block = 0) or in blocks: `block` gate
// columns followed by the `block` up columns of the same channels (F a multiple of block).
CCB_API int ccb_silu_mul(void* act, const void* gate_up, int T_, int F, int block, int dtype, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (F <= 0 || block < 0 || (block > 0 && F % block != 0)) return CCB_REFUSE_SIZE;
  const int B = block == 0 ? F : block;
  const size_t total = (size_t)T_ * F;
  const int threads = 256;
  if (dtype == CCB_BF16 && (F % 8) == 0 && (B % 8) == 0 && ((reinterpret_cast<uintptr_t>(act) | reinterpret_cast<uintptr_t>(gate_up)) & 15) == 0) {
    const size_t total8 = total / 8;
    const size_t want = (total8 + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
    ccb_launch(silu_mul_bf16x8_kernel, blocks, threads, 0, stream, (uint4*)act, (const uint4*)gate_up, F / 8, B / 8,
               total8);
    return ccb_launch_status();
  }
  if (dtype == CCB_BF16 && (F % 2) == 0 && (B % 2) == 0) {
    const size_t total2 = total / 2;
    const int blocks = (int)((total2 + threads - 1) / threads < 148 * 16 ? (total2 + threads - 1) / threads : 148 * 16);
    ccb_launch(silu_mul_bf16x2_kernel, blocks, threads, 0, stream, (__nv_bfloat162*)act, (const __nv_bfloat162*)gate_up,
               F / 2, B / 2, total2);
    return ccb_launch_status();
  }
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (dtype == CCB_F32)
    ccb_launch(silu_mul_kernel<float>, blocks, threads, 0, stream, (float*)act, (const float*)gate_up, F, B, total);
  else if (dtype == CCB_BF16)
    ccb_launch(silu_mul_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (__nv_bfloat16*)act, (const __nv_bfloat16*)gate_up, F, B,
               total);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}
