// RMSNorm, alone and fused with the residual sum.
//
//   y = x * rsqrt(mean(x^2) + eps) * w          (7QiC/ccInfer: src/kernel/norm/rms_norm.cu:24-60)
//   h <- h + delta                              (7QiC/ccInfer: src/kernel/elementwise/elementwise.cu:13-24)
//
// The residual stream h is kept in float in both paths, the sum of squares is
// a plain float sum in a fixed order (the reference's bfloat16-rounded running
// sum is a parity trick for another oracle and is not reproduced), and w is a
// float vector.  One block per row.
#include "common.cuh"

using namespace ccb;

constexpr int kNormThreads = 256;

// y[r, :] = norm(h[src, :] + delta[src, :]) * w, src = row_idx ? row_idx[r] : r.
// With write_h the sum is stored back to h (only without row_idx).
template <typename T>
__global__ void residual_rmsnorm_kernel(T* __restrict__ y, float* __restrict__ h, const T* __restrict__ delta,
                                        const float* __restrict__ w, const int* __restrict__ row_idx,
                                        int n_src_rows, int D, float eps, int write_h, int* status) {
  ccb::pdl_begin();
  __shared__ float red[32];
  const int r = blockIdx.x;
  int src = row_idx ? row_idx[r] : r;
  T* yr = y + (size_t)r * D;
  if (src < 0 || src >= n_src_rows) {
    if (threadIdx.x == 0) set_status(status, CCB_ST_BAD_ROW);
    for (int d = threadIdx.x; d < D; d += kNormThreads) yr[d] = from_f32<T>(0.f);
    return;
  }
  float* hr = h + (size_t)src * D;
  const T* dr = delta ? delta + (size_t)src * D : nullptr;
  float ss = 0.f;
  for (int d = threadIdx.x; d < D; d += kNormThreads) {
    float v = hr[d];
    if (dr) {
      v += to_f32(dr[d]);
      if (write_h) hr[d] = v;
    }
    ss += v * v;
  }
  ss = block_sum<kNormThreads>(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)D + eps);
  for (int d = threadIdx.x; d < D; d += kNormThreads) {
    float v = hr[d];
    if (dr && !write_h) v += to_f32(dr[d]);
    yr[d] = from_f32<T>(v * inv * w[d]);
  }
}

// The same for D a multiple of 4 up to 8192: the row is read once with 16-byte loads and kept in registers
// between the sum of squares and the scaling.  The order of the sum (per thread in ascending d, then the
// block's fixed tree) differs from the kernel above only in which thread adds which element.
constexpr int kNormVecs = 8;

template <typename T> struct Vec4 {};
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 r;
    r.x = *reinterpret_cast<const uint32_t*>(&a);
    r.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
  }
};

template <typename T>
__global__ void __launch_bounds__(kNormThreads)
residual_rmsnorm_vec_kernel(T* __restrict__ y, float* __restrict__ h, const T* __restrict__ delta,
                            const float* __restrict__ w, const int* __restrict__ row_idx, int n_src_rows, int D,
                            float eps, int write_h, int* status) {
  ccb::pdl_begin();
  __shared__ float red[32];
  const int r = blockIdx.x;
  const int src = row_idx ? row_idx[r] : r;
  T* yr = y + (size_t)r * D;
  const int nvec = D >> 2;
  if (src < 0 || src >= n_src_rows) {
    if (threadIdx.x == 0) set_status(status, CCB_ST_BAD_ROW);
    for (int i = threadIdx.x; i < nvec; i += kNormThreads) Vec4<T>::store(yr + 4 * i, make_float4(0.f, 0.f, 0.f, 0.f));
    return;
  }
  float* hr = h + (size_t)src * D;
  const T* dr = delta ? delta + (size_t)src * D : nullptr;
  float4 v[kNormVecs], g[kNormVecs];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kNormVecs; ++j) {   // the weights are asked for with the row, not after the sum
    const int i = threadIdx.x + j * kNormThreads;
    if (i < nvec) g[j] = Vec4<float>::load(w + 4 * i);
  }
#pragma unroll
  for (int j = 0; j < kNormVecs; ++j) {
    const int i = threadIdx.x + j * kNormThreads;
    if (i < nvec) {
      float4 a = Vec4<float>::load(hr + 4 * i);
      if (dr) {
        const float4 d = Vec4<T>::load(dr + 4 * i);
        a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
        if (write_h) Vec4<float>::store(hr + 4 * i, a);
      }
      v[j] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  ss = block_sum<kNormThreads>(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
  for (int j = 0; j < kNormVecs; ++j) {
    const int i = threadIdx.x + j * kNormThreads;
    if (i < nvec)
      Vec4<T>::store(yr + 4 * i, make_float4(v[j].x * inv * g[j].x, v[j].y * inv * g[j].y, v[j].z * inv * g[j].z,
                                             v[j].w * inv * g[j].w));
  }
}

CCB_API int ccb_residual_rmsnorm(void* y, float* h, const void* delta, const float* w, const int* row_idx,
                                 int rows, int n_src_rows, int D, float eps, int dtype, int* status,
                                 cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D <= 0) return CCB_REFUSE_SIZE;
  const int write_h = (delta != nullptr && row_idx == nullptr) ? 1 : 0;
  const bool vec = (D % 4 == 0) && D <= 4 * kNormVecs * kNormThreads &&
                   ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(h) |
                     reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(w)) & 15) == 0;
  if (vec && dtype == CCB_F32) {
    ccb_launch(residual_rmsnorm_vec_kernel<float>, rows, kNormThreads, 0, stream, 
        (float*)y, h, (const float*)delta, w, row_idx, n_src_rows, D, eps, write_h, status);
    return ccb_launch_status();
  }
  if (vec && dtype == CCB_BF16) {
    ccb_launch(residual_rmsnorm_vec_kernel<__nv_bfloat16>, rows, kNormThreads, 0, stream, 
        (__nv_bfloat16*)y, h, (const __nv_bfloat16*)delta, w, row_idx, n_src_rows, D, eps, write_h, status);
    return ccb_launch_status();
  }
  if (dtype == CCB_F32)
    ccb_launch(residual_rmsnorm_kernel<float>, rows, kNormThreads, 0, stream, 
        (float*)y, h, (const float*)delta, w, row_idx, n_src_rows, D, eps, write_h, status);
  else if (dtype == CCB_BF16)
    ccb_launch(residual_rmsnorm_kernel<__nv_bfloat16>, rows, kNormThreads, 0, stream, 
        (__nv_bfloat16*)y, h, (const __nv_bfloat16*)delta, w, row_idx, n_src_rows, D, eps, write_h, status);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

// The first layer's norm together with the embedding: h[t, :] = float(table[ids[t], :]) and
// y[t, :] = norm(h[t, :]) * w in one pass (7QiC/ccInfer runs the gather, src/kernel/elementwise/elementwise.cu:67-78,
// and the norm as two kernels).  An id of -1 - s stands for pending[s], as in embed_gather.
template <typename T>
__global__ void __launch_bounds__(kNormThreads)
embed_rmsnorm_kernel(T* __restrict__ y, float* __restrict__ h, const T* __restrict__ table, const int* __restrict__ ids,
                     const float* __restrict__ w, int D, int V, float eps, const int* __restrict__ pending,
                     int n_pending, int vec, int* status) {
  ccb::pdl_begin();
  __shared__ float red[32];
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 && pending != nullptr && -1 - id < n_pending) id = pending[-1 - id];
  float* hr = h + (size_t)t * D;
  T* yr = y + (size_t)t * D;
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) set_status(status, CCB_ST_BAD_TOKEN);
    for (int d = threadIdx.x; d < D; d += kNormThreads) {
      hr[d] = 0.f;
      yr[d] = from_f32<T>(0.f);
    }
    return;
  }
  const T* row = table + (size_t)id * D;
  float ss = 0.f;
  if (vec) {   // D a multiple of 4 and at most 4 kNormVecs kNormThreads, everything 16-byte aligned
    const int nvec = D >> 2;
    float4 v[kNormVecs], g[kNormVecs];
#pragma unroll
    for (int j = 0; j < kNormVecs; ++j) {
      const int i = threadIdx.x + j * kNormThreads;
      if (i < nvec) {
        g[j] = Vec4<float>::load(w + 4 * i);
        v[j] = Vec4<T>::load(row + 4 * i);
        Vec4<float>::store(hr + 4 * i, v[j]);
        ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
      }
    }
    ss = block_sum<kNormThreads>(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
    for (int j = 0; j < kNormVecs; ++j) {
      const int i = threadIdx.x + j * kNormThreads;
      if (i < nvec)
        Vec4<T>::store(yr + 4 * i, make_float4(v[j].x * inv * g[j].x, v[j].y * inv * g[j].y, v[j].z * inv * g[j].z,
                                               v[j].w * inv * g[j].w));
    }
    return;
  }
  for (int d = threadIdx.x; d < D; d += kNormThreads) {
    const float v = to_f32(row[d]);
    hr[d] = v;
    ss += v * v;
  }
  ss = block_sum<kNormThreads>(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)D + eps);
  for (int d = threadIdx.x; d < D; d += kNormThreads) yr[d] = from_f32<T>(to_f32(row[d]) * inv * w[d]);
}

CCB_API int ccb_embed_rmsnorm(void* y, float* h, const void* table, const int* ids, const float* w, int rows, int D,
                              int V, float eps, int dtype, const int* pending, int n_pending, int* status,
                              cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D <= 0 || V <= 0) return CCB_REFUSE_SIZE;
  const int esize = dtype == CCB_F32 ? 4 : 2;
  const int vec = (D % 4 == 0) && D <= 4 * kNormVecs * kNormThreads && ((size_t)D * esize) % 8 == 0 &&
                  ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(table) |
                    reinterpret_cast<uintptr_t>(w)) & 15) == 0;
  if (dtype == CCB_F32)
    ccb_launch(embed_rmsnorm_kernel<float>, rows, kNormThreads, 0, stream, (float*)y, h, (const float*)table, ids, w,
               D, V, eps, pending, n_pending, vec, status);
  else if (dtype == CCB_BF16)
    ccb_launch(embed_rmsnorm_kernel<__nv_bfloat16>, rows, kNormThreads, 0, stream, (__nv_bfloat16*)y, h,
               (const __nv_bfloat16*)table, ids, w, D, V, eps, pending, n_pending, vec, status);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

// Plain RMSNorm over the last axis of a [rows, D] tensor of the storage type.
template <typename T>
__global__ void rmsnorm_kernel(T* __restrict__ y, const T* __restrict__ x, const float* __restrict__ w, int D,
                               float eps) {
  ccb::pdl_begin();
  __shared__ float red[32];
  const T* xr = x + (size_t)blockIdx.x * D;
  T* yr = y + (size_t)blockIdx.x * D;
  float ss = 0.f;
  for (int d = threadIdx.x; d < D; d += kNormThreads) {
    const float v = to_f32(xr[d]);
    ss += v * v;
  }
  ss = block_sum<kNormThreads>(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)D + eps);
  for (int d = threadIdx.x; d < D; d += kNormThreads) yr[d] = from_f32<T>(to_f32(xr[d]) * inv * w[d]);
}

CCB_API int ccb_rmsnorm(void* y, const void* x, const float* w, int rows, int D, float eps, int dtype,
                        cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D <= 0) return CCB_REFUSE_SIZE;
  if (dtype == CCB_F32)
    ccb_launch(rmsnorm_kernel<float>, rows, kNormThreads, 0, stream, (float*)y, (const float*)x, w, D, eps);
  else if (dtype == CCB_BF16)
    ccb_launch(rmsnorm_kernel<__nv_bfloat16>, rows, kNormThreads, 0, stream, (__nv_bfloat16*)y, (const __nv_bfloat16*)x, w, D, eps);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}
