// Paged causal attention over block tables, generic in every size.
//
//   q head h uses kv head h / (nq / nkv); s_j = (q . k_j) * scale;
//   a query at absolute position p sees keys j <= p (and, with a window W,
//   only p - j < W); o = sum_j softmax(s)_j v_j
//   (7QiC/ccInfer: src/kernel/attention/prefill_attn.cu:98-110, 145-241;
//    src/kernel/attention/decode_attn.cu:417-473).
//
// One block per (query token, q head), for prompt portions and decoded tokens
// alike: a token carries its own position and its request's block-table row,
// so the kernel does not know how the batch was cut.  Keys are visited in
// tiles of 32 aligned to absolute positions; warp w owns tiles w, w+4, ... and
// keeps a running (max, sum, accumulator); the four warps are merged in a
// fixed order.  The order of every sum therefore depends only on the query's
// position, never on the batch.  All arithmetic in float, accurate expf.
// Any head size that is a multiple of 16 up to 256, any page size.
#include "common.cuh"
#include <math_constants.h>

using namespace ccb;

constexpr int kAttnWarps = 4;
constexpr int kMaxDimsPerLane = 8;  // head sizes up to 256

__device__ __forceinline__ void load8(const float* p, float* o) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
  o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* o) {
  const uint4 r = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    o[2 * i] = f.x;
    o[2 * i + 1] = f.y;
  }
}

template <typename T>
__global__ void __launch_bounds__(kAttnWarps * 32)
paged_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_cache,
                               const T* __restrict__ v_cache, T* __restrict__ out,
                               const int* __restrict__ positions, const int* __restrict__ entry_of_token,
                               const int* __restrict__ block_table, int bt_stride, int n_entries, int nq, int nkv,
                               int hd, int page_size, int num_pages, int window, float scale, int* status) {
  ccb::pdl_begin();
  extern __shared__ float smem[];
  float* q_s = smem;                          // [hd]
  float* acc_s = smem + hd;                   // [warps][hd]
  float* m_s = acc_s + kAttnWarps * hd;       // [warps]
  float* l_s = m_s + kAttnWarps;              // [warps]

  const int t = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  T* o = out + ((size_t)t * nq + h) * hd;
  const int b = entry_of_token[t];
  const int p = positions[t];
  if (b < 0 || b >= n_entries || p < 0) {  // padded row
    for (int d = threadIdx.x; d < hd; d += blockDim.x) o[d] = from_f32<T>(0.f);
    return;
  }
  const int kvh = h / (nq / nkv);
  const int* bt = block_table + (size_t)b * bt_stride;
  const T* qr = q + ((size_t)t * nq + h) * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) q_s[d] = to_f32(qr[d]) * scale;
  __syncthreads();

  const int j0 = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;  // first visible key
  float m = -CUDART_INF_F, l = 0.f;
  float acc[kMaxDimsPerLane];
#pragma unroll
  for (int i = 0; i < kMaxDimsPerLane; ++i) acc[i] = 0.f;

  for (int tile = (j0 >> 5) + warp; tile * 32 <= p; tile += kAttnWarps) {
    const int j = tile * 32 + lane;
    bool valid = j >= j0 && j <= p;
    size_t row = 0;
    if (valid) {
      const int lp = j / page_size;
      const int page = lp < bt_stride ? bt[lp] : -1;
      if (page < 0 || page >= num_pages) {
        set_status(status, CCB_ST_BAD_PAGE);
        valid = false;
      } else {
        row = (((size_t)page * nkv + kvh) * page_size + (j - lp * page_size)) * hd;
      }
    }
    float s = -CUDART_INF_F;
    if (valid) {
      const T* kr = k_cache + row;
      float dot = 0.f;
      for (int d = 0; d < hd; d += 8) {
        float kv[8];
        load8(kr + d, kv);
#pragma unroll
        for (int e = 0; e < 8; ++e) dot = fmaf(q_s[d + e], kv[e], dot);
      }
      s = dot;
    }
    const float tile_max = warp_max(s);
    if (tile_max == -CUDART_INF_F) continue;  // nothing visible in this tile
    const float m_new = fmaxf(m, tile_max);
    const float corr = expf(m - m_new);  // 0 when m was -inf
    const float pj = valid ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(pj);
    m = m_new;
#pragma unroll
    for (int i = 0; i < kMaxDimsPerLane; ++i) acc[i] *= corr;
    for (int jj = 0; jj < 32; ++jj) {
      const float pw = __shfl_sync(0xffffffffu, pj, jj);
      const unsigned long long rw = __shfl_sync(0xffffffffu, (unsigned long long)row, jj);
      if (pw == 0.f) continue;  // uniform over the warp
      const T* vr = v_cache + rw;
#pragma unroll
      for (int i = 0; i < kMaxDimsPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] = fmaf(pw, to_f32(vr[d]), acc[i]);
      }
    }
  }

#pragma unroll
  for (int i = 0; i < kMaxDimsPerLane; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) acc_s[warp * hd + d] = acc[i];
  }
  if (lane == 0) {
    m_s[warp] = m;
    l_s[warp] = l;
  }
  __syncthreads();
  float mm = -CUDART_INF_F;
#pragma unroll
  for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, m_s[w]);
  if (mm == -CUDART_INF_F) {
    for (int d = threadIdx.x; d < hd; d += blockDim.x) o[d] = from_f32<T>(0.f);
    return;
  }
  float f[kAttnWarps], denom = 0.f;
#pragma unroll
  for (int w = 0; w < kAttnWarps; ++w) {
    f[w] = expf(m_s[w] - mm);
    denom += l_s[w] * f[w];
  }
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) v += acc_s[w * hd + d] * f[w];
    o[d] = from_f32<T>(v / denom);
  }
}

CCB_API int ccb_paged_attention_generic(const void* q, const void* k_cache, const void* v_cache, void* out,
                                        const int* positions, const int* entry_of_token, const int* block_table,
                                        int bt_stride, int n_entries, int T_, int nq, int nkv, int hd,
                                        int page_size, int num_pages, int window, float scale, int dtype,
                                        int* status, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (hd <= 0 || hd % 16 != 0 || hd > 32 * kMaxDimsPerLane || nq <= 0 || nkv <= 0 || nq % nkv != 0 ||
      page_size <= 0 || bt_stride <= 0)
    return CCB_REFUSE_SIZE;
  dim3 grid(T_, nq);
  const size_t smem = sizeof(float) * (hd + kAttnWarps * hd + 2 * kAttnWarps);
  if (dtype == CCB_F32)
    ccb_launch(paged_attention_generic_kernel<float>, grid, kAttnWarps * 32, smem, stream, 
        (const float*)q, (const float*)k_cache, (const float*)v_cache, (float*)out, positions, entry_of_token,
        block_table, bt_stride, n_entries, nq, nkv, hd, page_size, num_pages, window, scale, status);
  else if (dtype == CCB_BF16)
    ccb_launch(paged_attention_generic_kernel<__nv_bfloat16>, grid, kAttnWarps * 32, smem, stream, 
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
        (__nv_bfloat16*)out, positions, entry_of_token, block_table, bt_stride, n_entries, nq, nkv, hd, page_size,
        num_pages, window, scale, status);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}
