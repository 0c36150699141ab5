// Per-head q/k RMSNorm, rotate-half position encoding and the write of k and v
// into their cache pages, in one pass over the merged projection output.
//
//   q^ = RMSNorm_hd(q; wq), k^ = RMSNorm_hd(k; wk)      (7QiC/ccInfer: src/model/qwen3/qwen3_model.cpp:189-211)
//   angle_i = float(pos) * inv_freq[i], pairs (i, i + hd/2):
//   x_i' = x_i cos - x_{i+hd/2} sin ; x_{i+hd/2}' = x_{i+hd/2} cos + x_i sin
//                                                       (src/kernel/pos/rope.cu:41-46, src/model/rope/rope_cache.cpp:38-45)
//   Kc[slot, h, :] = k^', Vc[slot, h, :] = v            (src/kernel/attention/write_kv_cache.cu:12-34)
//
// One warp per (token, head); the norm weights and the frequency table are
// optional (null = that step is left out), so the same kernel serves a mixer
// without head norms or without rotation.  Cache layout: [page, kv head,
// token in page, hd], slot = page * page_size + token in page.
#include "common.cuh"

using namespace ccb;

constexpr int kMaxPairsPerLane = 4;  // head sizes up to 256

template <typename T>
__global__ void qk_norm_rope_kv_write_kernel(const T* __restrict__ qkv, int row_stride, T* __restrict__ q_out,
                                             T* __restrict__ k_cache, T* __restrict__ v_cache,
                                             const int* __restrict__ positions, const int* __restrict__ slot_map,
                                             const float* __restrict__ inv_freq, const float* __restrict__ q_w,
                                             const float* __restrict__ k_w, float eps, int nq, int nkv, int hd,
                                             int page_size, int num_slots, int* status) {
  ccb::pdl_begin();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (head >= nq + 2 * nkv) return;
  const int half = hd >> 1;
  const T* src = qkv + (size_t)t * row_stride + (size_t)head * hd;

  const bool is_q = head < nq;
  const bool is_k = !is_q && head < nq + nkv;
  T* dst;
  if (is_q) {
    dst = q_out + ((size_t)t * nq + head) * hd;
  } else {
    const int slot = slot_map[t];
    if (slot < 0) return;  // padded row: nothing is cached
    if (slot >= num_slots) {
      if (lane == 0) set_status(status, CCB_ST_BAD_SLOT);
      return;
    }
    const int kvh = is_k ? head - nq : head - nq - nkv;
    const int page = slot / page_size, off = slot - page * page_size;
    T* base = is_k ? k_cache : v_cache;
    dst = base + (((size_t)page * nkv + kvh) * page_size + off) * hd;
  }

  float x0[kMaxPairsPerLane], x1[kMaxPairsPerLane];
  float ss = 0.f;
#pragma unroll
  for (int m = 0; m < kMaxPairsPerLane; ++m) {
    const int i = lane + 32 * m;
    if (i < half) {
      x0[m] = to_f32(src[i]);
      x1[m] = to_f32(src[i + half]);
      ss += x0[m] * x0[m] + x1[m] * x1[m];
    }
  }
  if (!is_q && !is_k) {  // v: plain copy
#pragma unroll
    for (int m = 0; m < kMaxPairsPerLane; ++m) {
      const int i = lane + 32 * m;
      if (i < half) {
        dst[i] = from_f32<T>(x0[m]);
        dst[i + half] = from_f32<T>(x1[m]);
      }
    }
    return;
  }
  const float* w = is_q ? q_w : k_w;
  float inv = 1.f;
  if (w != nullptr) {
    ss = warp_sum(ss);
    inv = 1.0f / sqrtf(ss / (float)hd + eps);
  }
  const float fpos = (float)positions[t];
#pragma unroll
  for (int m = 0; m < kMaxPairsPerLane; ++m) {
    const int i = lane + 32 * m;
    if (i < half) {
      float a = x0[m], b = x1[m];
      if (w != nullptr) {
        a = a * inv * w[i];
        b = b * inv * w[i + half];
      }
      if (inv_freq != nullptr) {
        float s, c;
        sincosf(fpos * inv_freq[i], &s, &c);
        const float ra = a * c - b * s;
        const float rb = b * c + a * s;
        a = ra;
        b = rb;
      }
      dst[i] = from_f32<T>(a);
      dst[i + half] = from_f32<T>(b);
    }
  }
}

CCB_API int ccb_qk_norm_rope_kv_write(const void* qkv, int row_stride, void* q_out, void* k_cache, void* v_cache,
                                      const int* positions, const int* slot_map, const float* inv_freq,
                                      const float* q_w, const float* k_w, float eps, int T_, int nq, int nkv,
                                      int hd, int page_size, int num_slots, int dtype, int* status,
                                      cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (hd <= 0 || (hd & 1) || hd > 64 * kMaxPairsPerLane || nq < 0 || nkv < 0 || nq + nkv == 0 || page_size <= 0)
    return CCB_REFUSE_SIZE;
  if (nkv > 0 && (k_cache == nullptr || v_cache == nullptr || slot_map == nullptr)) return CCB_REFUSE_ARG;
  const int heads = nq + 2 * nkv;
  dim3 grid(T_, (heads + 3) / 4);
  if (dtype == CCB_F32)
    ccb_launch(qk_norm_rope_kv_write_kernel<float>, grid, 128, 0, stream, 
        (const float*)qkv, row_stride, (float*)q_out, (float*)k_cache, (float*)v_cache, positions, slot_map,
        inv_freq, q_w, k_w, eps, nq, nkv, hd, page_size, num_slots, status);
  else if (dtype == CCB_BF16)
    ccb_launch(qk_norm_rope_kv_write_kernel<__nv_bfloat16>, grid, 128, 0, stream, 
        (const __nv_bfloat16*)qkv, row_stride, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache,
        (__nv_bfloat16*)v_cache, positions, slot_map, inv_freq, q_w, k_w, eps, nq, nkv, hd, page_size, num_slots,
        status);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}
