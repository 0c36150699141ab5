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

// The same with two neighbouring elements per lane and access (head size a multiple of 4): a warp reads
// and writes 128 (bfloat16) or 256 (float) contiguous bytes per instruction.
template <typename T> struct Pair2 {};
template <> struct Pair2<float> {
  static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
  static __device__ __forceinline__ void store(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
};
template <> struct Pair2<__nv_bfloat16> {
  static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float2 v) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y);
  }
};

template <typename T>
__global__ void qk_norm_rope_kv_write_vec_kernel(const T* __restrict__ qkv, int row_stride, T* __restrict__ q_out,
                                                 T* __restrict__ k_cache, T* __restrict__ v_cache,
                                                 const int* __restrict__ positions,
                                                 const int* __restrict__ slot_map, const float* __restrict__ inv_freq,
                                                 const float* __restrict__ q_w, const float* __restrict__ k_w,
                                                 float eps, int nq, int nkv, int hd, int page_size, int num_slots,
                                                 int heads_per_block, int* status) {
  ccb::pdl_begin();
  constexpr int kIters = 2;  // pairs of elements per lane: head sizes up to 256
  __shared__ float2 cs_table[128];  // (cos, sin) of this token's angles, shared by all heads of the block
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int half = hd >> 1;
  if (inv_freq != nullptr) {
    const float fpos_t = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      float sn, cs;
      sincosf(fpos_t * inv_freq[i], &sn, &cs);
      cs_table[i] = make_float2(cs, sn);
    }
  }
  __syncthreads();
  const int head_end = min(nq + 2 * nkv, (int)(blockIdx.y + 1) * heads_per_block);
  for (int head = blockIdx.y * heads_per_block + (threadIdx.x >> 5); head < head_end; head += (blockDim.x >> 5)) {
  const T* src = qkv + (size_t)t * row_stride + (size_t)head * hd;
  const bool is_q = head < nq;
  const bool is_k = !is_q && head < nq + nkv;
  T* dst;
  if (is_q) {
    dst = q_out + ((size_t)t * nq + head) * hd;
  } else {
    const int slot = slot_map[t];
    if (slot < 0) continue;
    if (slot >= num_slots) {
      if (lane == 0) set_status(status, CCB_ST_BAD_SLOT);
      continue;
    }
    const int kvh = is_k ? head - nq : head - nq - nkv;
    const int page = slot / page_size, off = slot - page * page_size;
    dst = (is_k ? k_cache : v_cache) + (((size_t)page * nkv + kvh) * page_size + off) * hd;
  }
  float2 x0[kIters], x1[kIters];
  float ss = 0.f;
#pragma unroll
  for (int m = 0; m < kIters; ++m) {
    const int i = 2 * lane + 64 * m;
    if (i < half) {
      x0[m] = Pair2<T>::load(src + i);
      x1[m] = Pair2<T>::load(src + i + half);
      ss += x0[m].x * x0[m].x + x0[m].y * x0[m].y + x1[m].x * x1[m].x + x1[m].y * x1[m].y;
    }
  }
  if (!is_q && !is_k) {
#pragma unroll
    for (int m = 0; m < kIters; ++m) {
      const int i = 2 * lane + 64 * m;
      if (i < half) {
        Pair2<T>::store(dst + i, x0[m]);
        Pair2<T>::store(dst + i + half, x1[m]);
      }
    }
    continue;
  }
  const float* w = is_q ? q_w : k_w;
  float inv = 1.f;
  if (w != nullptr) {
    ss = warp_sum(ss);
    inv = 1.0f / sqrtf(ss / (float)hd + eps);
  }
#pragma unroll
  for (int m = 0; m < kIters; ++m) {
    const int i = 2 * lane + 64 * m;
    if (i < half) {
      float a[2] = {x0[m].x, x0[m].y}, b[2] = {x1[m].x, x1[m].y};
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        if (w != nullptr) {
          a[e] = a[e] * inv * w[i + e];
          b[e] = b[e] * inv * w[i + e + half];
        }
        if (inv_freq != nullptr) {
          const float2 c = cs_table[i + e];
          const float ra = a[e] * c.x - b[e] * c.y;
          const float rb = b[e] * c.x + a[e] * c.y;
          a[e] = ra;
          b[e] = rb;
        }
      }
      Pair2<T>::store(dst + i, make_float2(a[0], a[1]));
      Pair2<T>::store(dst + i + half, make_float2(b[0], b[1]));
    }
  }
  }
}

// bfloat16 with 16-byte accesses: LPH lanes share a head (8 elements of each half per lane), so a warp works
// on 32 / LPH heads at once.  Head sizes 16 * LPH with LPH a power of two (128 -> 8 lanes).
template <int LPH>
__global__ void __launch_bounds__(128)
qk_norm_rope_kv_write_bf16x8_kernel(const __nv_bfloat16* __restrict__ qkv, int row_stride,
                                    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache,
                                    __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ positions,
                                    const int* __restrict__ slot_map, const float* __restrict__ inv_freq,
                                    const float* __restrict__ q_w, const float* __restrict__ k_w, float eps, int nq,
                                    int nkv, int page_size, int num_slots, int heads_per_block, int* status) {
  ccb::pdl_begin();
  constexpr int HD = 16 * LPH, HALF = 8 * LPH, HPW = 32 / LPH;
  __shared__ float2 cs_table[HALF];  // (cos, sin) of this token's angles, shared by all heads of the block
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (inv_freq != nullptr) {
    const float fpos_t = (float)positions[t];
    for (int i = threadIdx.x; i < HALF; i += blockDim.x) {
      float sn, cs;
      sincosf(fpos_t * inv_freq[i], &sn, &cs);
      cs_table[i] = make_float2(cs, sn);
    }
  }
  __syncthreads();
  const int sub = lane % LPH, i0 = 8 * sub;
  const int head_end = min(nq + 2 * nkv, (int)(blockIdx.y + 1) * heads_per_block);
  for (int head = blockIdx.y * heads_per_block + warp * HPW + lane / LPH; head < head_end; head += 4 * HPW) {
    const __nv_bfloat16* src = qkv + (size_t)t * row_stride + (size_t)head * HD;
    const bool is_q = head < nq;
    const bool is_k = !is_q && head < nq + nkv;
    __nv_bfloat16* dst;
    bool live = true;
    if (is_q) {
      dst = q_out + ((size_t)t * nq + head) * HD;
    } else {
      const int slot = slot_map[t];
      live = slot >= 0 && slot < num_slots;
      if (slot >= num_slots && sub == 0) set_status(status, CCB_ST_BAD_SLOT);
      const int kvh = is_k ? head - nq : head - nq - nkv;
      const int page = live ? slot / page_size : 0, off = live ? slot - page * page_size : 0;
      dst = (is_k ? k_cache : v_cache) + (((size_t)page * nkv + kvh) * page_size + off) * HD;
    }
    uint4 ra = make_uint4(0u, 0u, 0u, 0u), rb = ra;
    if (live) {
      ra = *reinterpret_cast<const uint4*>(src + i0);
      rb = *reinterpret_cast<const uint4*>(src + i0 + HALF);
    }
    if (!is_q && !is_k) {
      if (live) {
        *reinterpret_cast<uint4*>(dst + i0) = ra;
        *reinterpret_cast<uint4*>(dst + i0 + HALF) = rb;
      }
      continue;  // the lanes of a head take this branch together; the shuffles below name their lanes
    }
    float a[8], b[8];
    {
      const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ra);
      const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&rb);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 fa = __bfloat1622float2(pa[e]), fb = __bfloat1622float2(pb[e]);
        a[2 * e] = fa.x; a[2 * e + 1] = fa.y;
        b[2 * e] = fb.x; b[2 * e + 1] = fb.y;
      }
    }
    const float* w = is_q ? q_w : k_w;
    float inv = 1.f;
    if (w != nullptr) {
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += a[e] * a[e] + b[e] * b[e];
      // the lanes of one head: a butterfly inside their group (other groups may be elsewhere in the loop)
      const unsigned group_mask = LPH == 32 ? 0xffffffffu : (((1u << LPH) - 1u) << (lane - sub));
#pragma unroll
      for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(group_mask, ss, o);
      inv = 1.0f / sqrtf(ss / (float)HD + eps);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      if (w != nullptr) {
        a[e] = a[e] * inv * w[i0 + e];
        b[e] = b[e] * inv * w[i0 + e + HALF];
      }
      if (inv_freq != nullptr) {
        const float2 c = cs_table[i0 + e];
        const float xa = a[e] * c.x - b[e] * c.y;
        const float xb = b[e] * c.x + a[e] * c.y;
        a[e] = xa;
        b[e] = xb;
      }
    }
    if (live) {
      uint4 oa, ob;
      __nv_bfloat162* qa = reinterpret_cast<__nv_bfloat162*>(&oa);
      __nv_bfloat162* qb = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        qa[e] = __floats2bfloat162_rn(a[2 * e], a[2 * e + 1]);
        qb[e] = __floats2bfloat162_rn(b[2 * e], b[2 * e + 1]);
      }
      *reinterpret_cast<uint4*>(dst + i0) = oa;
      *reinterpret_cast<uint4*>(dst + i0 + HALF) = ob;
    }
  }
}

template <int LPH>
static void launch_x8(dim3 grid, cudaStream_t stream, const void* qkv, int row_stride, void* q_out, void* k_cache,
                      void* v_cache, const int* positions, const int* slot_map, const float* inv_freq,
                      const float* q_w, const float* k_w, float eps, int nq, int nkv, int page_size, int num_slots,
                      int hpb, int* status) {
  ccb_launch(qk_norm_rope_kv_write_bf16x8_kernel<LPH>, grid, 128, 0, stream, (const __nv_bfloat16*)qkv, row_stride,
             (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, positions, slot_map, inv_freq,
             q_w, k_w, eps, nq, nkv, page_size, num_slots, hpb, status);
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
  // two elements per access where every pointer and stride allows it
  const bool vec = (hd % 4 == 0) && (row_stride % 2 == 0) &&
                   ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) |
                     reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 7) == 0;
  // few tokens: many small blocks; many tokens: 16 heads a block, so the angles are computed 16x less often
  const int hpb = T_ <= 64 ? 4 : 16;
  dim3 vgrid(T_, (heads + hpb - 1) / hpb);
  // bfloat16, many tokens, head sizes 32 .. 256 that are 16 x a power of two: 16-byte accesses
  const bool x8 = dtype == CCB_BF16 && T_ > 64 && (hd == 32 || hd == 64 || hd == 128 || hd == 256) &&
                  (row_stride % 8 == 0) &&
                  ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) |
                    reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15) == 0;
  if (x8) {
    const int lph = hd / 16;
    const int per_pass = 4 * (32 / lph);              // heads a block of four warps takes at once
    const int hpb8 = per_pass * ((16 + per_pass - 1) / per_pass);
    dim3 g8(T_, (heads + hpb8 - 1) / hpb8);
#define CCB_X8(L)                                                                                                  \
  launch_x8<L>(g8, stream, qkv, row_stride, q_out, k_cache, v_cache, positions, slot_map, inv_freq, q_w, k_w, eps, \
               nq, nkv, page_size, num_slots, hpb8, status)
    if (lph == 2) CCB_X8(2);
    else if (lph == 4) CCB_X8(4);
    else if (lph == 8) CCB_X8(8);
    else CCB_X8(16);
#undef CCB_X8
    return ccb_launch_status();
  }
  if (vec && dtype == CCB_F32) {
    ccb_launch(qk_norm_rope_kv_write_vec_kernel<float>, vgrid, 128, 0, stream, (const float*)qkv, row_stride,
               (float*)q_out, (float*)k_cache, (float*)v_cache, positions, slot_map, inv_freq, q_w, k_w, eps, nq, nkv,
               hd, page_size, num_slots, hpb, status);
    return ccb_launch_status();
  }
  if (vec && dtype == CCB_BF16) {
    ccb_launch(qk_norm_rope_kv_write_vec_kernel<__nv_bfloat16>, vgrid, 128, 0, stream, (const __nv_bfloat16*)qkv,
               row_stride, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, positions,
               slot_map, inv_freq, q_w, k_w, eps, nq, nkv, hd, page_size, num_slots, hpb, status);
    return ccb_launch_status();
  }
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
