// Paged attention for single query tokens with the key range split over several blocks
// (decoding, short portions, and the whole of the 32-bit path).
//
//   s_j = (q . k_j) * scale over the visible keys j0 .. p of the token's request, softmax, o = P v
//   (7QiC/ccInfer: src/kernel/attention/decode_attn.cu:417-473).  The reference keeps all scores of a
//   request in shared memory (two passes, context <= 24,576) and runs one block per (request, q head);
//   here the softmax is online, a block serves up to four q heads of one kv head so that keys and
//   values are read once for the group, and the key range of a token is cut into `num_splits` pieces
//   that run in parallel and are merged afterwards, which keeps all SMs busy at batch 1.
//
// Block = (token row, kv head x head chunk, split), 4 warps.  Keys are taken in tiles of 16 aligned to
// absolute positions; a tile belongs to split (tile - first_tile) / tiles_per_split and, inside the
// block, to warp (tile % 4).  Within a warp 8 lanes share a key (each holds 8-element pieces of the
// head), 4 keys go side by side.  All arithmetic in float.  Partial results (running maximum, sum,
// unnormalised accumulator) of the splits go to scratch memory and are merged in a fixed order by
// ccb_attention_merge; with one split the block writes the output itself.
#include "common.cuh"
#include <math_constants.h>
#include <type_traits>

using namespace ccb;

namespace {

constexpr int kWarps = 4;
constexpr int kIt = 4;             // keys per lane group and tile
constexpr int kTile = 4 * kIt;      // keys per tile (4 lane groups side by side)
constexpr int kTileShift = 4;

__device__ __forceinline__ void load8(const float* p, float* o) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p + 4));
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
  o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* o) {
  const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    o[2 * i] = f.x;
    o[2 * i + 1] = f.y;
  }
}

template <typename T> __device__ __forceinline__ float exp_of(float x);
template <> __device__ __forceinline__ float exp_of<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ float exp_of<__nv_bfloat16>(float x) { return __expf(x); }

// GT: q heads per block; NV: 8-element pieces of the head per lane (head size <= 64 * NV)
template <typename T, int GT, int NV>
__global__ void __launch_bounds__(kWarps * 32)
attention_split_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                       T* __restrict__ out, float* __restrict__ part_acc, float* __restrict__ part_ml,
                       const int* __restrict__ positions, const int* __restrict__ entry_of_token,
                       const int* __restrict__ block_table, int bt_stride, int n_entries, int row0, int nq, int nkv,
                       int hd, int page_size, int num_pages, int window, float scale, int num_splits,
                       int* status) {
  ccb::pdl_begin();
  extern __shared__ float smem[];  // [warps][GT][hd] accumulators, then [warps][GT] max, [warps][GT] sum
  const int G = nq / nkv;
  const int gchunks = (G + GT - 1) / GT;
  const int split = blockIdx.z;
  const int kvh = blockIdx.y / gchunks, gc = blockIdx.y - kvh * gchunks;
  const int r = blockIdx.x, t = row0 + r;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int kg = lane >> 3, dc = lane & 7;  // key slot in the warp, piece of the head
  const int h0 = kvh * G + gc * GT;         // first q head of this block
  const int n_heads = min(GT, G - gc * GT);

  const int b = entry_of_token[t];
  const int p = positions[t];
  const bool padded = b < 0 || b >= n_entries || p < 0;

  float m[GT], l[GT], acc[GT][NV][8], qr[GT][NV][8];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    m[g] = -CUDART_INF_F;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][i][e] = 0.f;
  }

  if (!padded) {
#pragma unroll
    for (int g = 0; g < GT; ++g)
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int d = (dc + 8 * i) * 8;
        if (g < n_heads && d < hd) {
          load8(q + ((size_t)t * nq + h0 + g) * hd + d, qr[g][i]);
#pragma unroll
          for (int e = 0; e < 8; ++e) qr[g][i][e] *= scale;
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) qr[g][i][e] = 0.f;
        }
      }
    const int* bt = block_table + (size_t)b * bt_stride;
    const int j0 = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int first_tile = j0 >> kTileShift, last_tile = p >> kTileShift;
    const int n_tiles = last_tile - first_tile + 1;
    const int per_split = (n_tiles + num_splits - 1) / num_splits;
    const int my_first = first_tile + split * per_split;
    const int my_end = min(my_first + per_split, last_tile + 1);
    // the first tile of this warp: the smallest tile >= my_first with tile % kWarps == warp
    int tile = my_first + ((warp - my_first) & (kWarps - 1));
    for (; tile < my_end; tile += kWarps) {
      float s[GT][kIt];
      size_t rows[kIt];
      bool valid[kIt];
#pragma unroll
      for (int it = 0; it < kIt; ++it) {
        const int j = tile * kTile + it * 4 + kg;
        valid[it] = j >= j0 && j <= p;
        rows[it] = 0;
        if (valid[it]) {
          const int lp = j / page_size;
          const int page = lp < bt_stride ? bt[lp] : -1;
          if (page < 0 || page >= num_pages) {
            set_status(status, CCB_ST_BAD_PAGE);
            valid[it] = false;
          } else {
            rows[it] = (((size_t)page * nkv + kvh) * page_size + (j - lp * page_size)) * hd;
          }
        }
      }
#pragma unroll
      for (int it = 0; it < kIt; ++it) {
        float dot[GT];
#pragma unroll
        for (int g = 0; g < GT; ++g) dot[g] = 0.f;
        if (valid[it]) {
#pragma unroll
          for (int i = 0; i < NV; ++i) {
            const int d = (dc + 8 * i) * 8;
            if (d < hd) {
              float kv[8];
              load8(k_cache + rows[it] + d, kv);
#pragma unroll
              for (int g = 0; g < GT; ++g)
#pragma unroll
                for (int e = 0; e < 8; ++e) dot[g] = fmaf(qr[g][i][e], kv[e], dot[g]);
            }
          }
        }
#pragma unroll
        for (int g = 0; g < GT; ++g) {
          float v = dot[g];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          v += __shfl_xor_sync(0xffffffffu, v, 4);
          s[g][it] = valid[it] ? v : -CUDART_INF_F;
        }
      }
      float corr[GT];
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        float tm = s[g][0];
#pragma unroll
        for (int it = 1; it < kIt; ++it) tm = fmaxf(tm, s[g][it]);
        tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 8));
        tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 16));
        const float m_new = fmaxf(m[g], tm);
        float ls = 0.f;
        if (m_new == -CUDART_INF_F) {  // nothing visible yet
          corr[g] = 1.f;
#pragma unroll
          for (int it = 0; it < kIt; ++it) s[g][it] = 0.f;
        } else {
          corr[g] = exp_of<T>(m[g] - m_new);  // 0 when m was -inf
#pragma unroll
          for (int it = 0; it < kIt; ++it) {
            s[g][it] = valid[it] ? exp_of<T>(s[g][it] - m_new) : 0.f;
            ls += s[g][it];
          }
        }
        ls += __shfl_xor_sync(0xffffffffu, ls, 8);
        ls += __shfl_xor_sync(0xffffffffu, ls, 16);
        l[g] = l[g] * corr[g] + ls;
        m[g] = m_new;
#pragma unroll
        for (int i = 0; i < NV; ++i)
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[g][i][e] *= corr[g];
      }
#pragma unroll
      for (int it = 0; it < kIt; ++it) {
        if (!valid[it]) continue;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int d = (dc + 8 * i) * 8;
          if (d < hd) {
            float vv[8];
            load8(v_cache + rows[it] + d, vv);
#pragma unroll
            for (int g = 0; g < GT; ++g)
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[g][i][e] = fmaf(s[g][it], vv[e], acc[g][i][e]);
          }
        }
      }
    }
    // the four key slots of the warp hold partial accumulators of the same maximum: add them
#pragma unroll
    for (int g = 0; g < GT; ++g)
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float v = acc[g][i][e];
          v += __shfl_xor_sync(0xffffffffu, v, 8);
          v += __shfl_xor_sync(0xffffffffu, v, 16);
          acc[g][i][e] = v;
        }
  }

  float* acc_s = smem;
  float* m_s = smem + kWarps * GT * hd;
  float* l_s = m_s + kWarps * GT;
  if (kg == 0) {
#pragma unroll
    for (int g = 0; g < GT; ++g)
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int d = (dc + 8 * i) * 8;
        if (d < hd) {
#pragma unroll
          for (int e = 0; e < 8; ++e) acc_s[(warp * GT + g) * hd + d + e] = acc[g][i][e];
        }
      }
  }
  if (lane == 0) {
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      m_s[warp * GT + g] = m[g];
      l_s[warp * GT + g] = l[g];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < n_heads * hd; idx += blockDim.x) {
    const int g = idx / hd, d = idx - g * hd;
    float mm = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, m_s[w * GT + g]);
    float a = 0.f, ll = 0.f;
    if (mm != -CUDART_INF_F) {
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const float f = exp_of<T>(m_s[w * GT + g] - mm);
        a += acc_s[(w * GT + g) * hd + d] * f;
        ll += l_s[w * GT + g] * f;
      }
    }
    const int h = h0 + g;
    if (num_splits == 1) {
      out[((size_t)t * nq + h) * hd + d] = from_f32<T>(ll > 0.f ? a / ll : 0.f);
    } else {
      const size_t slot = ((size_t)r * nq + h) * num_splits + split;
      part_acc[slot * hd + d] = a;
      if (d == 0) {
        part_ml[slot * 2] = mm;
        part_ml[slot * 2 + 1] = ll;
      }
    }
  }
}

template <typename T>
__global__ void attention_merge_kernel(T* __restrict__ out, const float* __restrict__ part_acc,
                                       const float* __restrict__ part_ml, int row0, int nq, int hd, int num_splits) {
  ccb::pdl_begin();
  const int r = blockIdx.x, h = blockIdx.y;
  const size_t base = ((size_t)r * nq + h) * num_splits;
  float mm = -CUDART_INF_F;
  for (int s = 0; s < num_splits; ++s) mm = fmaxf(mm, part_ml[(base + s) * 2]);
  T* o = out + ((size_t)(row0 + r) * nq + h) * hd;
  if (mm == -CUDART_INF_F) {
    for (int d = threadIdx.x; d < hd; d += blockDim.x) o[d] = from_f32<T>(0.f);
    return;
  }
  float ll = 0.f;
  for (int s = 0; s < num_splits; ++s) ll += part_ml[(base + s) * 2 + 1] * exp_of<T>(part_ml[(base + s) * 2] - mm);
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < num_splits; ++s)
      a += part_acc[(base + s) * hd + d] * exp_of<T>(part_ml[(base + s) * 2] - mm);
    o[d] = from_f32<T>(a / ll);
  }
}

template <typename T, int GT, int NV>
int launch_split(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_acc, float* part_ml,
                 const int* positions, const int* entry_of_token, const int* block_table, int bt_stride,
                 int n_entries, int row0, int n_rows, int nq, int nkv, int hd, int page_size, int num_pages,
                 int window, float scale, int num_splits, int* status, cudaStream_t stream) {
  const int G = nq / nkv, gchunks = (G + GT - 1) / GT;
  dim3 grid(n_rows, nkv * gchunks, num_splits);
  const size_t smem = sizeof(float) * (kWarps * GT * hd + 2 * kWarps * GT);
  ccb_launch(attention_split_kernel<T, GT, NV>, grid, kWarps * 32, smem, stream, 
      (const T*)q, (const T*)k_cache, (const T*)v_cache, (T*)out, part_acc, part_ml, positions, entry_of_token,
      block_table, bt_stride, n_entries, row0, nq, nkv, hd, page_size, num_pages, window, scale, num_splits, status);
  int rc = ccb_launch_status();
  if (rc != 0 || num_splits == 1) return rc;
  if (std::is_same<T, float>::value)
    ccb_launch(attention_merge_kernel<float>, dim3(n_rows, nq), 128, 0, stream, (float*)out, part_acc, part_ml, row0, nq, hd,
                                                                         num_splits);
  else
    ccb_launch(attention_merge_kernel<__nv_bfloat16>, dim3(n_rows, nq), 128, 0, stream, (__nv_bfloat16*)out, part_acc,
                                                                                 part_ml, row0, nq, hd, num_splits);
  return ccb_launch_status();
}

template <typename T, int GT>
int pick_nv(int hd, const void* q, const void* k, const void* v, void* out, float* pa, float* pm, const int* pos,
            const int* eot, const int* bt, int bts, int ne, int row0, int n_rows, int nq, int nkv, int ps, int np,
            int window, float scale, int splits, int* status, cudaStream_t st) {
  if (hd <= 64)
    return launch_split<T, GT, 1>(q, k, v, out, pa, pm, pos, eot, bt, bts, ne, row0, n_rows, nq, nkv, hd, ps, np,
                                  window, scale, splits, status, st);
  if (hd <= 128)
    return launch_split<T, GT, 2>(q, k, v, out, pa, pm, pos, eot, bt, bts, ne, row0, n_rows, nq, nkv, hd, ps, np,
                                  window, scale, splits, status, st);
  return launch_split<T, GT, 4>(q, k, v, out, pa, pm, pos, eot, bt, bts, ne, row0, n_rows, nq, nkv, hd, ps, np,
                                window, scale, splits, status, st);
}

template <typename T>
int pick_gt(int hd, const void* q, const void* k, const void* v, void* out, float* pa, float* pm, const int* pos,
            const int* eot, const int* bt, int bts, int ne, int row0, int n_rows, int nq, int nkv, int ps, int np,
            int window, float scale, int splits, int* status, cudaStream_t st) {
  const int G = nq / nkv;
  // wide heads keep fewer q heads per block so that the accumulators stay in registers
  if (G >= 4 && hd <= 128)
    return pick_nv<T, 4>(hd, q, k, v, out, pa, pm, pos, eot, bt, bts, ne, row0, n_rows, nq, nkv, ps, np, window,
                         scale, splits, status, st);
  if (G >= 2)
    return pick_nv<T, 2>(hd, q, k, v, out, pa, pm, pos, eot, bt, bts, ne, row0, n_rows, nq, nkv, ps, np, window,
                         scale, splits, status, st);
  return pick_nv<T, 1>(hd, q, k, v, out, pa, pm, pos, eot, bt, bts, ne, row0, n_rows, nq, nkv, ps, np, window,
                       scale, splits, status, st);
}

}  // namespace

// Scratch: part_acc holds n_rows * nq * num_splits * hd floats, part_ml n_rows * nq * num_splits * 2
// (both unused with one split).  Rows row0 .. row0 + n_rows - 1 of q / out / positions are handled.
CCB_API int ccb_attention_split(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_acc,
                                float* part_ml, const int* positions, const int* entry_of_token,
                                const int* block_table, int bt_stride, int n_entries, int row0, int n_rows, int nq,
                                int nkv, int hd, int page_size, int num_pages, int window, float scale,
                                int num_splits, int dtype, int* status, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hd <= 0 || hd % 8 != 0 || hd > 256 || nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0 ||
      bt_stride <= 0 || num_splits <= 0 || num_splits > 64)
    return CCB_REFUSE_SIZE;
  if (num_splits > 1 && (part_acc == nullptr || part_ml == nullptr)) return CCB_REFUSE_ARG;
  if (dtype == CCB_F32)
    return pick_gt<float>(hd, q, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token, block_table,
                          bt_stride, n_entries, row0, n_rows, nq, nkv, page_size, num_pages, window, scale,
                          num_splits, status, stream);
  if (dtype == CCB_BF16)
    return pick_gt<__nv_bfloat16>(hd, q, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token,
                                  block_table, bt_stride, n_entries, row0, n_rows, nq, nkv, page_size, num_pages,
                                  window, scale, num_splits, status, stream);
  return CCB_REFUSE_DTYPE;
}

// ---------------------------------------------------------------------------------------------
// The same attention for callers that cannot allocate (declared in attention_split_noalloc.h).
// ---------------------------------------------------------------------------------------------
#include "attention_split_noalloc.h"
#include <mutex>

namespace {

// Scratch of the split partials, part of the library image itself: every GPU that loads the library holds
// these CCB_NOALLOC_SCRATCH_FLOATS * 4 bytes until the process exits.
static __device__ __align__(256) float g_noalloc_scratch[CCB_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {};  // device address of the array on each device, found at set-up
std::mutex g_noalloc_mu;

// In host code `g_noalloc_scratch` is only a handle of the symbol, not an address a kernel may use; the
// device address is asked for once per device, with that device current.
int noalloc_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return CCB_REFUSE_ARG;
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (g_noalloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return CCB_REFUSE_ARG;
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}

}  // namespace

CCB_API int ccb_attention_split_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                        const int* positions, const int* entry_of_token, const int* block_table,
                                        int bt_stride, int n_entries, int row0, int n_rows, int nq, int nkv,
                                        int hd, int page_size, int num_pages, int window, float scale,
                                        int num_splits, int dtype, int* status, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (num_splits <= 0 || nq <= 0 || hd <= 0) return CCB_REFUSE_SIZE;
  float* part_acc = nullptr;
  float* part_ml = nullptr;
  if (num_splits > 1) {
    // accumulators first, then (maximum, sum) pairs; both are written in full by every launch before they
    // are read, so nothing has to be cleared between calls
    const size_t n_acc = (size_t)n_rows * nq * num_splits * hd;
    const size_t n_ml = (size_t)n_rows * nq * num_splits * 2;
    if (n_acc + n_ml > (size_t)CCB_NOALLOC_SCRATCH_FLOATS) return CCB_REFUSE_NOALLOC_TOO_LARGE;
    float* base = nullptr;
    const int rc = noalloc_scratch(&base);
    if (rc != 0) return rc;
    part_acc = base;
    part_ml = base + n_acc;
  }
  return ccb_attention_split(q, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token, block_table,
                             bt_stride, n_entries, row0, n_rows, nq, nkv, hd, page_size, num_pages, window, scale,
                             num_splits, dtype, status, stream);
}
