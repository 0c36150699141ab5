// Prefill attention on tensor cores (bfloat16, head size 64 or 128): portions of prompts over paged keys.
//
//   causal (optionally windowed) attention of the new tokens of each request over everything the request
//   has cached, its own new keys included (7QiC/ccInfer: src/kernel/attention/prefill_attn.cu:42-242, where
//   one block serves ONE query token and one head, re-reading the keys for every token).  Here a block
//   serves 64 consecutive query tokens of one request and one q head: 4 warps x 16 rows.  Keys and values
//   of 64 positions at a time travel global -> shared memory through a two-stage cp.async pipeline shared
//   by the 4 warps; S = Q K^T and O += P V by mma.sync m16n8k16, online softmax in float registers (base-2
//   exponentials), one pass over the keys, no scores stored.
//
// Grid = (query tile, q head, request).  A request's query tiles are counted from its own first new token,
// so tiles never span two requests; blocks of tiles a request does not have return at once.  Tiles run in
// descending order so that the long ones (late tokens see many keys) start first.  The result of a row
// depends on its position, its request's keys and the 64-key tile grid aligned to absolute positions only.
#include "common.cuh"
#include "mma_common.cuh"
#include <math_constants.h>

using namespace ccb;

namespace {

constexpr int kQTile = 64;
constexpr int kKTile = 64;
constexpr int kPStages = 2;
constexpr int kPThreads = 128;

template <int HD>
__global__ void __launch_bounds__(kPThreads, 3)
attention_prefill_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                             const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out,
                             const int* __restrict__ cu_q, const int* __restrict__ pos0,
                             const int* __restrict__ block_table, int bt_stride, int entry0, int nq, int nkv,
                             int page_size, int num_pages, int window, float scale_log2, int* status) {
  ccb::pdl_begin();
  constexpr int CH = HD / 8;
  constexpr int KS = HD / 16;
  constexpr int TILE_ELEMS = kKTile * HD;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  // Two stages of a key tile and a value tile.  The query tile borrows the second stage's key buffer until
  // its fragments sit in registers, which keeps a block at 64 KB (head size 128): three blocks per SM.
  __nv_bfloat16* k_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [stages][64][HD]
  __nv_bfloat16* v_s = k_s + kPStages * TILE_ELEMS;
  __nv_bfloat16* q_s = k_s + TILE_ELEMS;                             // [64][HD], before the pipeline starts

  const int b = entry0 + blockIdx.z;
  const int h = blockIdx.y;
  const int row_begin = cu_q[b], n_new = cu_q[b + 1] - row_begin;
  const int n_qtiles = (n_new + kQTile - 1) / kQTile;
  const int qt = n_qtiles - 1 - (int)blockIdx.x;  // long tiles first
  if (qt < 0) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int kvh = h / (nq / nkv);
  const int p0 = pos0[b];                       // position of the request's first new token
  const int q_first = qt * kQTile;              // first new-token index of this tile
  const int rows_here = min(kQTile, n_new - q_first);
  const int p_first = p0 + q_first, p_last = p_first + rows_here - 1;
  const int* bt = block_table + (size_t)b * bt_stride;
  const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;

  // Q tile -> shared memory (rows beyond the request's tokens are zero)
#pragma unroll
  for (int i = 0; i < kQTile * CH / kPThreads; ++i) {
    const int idx = tid + kPThreads * i;
    const int row = idx / CH, c = idx - row * CH;
    const bool valid = row < rows_here;
    const __nv_bfloat16* src = q + ((size_t)(row_begin + q_first + (valid ? row : 0)) * nq + h) * HD + c * 8;
    cp_async16(smem_u32(q_s + swz<HD>(row, c)), src, valid);
  }
  cp_async_commit();

  const int j_lo = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;  // first key any row sees
  const int first_tile = j_lo / kKTile, last_tile = p_last / kKTile;
  const int n_tiles = last_tile - first_tile + 1;

  // Two threads share a key row: one page lookup and one address per thread and tile, then 16-byte copies of
  // alternating chunks, so that a pair of lanes always asks for one whole 32-byte sector.
  static_assert(kPThreads == 2 * kKTile, "two threads per key row");
  const int ld_row = tid >> 1, ld_half = tid & 1;
  auto issue = [&](int tile, int stage) {
    __nv_bfloat16* ks_ = k_s + stage * TILE_ELEMS;
    __nv_bfloat16* vs_ = v_s + stage * TILE_ELEMS;
    const int j = tile * kKTile + ld_row;
    bool valid = j >= j_lo && j <= p_last;
    size_t src = 0;
    if (valid) {
      const int lp = page_shift >= 0 ? (j >> page_shift) : (j / page_size);
      const int page = lp < bt_stride ? bt[lp] : -1;
      if (page < 0 || page >= num_pages) {
        set_status(status, CCB_ST_BAD_PAGE);
        valid = false;
      } else {
        src = (((size_t)page * nkv + kvh) * page_size + (j - lp * page_size)) * HD;
      }
    }
    const __nv_bfloat16* ksrc = k_cache + src;
    const __nv_bfloat16* vsrc = v_cache + src;
    const uint32_t kdst = smem_u32(ks_ + ld_row * HD), vdst = smem_u32(vs_ + ld_row * HD);
    const int sw = ld_row & 7;
#pragma unroll
    for (int i = 0; i < CH / 2; ++i) {
      const int c = 2 * i + ld_half;
      const uint32_t off = (uint32_t)((c ^ sw) << 4);
      cp_async16(kdst + off, ksrc + c * 8, valid);
      cp_async16(vdst + off, vsrc + c * 8, valid);
    }
  };

  // Q fragments of this warp's 16 rows
  cp_async_wait<0>();
  __syncthreads();
  uint32_t qa[KS][4];
  {
    const int qrow = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
    const int qchunk = lane >> 4;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
      ldmatrix_x4(qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], smem_u32(q_s + swz<HD>(qrow, 2 * ks + qchunk)));
  }
  __syncthreads();  // everybody has its fragments: the buffer is a pipeline stage from here on
  issue(first_tile, 0);
  cp_async_commit();
  // rows gid and gid + 8 of the warp: their positions and the first key each may see
  const int pr0 = p_first + warp * 16 + gid, pr1 = pr0 + 8;
  const int lo0 = window > 0 ? max(0, pr0 - window + 1) : 0, lo1 = window > 0 ? max(0, pr1 - window + 1) : 0;

  float o[2 * KS][4];
#pragma unroll
  for (int i = 0; i < 2 * KS; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;

  for (int it = 0; it < n_tiles; ++it) {
    cp_async_wait<kPStages - 2>();
    __syncthreads();
    if (it + kPStages - 1 < n_tiles) issue(first_tile + it + kPStages - 1, (it + kPStages - 1) % kPStages);
    cp_async_commit();
    const __nv_bfloat16* ks_ = k_s + (it % kPStages) * TILE_ELEMS;
    const __nv_bfloat16* vs_ = v_s + (it % kPStages) * TILE_ELEMS;
    const int jt = (first_tile + it) * kKTile;
    // a warp whose rows all lie before this tile's first key has nothing to do in it (causal)
    const bool warp_active = jt <= p_first + warp * 16 + 15;
    if (warp_active) {
      float s[8][4];
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
      {
        const int krow = (lane & 7) + 8 * (lane >> 4);
        const int kchunk = (lane >> 3) & 1;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
          for (int np = 0; np < 4; ++np) {
            uint32_t b00, b01, b10, b11;
            ldmatrix_x4(b00, b01, b10, b11, smem_u32(ks_ + swz<HD>(np * 16 + krow, 2 * ks + kchunk)));
            mma_bf16_16816(s[2 * np], qa[ks], b00, b01);
            mma_bf16_16816(s[2 * np + 1], qa[ks], b10, b11);
          }
        }
      }
      float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
      for (int nb = 0; nb < 8; ++nb)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = jt + nb * 8 + 2 * tig + e;
          s[nb][e] = (j <= pr0 && j >= lo0) ? s[nb][e] * scale_log2 : -CUDART_INF_F;
          s[nb][2 + e] = (j <= pr1 && j >= lo1) ? s[nb][2 + e] * scale_log2 : -CUDART_INF_F;
          mx0 = fmaxf(mx0, s[nb][e]);
          mx1 = fmaxf(mx1, s[nb][2 + e]);
        }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float c0 = mn0 == -CUDART_INF_F ? 1.f : exp2f(m0 - mn0);
      const float c1 = mn1 == -CUDART_INF_F ? 1.f : exp2f(m1 - mn1);
      const float sub0 = mn0 == -CUDART_INF_F ? 0.f : mn0, sub1 = mn1 == -CUDART_INF_F ? 0.f : mn1;
      m0 = mn0;
      m1 = mn1;
      float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
      for (int nb = 0; nb < 8; ++nb)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          s[nb][e] = exp2f(s[nb][e] - sub0);
          s[nb][2 + e] = exp2f(s[nb][2 + e] - sub1);
          ps0 += s[nb][e];
          ps1 += s[nb][2 + e];
        }
      l0 = l0 * c0 + ps0;
      l1 = l1 * c1 + ps1;
#pragma unroll
      for (int i = 0; i < 2 * KS; ++i) {
        o[i][0] *= c0; o[i][1] *= c0;
        o[i][2] *= c1; o[i][3] *= c1;
      }
      {
        const int vrow = (lane & 7) + 8 * ((lane >> 3) & 1);
        const int vchunk = lane >> 4;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {  // 16 keys at a time
          uint32_t pa[4];
          pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
          pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
          pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
          pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
          for (int nn = 0; nn < KS; ++nn) {
            uint32_t b00, b01, b10, b11;
            ldmatrix_x4_trans(b00, b01, b10, b11, smem_u32(vs_ + swz<HD>(kk * 16 + vrow, 2 * nn + vchunk)));
            mma_bf16_16816(o[2 * nn], pa, b00, b01);
            mma_bf16_16816(o[2 * nn + 1], pa, b10, b11);
          }
        }
      }
    }
  }
  cp_async_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const int r0 = warp * 16 + gid, r1 = r0 + 8;
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
  __nv_bfloat16* o0 = out + ((size_t)(row_begin + q_first + r0) * nq + h) * HD;
  __nv_bfloat16* o1 = out + ((size_t)(row_begin + q_first + r1) * nq + h) * HD;
#pragma unroll
  for (int i = 0; i < 2 * KS; ++i) {
    const int d = i * 8 + 2 * tig;
    if (r0 < rows_here) *reinterpret_cast<uint32_t*>(o0 + d) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
    if (r1 < rows_here) *reinterpret_cast<uint32_t*>(o1 + d) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
  }
}

template <int HD>
int launch(const void* q, const void* k_cache, const void* v_cache, void* out, const int* cu_q, const int* pos0,
           const int* block_table, int bt_stride, int entry0, int n_entries, int max_new, int nq, int nkv,
           int page_size, int num_pages, int window, float scale, int* status, cudaStream_t stream) {
  const size_t smem = (size_t)(2 * kPStages * kKTile * HD) * sizeof(__nv_bfloat16);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_mma_kernel<HD>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((max_new + kQTile - 1) / kQTile, nq, n_entries);
  ccb_launch(attention_prefill_mma_kernel<HD>, grid, kPThreads, smem, stream, 
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)out,
      cu_q, pos0, block_table, bt_stride, entry0, nq, nkv, page_size, num_pages, window,
      scale * 1.4426950408889634f, status);
  return ccb_launch_status();
}

}  // namespace

// Requests entry0 .. entry0 + n_entries - 1 of the step (cu_q, pos0 and block_table rows are indexed by the
// request's place in the step); max_new = the most new tokens any of them brings.  bfloat16, head size 64
// or 128; other sizes are refused and belong to ccb_attention_split.
CCB_API int ccb_attention_prefill_mma(const void* q, const void* k_cache, const void* v_cache, void* out,
                                      const int* cu_q, const int* pos0, const int* block_table, int bt_stride,
                                      int entry0, int n_entries, int max_new, int nq, int nkv, int hd,
                                      int page_size, int num_pages, int window, float scale, int* status,
                                      cudaStream_t stream) {
  if (n_entries <= 0 || max_new <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || bt_stride <= 0 || n_entries > 65535 || nq > 65535)
    return CCB_REFUSE_SIZE;
  if (hd == 128)
    return launch<128>(q, k_cache, v_cache, out, cu_q, pos0, block_table, bt_stride, entry0, n_entries, max_new,
                       nq, nkv, page_size, num_pages, window, scale, status, stream);
  if (hd == 64)
    return launch<64>(q, k_cache, v_cache, out, cu_q, pos0, block_table, bt_stride, entry0, n_entries, max_new, nq,
                      nkv, page_size, num_pages, window, scale, status, stream);
  return CCB_REFUSE_SIZE;
}
