// Prefill attention on the 5th-generation tensor cores (bfloat16, head size 128 or 64).
//
//   causal (optionally windowed) attention of the new tokens of each request over its paged cache, as
//   attention_prefill_mma_kernel computes it (7QiC/ccInfer: src/kernel/attention/prefill_attn.cu:42-242),
//   but with both products on tcgen05.mma and both accumulators in tensor memory:
//
//   block = (128 query tokens of one request, one q head); per tile of 128 key positions
//     S = Q K^T          tcgen05.mma  M=128 N=128 K=head   -> TMEM, two buffers: the product of tile i+1 runs
//                        while the softmax warps work on tile i
//     P = softmax part   four warps, one query row per thread: tcgen05.ld S, mask, running max and sum in
//                        float (base-2 exponentials), P as bfloat16 pairs into tensor memory (tcgen05.st);
//                        the running output in TMEM is rescaled when the maximum moved
//     O += P V           tcgen05.mma  M=128 N=head K=128, P the A operand in tensor memory, V the MN-major
//                        B operand in shared memory -> TMEM
//   Q, K and V tiles arrive by TMA: Q as two boxes of 128 rows x 64 columns, K and V page by page (a box is
//   one page of one kv head: page_size rows x 64 columns), two stages each.  Warp 0 issues the key copies,
//   warp 6 the value copies (one warp for both set the pace of the block: every box is an instruction of its
//   own), warp 1 the products, warps 2..5 do the softmax, the rescaling and the final division and store.
//   A key stage is handed back as soon as its product Q K^T has run, a value stage after its P V; P has two
//   buffers, so the softmax of a tile does not wait for the previous tile's P V unless it must rescale O.
//   Tensor memory: S at columns 0 and 128, O at 256, P at 384 and 448.
//   Measured per 128-key tile on B200 (clock64 of one block, 2,048-token prompt): 3,740 cycles with one
//   producer warp and one stage barrier for keys and values, 2,190 with P in shared memory, 2,060 as it
//   is now, of which the softmax threads are busy 1,800 (tcgen05.ld and maximum 345, exponentials, sum,
//   conversion and store 1,270).  Measured and dropped, because none made a tile faster: two threads a row
//   (eight softmax warps); a share of the exponentials as a cubic on the FMA pipe; two groups of softmax warps
//   on alternating tiles with three S buffers and P written over its own S; four producer warps.
//
// Key tiles are aligned to absolute positions, so a row's result depends on its position and its request's
// keys only.  Every mbarrier wait is bounded (CCB_ST_WAIT_TIMEOUT, then the block tears down and returns).
#include "common.cuh"
#include "tc_common.cuh"
#include "tma_host.h"
#include <math_constants.h>

using namespace ccb;

// 1: always one q head per block (the older kernel), for comparisons; set by ccb_attention_prefill_tc_single_head
static int g_ccb_prefill_single_head = 0;

namespace {

constexpr int kTQ = 128;     // query rows per block = TMEM lanes
constexpr int kTK = 128;     // keys per tile
constexpr int kTcThreads = 224;  // warps: 0 key loads, 1 products, 2..5 softmax, 6 value loads
constexpr int kKvStages = 2;   // a third stage (the shared memory is there since P left it) measured no faster

// 2^x by the special-function unit alone (one instruction; 2^-inf = 0)
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Two floats in one 64-bit register, for the packed float instructions of sm_100 (one issue slot for two
// results on the FMA pipe).
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// HD = 64 * NH
template <int NH>
__global__ void __launch_bounds__(kTcThreads, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                            const __grid_constant__ CUtensorMap tmV, __nv_bfloat16* __restrict__ out,
                            const int* __restrict__ cu_q, const int* __restrict__ pos0,
                            const int* __restrict__ block_table, int bt_stride, int entry0, int nq, int nkv,
                            int page_size, int page_shift, int num_pages, int window, float scale_log2,
                            int* status) {
  constexpr int HD = 64 * NH;
  constexpr int HALF_BYTES = 128 * 128;            // 128 rows x 128 bytes: one 64-column half of a tile
  constexpr int TILE_BYTES = NH * HALF_BYTES;      // Q, K or V tile
  constexpr int TMEM_COLS = 512;                   // S: two buffers of 128 columns, O: HD columns, P: two of 64
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE_BYTES;                   // [stages]
  uint8_t* sV = sK + kKvStages * TILE_BYTES;       // [stages]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + kKvStages * TILE_BYTES);
  // barriers: q_full, k_full[3], v_full[3], k_empty[3], v_empty[3], s_full[2], p_ready, pv_done[2]
  const uint32_t b_q = s32(bars), b_kf = s32(bars + 1), b_vf = s32(bars + 4), b_ke = s32(bars + 7),
                 b_ve = s32(bars + 10), b_sf = s32(bars + 13), b_pr = s32(bars + 15), b_pv = s32(bars + 16);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);

  const int b = entry0 + blockIdx.z;
  const int h = blockIdx.x;
  const int row_begin = cu_q[b], n_new = cu_q[b + 1] - row_begin;
  const int n_qtiles = (n_new + kTQ - 1) / kTQ;
  // Blocks start in the order of their linear index, x fastest: with the heads in x, every head's longest
  // query tile (the last one: it sees the most keys) starts first and the short ones fill in at the end.
  // With the tiles in x the lengths came mixed and the SMs finished up to 2.6x apart.
  const int qt = n_qtiles - 1 - (int)blockIdx.y;
  if (qt < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = h / (nq / nkv);
  const int p0 = pos0[b];
  const int q_first = qt * kTQ;
  const int rows_here = min(kTQ, n_new - q_first);
  const int p_first = p0 + q_first, p_last = p_first + rows_here - 1;
  const int* bt = block_table + (size_t)b * bt_stride;
  const int j_lo = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
  const int first_tile = j_lo / kTK, last_tile = p_last / kTK;
  const int n_tiles = last_tile - first_tile + 1;

  if (threadIdx.x == 0) {
    mbar_init(b_q, 1);
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(b_kf + 8 * s, 1);
      mbar_init(b_vf + 8 * s, 1);
      mbar_init(b_ke + 8 * s, 1);
      mbar_init(b_ve + 8 * s, 1);
    }
    mbar_init(b_sf, 1);
    mbar_init(b_sf + 8, 1);
    mbar_init(b_pr, 128);
    mbar_init(b_pv, 1);
    mbar_init(b_pv + 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_s = *tmem_slot, tmem_o = tmem_s + 256;  // S buffers at columns 0 and 128
  const uint32_t tmem_p = tmem_s + 384;                       // P: two buffers of 64 columns (bfloat16 pairs)

  if (warp == 0 || warp == 6) {
    // ---- TMA producers: whole warps, one lane per page of a tile, so that the page look-ups (dependent
    // global loads) of a tile run side by side instead of one after the other ----
    pdl_wait();
    if (warp == 0 && lane == 0) {
      mbar_expect_tx(b_q, TILE_BYTES);
#pragma unroll
      for (int hf = 0; hf < NH; ++hf)
        tma_load_2d(s32(sQ + hf * HALF_BYTES), &tmQ, h * HD + hf * 64, row_begin + q_first, b_q);
    }
    const int pages_per_tile = kTK >> page_shift;
    const int lp_last = p_last >> page_shift;  // a page that certainly exists: stands in for pages a tile
                                               // reaches but the request does not hold (their keys are masked)
    // first row (in the [rows, HD] view of the cache) of this lane's page of tile t
    auto page_row = [&](int t) -> int {
      const int lp = (((first_tile + t) * kTK) >> page_shift) + lane;
      int page = (lp <= lp_last && lp < bt_stride) ? bt[lp] : -1;
      if (page < 0 || page >= num_pages) {
        // stands in only for pages none of the tile's queries reads; a missing page with a visible key is reported
        const int k_lo = lp << page_shift;
        if (k_lo <= p_last && k_lo + page_size - 1 >= j_lo) set_status(status, CCB_ST_BAD_PAGE);
        page = bt[lp_last];
      }
      if (page < 0 || page >= num_pages) {
        set_status(status, CCB_ST_BAD_PAGE);
        page = 0;
      }
      return (page * nkv + kvh) * page_size;
    };
    const uint32_t off = (uint32_t)(lane * page_size) * 128u;
    // Two producer warps, one for the keys and one for the values: a tile is 2 * NH boxes per page, each
    // its own instruction, and one warp issuing them all was what set the pace of the whole block.  A key
    // stage is free as soon as ITS product Q K^T has run, long before the same tile's P V.
    const bool keys = warp == 0;
    const uint32_t b_full = keys ? b_kf : b_vf, b_empty = keys ? b_ke : b_ve;
    uint8_t* stage0 = keys ? sK : sV;
    const CUtensorMap* tm = keys ? &tmK : &tmV;
    for (int i = 0; i < n_tiles; ++i) {
      const int s = i % kKvStages, ph = (i / kKvStages) & 1;
      int ok = 1;
      if (lane == 0) {
        ok = mbar_wait(b_empty + 8 * s, ph ^ 1) ? 1 : 0;
        if (ok) mbar_expect_tx(b_full + 8 * s, TILE_BYTES);
        else set_status(status, CCB_ST_WAIT_TIMEOUT);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane < pages_per_tile) {
        const int grow = page_row(i);
#pragma unroll
        for (int hf = 0; hf < NH; ++hf)
          tma_load_2d(s32(stage0 + s * TILE_BYTES + hf * HALF_BYTES) + off, tm, hf * 64, grow, b_full + 8 * s);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---- MMA issuer ----
      // S = Q K^T: M 128, N 128, both K-major.  O += P V: M 128, N HD, A K-major, B (V) MN-major (bit 16).
      constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) |
                                   ((uint32_t)(128 >> 4) << 24);
      // S of tile t goes to buffer t & 1: the product of the NEXT tile is issued before this tile's P V, so it
      // runs while the softmax warps work on this tile, and their next S is ready when they come back.
      auto issue_qk = [&](int t) -> bool {
        const int s = t % kKvStages, ph = (t / kKvStages) & 1;
        if (!mbar_wait(b_kf + 8 * s, ph)) return false;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint64_t da = smem_desc(s32(sQ + (ks >> 2) * HALF_BYTES)) + 2 * (ks & 3);
          const uint64_t db = smem_desc(s32(sK + s * TILE_BYTES + (ks >> 2) * HALF_BYTES)) + 2 * (ks & 3);
          tc_mma(tmem_s + (t & 1) * 128, da, db, idesc_s, ks > 0 ? 1u : 0u);
        }
        tc_commit(b_sf + 8 * (t & 1));
        tc_commit(b_ke + 8 * s);  // the key stage may be refilled as soon as this product has run
        return true;
      };
      bool alive = mbar_wait(b_q, 0);
      if (alive) alive = issue_qk(0);
      for (int i = 0; i < n_tiles && alive; ++i) {
        const int s = i % kKvStages, ph = (i / kKvStages) & 1;
        // buffer (i + 1) & 1 is free: the softmax of tile i - 1 read it before it signalled p_ready(i - 1)
        if (i + 1 < n_tiles) {
          alive = issue_qk(i + 1);
          if (!alive) break;
        }
        // O += P V once the softmax warps have written P (and rescaled O) and V has landed
        alive = mbar_wait(b_pr, i & 1) && mbar_wait(b_vf + 8 * s, ph);
        if (!alive) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < kTK / 16; ++ks) {
          // P is the A operand in tensor memory (lane = query row, a column = two consecutive keys: 16 keys
          // = 8 columns).  V: 16 keys further = 16 rows of 128 bytes; 64 head columns further = the next half;
          // 8 keys = 1024 bytes
          const uint64_t db = smem_desc_mn(s32(sV + s * TILE_BYTES) + ks * 2048, HALF_BYTES, 1024);
          tc_mma_ts(tmem_o, tmem_p + (i & 1) * 64 + ks * 8, db, idesc_o, (i > 0 || ks > 0) ? 1u : 0u);
        }
        tc_commit(b_ve + 8 * s);  // the value stage may be refilled
        tc_commit(b_pv + 8 * (i & 1));  // this P buffer may be overwritten, O may be rescaled
      }
      if (!alive) set_status(status, CCB_ST_WAIT_TIMEOUT);
    }
  } else {  // ---- softmax, rescaling, epilogue: thread = query row = TMEM lane ----
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const int pr = p_first + row;                                   // this row's position
    const int lo = window > 0 ? max(0, pr - window + 1) : 0;        // first key it may see
    float m = -CUDART_INF_F, l = 0.f;
    bool alive = true;
    for (int i = 0; i < n_tiles; ++i) {
      alive = mbar_wait(b_sf + 8 * (i & 1), (i >> 1) & 1);
      if (!alive) break;
      tc_fence_after();
      const int jt = (first_tile + i) * kTK;
      const uint32_t tmem_si = tmem_s + (i & 1) * 128;
      // Most tiles lie wholly in every row's past (and inside its window): they need no mask.
      const bool need_mask = (jt + kTK - 1 > p_first) || (window > 0 && jt < p_first + kTQ - window);
      // the row's 128 scores, read once
      uint32_t v[kTK];
#pragma unroll
      for (int c0 = 0; c0 < kTK; c0 += 32) tc_ld32(tmem_si + lane_addr + c0, v + c0);
      tc_wait_ld();
      if (need_mask) {
#pragma unroll
        for (int e = 0; e < kTK; ++e) {
          const int j = jt + e;
          if (!(j <= pr && j >= lo)) v[e] = 0xff800000u;  // -inf: 2^(-inf) = 0 below
        }
      }
      float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};  // four independent chains
#pragma unroll
      for (int e = 0; e < kTK; e += 4)
#pragma unroll
        for (int u = 0; u < 4; ++u) mx4[u] = fmaxf(mx4[u], __uint_as_float(v[e + u]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
      // The running maximum only has to keep the exponentials in range, it need not be the true maximum:
      // it moves when the new one is more than 2^8 larger (or at the first visible key), which spares most
      // rescalings of O; the final division by l makes the result the same.
      const float m_new = (m == -CUDART_INF_F || mx > m + 8.f) ? fmaxf(m, mx) : m;
      const float corr = m_new == -CUDART_INF_F ? 1.f : ex2(m - m_new);
      const float sub = m_new == -CUDART_INF_F ? 0.f : m_new;
      m = m_new;
      // P has two buffers (in tensor memory): this tile's was last read by P V of tile i - 2, long over;
      // the previous tile's P V only has to be complete when O is rescaled, which is rare
      if (i >= 2) {
        alive = mbar_wait(b_pv + 8 * (i & 1), ((i - 2) >> 1) & 1);
        if (!alive) break;
      }
      if (i > 0) {
        if (__any_sync(0xffffffffu, corr != 1.f)) {
          alive = mbar_wait(b_pv + 8 * ((i - 1) & 1), ((i - 1) >> 1) & 1);
          if (!alive) break;
          tc_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < HD; c0 += 32) {
            uint32_t o[32];
            tc_ld32(tmem_o + lane_addr + c0, o);
            tc_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * corr);
            tc_st32(tmem_o + lane_addr + c0, o);
          }
          tc_wait_st();
        }
      }
      // probabilities -> bfloat16 pairs -> tensor memory, where P is the A operand of P V: no shared memory for
      // it, no generic-to-async fence, and the product reads one operand less through the shared-memory port
      float ps2[2] = {0.f, 0.f};
      const float nsub = -sub;
#pragma unroll
      for (int c0 = 0; c0 < kTK; c0 += 64) {
        uint32_t packed[32];
#pragma unroll
        for (int e = 0; e < 64; e += 2) {
          const float a = ex2(fmaf(__uint_as_float(v[c0 + e]), scale_log2, nsub));
          const float c = ex2(fmaf(__uint_as_float(v[c0 + e + 1]), scale_log2, nsub));
          ps2[0] += a;
          ps2[1] += c;
          const __nv_bfloat162 hh = __floats2bfloat162_rn(a, c);
          packed[e >> 1] = *reinterpret_cast<const uint32_t*>(&hh);
        }
        tc_st32(tmem_p + (i & 1) * 64 + lane_addr + (c0 >> 1), packed);
      }
      tc_wait_st();
      l = l * corr + (ps2[0] + ps2[1]);
      tc_fence_before();    // S reads, P and O writes before the next products
      mbar_arrive(b_pr);
    }
    if (alive) {
      alive = mbar_wait(b_pv + 8 * ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1);
      tc_fence_after();
    }
    if (!alive && lane == 0) set_status(status, CCB_ST_WAIT_TIMEOUT);
    pdl_trigger();
    if (alive) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = out + ((size_t)(row_begin + q_first + row) * nq + h) * HD;
#pragma unroll 1
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t v[32];
        tc_ld32(tmem_o + lane_addr + c0, v);
        tc_wait_ld();
        if (row < rows_here) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint32_t p4[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(v[e + 2 * u]) * inv,
                                                              __uint_as_float(v[e + 2 * u + 1]) * inv);
              p4[u] = *reinterpret_cast<const uint32_t*>(&hh);
            }
            *reinterpret_cast<uint4*>(orow + c0 + e) = make_uint4(p4[0], p4[1], p4[2], p4[3]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_s), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// Two q heads of one kv group per block.  The same key and value tiles feed two independent sets of S, P and
// O in tensor memory, and each head has its own group of four softmax warps: while one head's softmax works
// on a tile, the tensor pipe runs the other head's products, which a block of one head left idle for most
// of a tile (the chain S -> exponentials -> P -> P V is serial within a head).  Keys and values are fetched
// once for two heads.
//   warps 0..3   softmax, rescaling and store of head h0       (tensor-memory lanes 32 (warp % 4) ..)
//   warps 4..7   the same for head h0 + 1
//   warp 8 key loads, warp 9 products, warp 10 value loads, warp 11 idle
//   tensor memory: S of head a at column 0, of head b at 128; O at 256 and 384.  P (bfloat16 pairs, 64
//   columns) is written over the first half of its own S once the row's scores are in registers: the next
//   Q K^T of that head is issued after the P V that reads it, and the tensor pipe runs its products in the
//   order of their issue, so a head needs one S buffer only.  By the same order a head's S of tile i + 1 is
//   complete only after its P V of tile i: the softmax threads need no separate wait before they rescale O.
// ---------------------------------------------------------------------------------------------
constexpr int kPairThreads = 384;

template <int NH>
__global__ void __launch_bounds__(kPairThreads, 1)
attention_prefill_tc_pair_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                                 const __grid_constant__ CUtensorMap tmV, __nv_bfloat16* __restrict__ out,
                                 const int* __restrict__ cu_q, const int* __restrict__ pos0,
                                 const int* __restrict__ block_table, int bt_stride, int entry0, int nq, int nkv,
                                 int page_size, int page_shift, int num_pages, int window, float scale_log2,
                                 int* status) {
  constexpr int HD = 64 * NH;
  constexpr int HALF_BYTES = 128 * 128;
  constexpr int TILE_BYTES = NH * HALF_BYTES;
  constexpr int TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                              // [2 heads]
  uint8_t* sK = sQ + 2 * TILE_BYTES;               // [stages]
  uint8_t* sV = sK + kKvStages * TILE_BYTES;       // [stages]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + kKvStages * TILE_BYTES);
  // barriers: q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2 heads], p_ready[2 heads], pv_done[2 heads]
  const uint32_t b_q = s32(bars), b_kf = s32(bars + 1), b_vf = s32(bars + 3), b_ke = s32(bars + 5),
                 b_ve = s32(bars + 7), b_sf = s32(bars + 9), b_pr = s32(bars + 11), b_pv = s32(bars + 13);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  static_assert(kKvStages == 2, "the barrier layout above holds two stages");

  const int b = entry0 + blockIdx.z;
  const int h0 = 2 * blockIdx.x;                   // heads h0 and h0 + 1: the same kv head (the group is even)
  const int row_begin = cu_q[b], n_new = cu_q[b + 1] - row_begin;
  const int n_qtiles = (n_new + kTQ - 1) / kTQ;
  const int qt = n_qtiles - 1 - (int)blockIdx.y;   // the longest tiles first (see the kernel above)
  if (qt < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = h0 / (nq / nkv);
  const int p0 = pos0[b];
  const int q_first = qt * kTQ;
  const int rows_here = min(kTQ, n_new - q_first);
  const int p_first = p0 + q_first, p_last = p_first + rows_here - 1;
  const int* bt = block_table + (size_t)b * bt_stride;
  const int j_lo = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
  const int first_tile = j_lo / kTK, last_tile = p_last / kTK;
  const int n_tiles = last_tile - first_tile + 1;

  if (threadIdx.x == 0) {
    mbar_init(b_q, 1);
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(b_kf + 8 * s, 1);
      mbar_init(b_vf + 8 * s, 1);
      mbar_init(b_ke + 8 * s, 1);
      mbar_init(b_ve + 8 * s, 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(b_sf + 8 * x, 1);
      mbar_init(b_pr + 8 * x, 128);
      mbar_init(b_pv + 8 * x, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8 || warp == 10) {
    // ---- TMA producers (as in the kernel above): a lane per page of a tile ----
    pdl_wait();
    if (warp == 8 && lane == 0) {
      mbar_expect_tx(b_q, 2 * TILE_BYTES);
#pragma unroll
      for (int x = 0; x < 2; ++x)
#pragma unroll
        for (int hf = 0; hf < NH; ++hf)
          tma_load_2d(s32(sQ + x * TILE_BYTES + hf * HALF_BYTES), &tmQ, (h0 + x) * HD + hf * 64, row_begin + q_first, b_q);
    }
    const int pages_per_tile = kTK >> page_shift;
    const int lp_last = p_last >> page_shift;
    auto page_row = [&](int t) -> int {
      const int lp = (((first_tile + t) * kTK) >> page_shift) + lane;
      int page = (lp <= lp_last && lp < bt_stride) ? bt[lp] : -1;
      if (page < 0 || page >= num_pages) {
        const int k_lo = lp << page_shift;
        if (k_lo <= p_last && k_lo + page_size - 1 >= j_lo) set_status(status, CCB_ST_BAD_PAGE);
        page = bt[lp_last];
      }
      if (page < 0 || page >= num_pages) {
        set_status(status, CCB_ST_BAD_PAGE);
        page = 0;
      }
      return (page * nkv + kvh) * page_size;
    };
    const uint32_t off = (uint32_t)(lane * page_size) * 128u;
    const bool keys = warp == 8;
    const uint32_t b_full = keys ? b_kf : b_vf, b_empty = keys ? b_ke : b_ve;
    uint8_t* stage0 = keys ? sK : sV;
    const CUtensorMap* tm = keys ? &tmK : &tmV;
    for (int i = 0; i < n_tiles; ++i) {
      const int s = i % kKvStages, ph = (i / kKvStages) & 1;
      int ok = 1;
      if (lane == 0) {
        ok = mbar_wait(b_empty + 8 * s, ph ^ 1) ? 1 : 0;
        if (ok) mbar_expect_tx(b_full + 8 * s, TILE_BYTES);
        else set_status(status, CCB_ST_WAIT_TIMEOUT);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane < pages_per_tile) {
        const int grow = page_row(i);
#pragma unroll
        for (int hf = 0; hf < NH; ++hf)
          tma_load_2d(s32(stage0 + s * TILE_BYTES + hf * HALF_BYTES) + off, tm, hf * 64, grow, b_full + 8 * s);
      }
      __syncwarp();
    }
  } else if (warp == 9) {
    if (lane == 0) {  // ---- MMA issuer ----
      constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) |
                                   ((uint32_t)(128 >> 4) << 24);
      // S of head x, tile t (the key stage has landed)
      auto issue_qk = [&](int x, int t) {
        const int s = t % kKvStages;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint64_t da = smem_desc(s32(sQ + x * TILE_BYTES + (ks >> 2) * HALF_BYTES)) + 2 * (ks & 3);
          const uint64_t db = smem_desc(s32(sK + s * TILE_BYTES + (ks >> 2) * HALF_BYTES)) + 2 * (ks & 3);
          tc_mma(tmem_base + x * 128, da, db, idesc_s, ks > 0 ? 1u : 0u);
        }
        tc_commit(b_sf + 8 * x);
      };
      bool alive = mbar_wait(b_q, 0) && mbar_wait(b_kf, 0);
      if (alive) {
        tc_fence_after();
        issue_qk(0, 0);
        issue_qk(1, 0);
        tc_commit(b_ke);
      }
      for (int i = 0; i < n_tiles && alive; ++i) {
        const int s = i % kKvStages, ph = (i / kKvStages) & 1;
        const int s1 = (i + 1) % kKvStages, ph1 = ((i + 1) / kKvStages) & 1;
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          // O_x += P_x V once head x's softmax has written P (and rescaled O) and V has landed
          alive = mbar_wait(b_pr + 8 * x, i & 1) && (x == 1 || mbar_wait(b_vf + 8 * s, ph));
          if (!alive) break;
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < kTK / 16; ++ks) {
            const uint64_t db = smem_desc_mn(s32(sV + s * TILE_BYTES) + ks * 2048, HALF_BYTES, 1024);
            tc_mma_ts(tmem_base + 256 + x * 128, tmem_base + x * 128 + ks * 8, db, idesc_o, (i > 0 || ks > 0) ? 1u : 0u);
          }
          tc_commit(b_pv + 8 * x);
          if (x == 1) tc_commit(b_ve + 8 * s);   // both heads' P V of this tile are issued: the value stage
          // the head's next S, over its P: the tensor pipe keeps the order of issue
          if (i + 1 < n_tiles) {
            if (x == 0) {
              alive = mbar_wait(b_kf + 8 * s1, ph1);
              if (!alive) break;
              tc_fence_after();
            }
            issue_qk(x, i + 1);
            if (x == 1) tc_commit(b_ke + 8 * s1);
          }
        }
      }
      if (!alive) set_status(status, CCB_ST_WAIT_TIMEOUT);
    }
  } else if (warp < 8) {  // ---- softmax, rescaling, epilogue: thread = query row = TMEM lane, a group per head ----
    const int x = warp >> 2;
    const int h = h0 + x;
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t tmem_sx = tmem_base + x * 128, tmem_ox = tmem_base + 256 + x * 128;
    const uint32_t bar_sf = b_sf + 8 * x, bar_pr = b_pr + 8 * x, bar_pv = b_pv + 8 * x;
    const int pr = p_first + row;
    const int lo = window > 0 ? max(0, pr - window + 1) : 0;
    float m = -CUDART_INF_F, l = 0.f;
    bool alive = true;
    for (int i = 0; i < n_tiles; ++i) {
      alive = mbar_wait(bar_sf, i & 1);
      if (!alive) break;
      tc_fence_after();
      const int jt = (first_tile + i) * kTK;
      const bool need_mask = (jt + kTK - 1 > p_first) || (window > 0 && jt < p_first + kTQ - window);
      uint32_t v[kTK];
#pragma unroll
      for (int c0 = 0; c0 < kTK; c0 += 32) tc_ld32(tmem_sx + lane_addr + c0, v + c0);
      tc_wait_ld();
      if (need_mask) {
#pragma unroll
        for (int e = 0; e < kTK; ++e) {
          const int j = jt + e;
          if (!(j <= pr && j >= lo)) v[e] = 0xff800000u;
        }
      }
      float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};  // four chains, two scores a step
#pragma unroll
      for (int e = 0; e < kTK; e += 8)
#pragma unroll
        for (int u = 0; u < 4; ++u) mx4[u] = max3(mx4[u], __uint_as_float(v[e + 2 * u]), __uint_as_float(v[e + 2 * u + 1]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
      const float m_new = (m == -CUDART_INF_F || mx > m + 8.f) ? fmaxf(m, mx) : m;
      const float corr = m_new == -CUDART_INF_F ? 1.f : ex2(m - m_new);
      const float sub = m_new == -CUDART_INF_F ? 0.f : m_new;
      m = m_new;
      // this head's P V of tile i - 1 was issued before the Q K^T whose S has just arrived: it is complete
      if (i > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t o[32];
          tc_ld32(tmem_ox + lane_addr + c0, o);
          tc_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * corr);
          tc_st32(tmem_ox + lane_addr + c0, o);
        }
        tc_wait_st();
      }
      // Exponentials; scale, subtraction and sums run as packed pairs (one issue slot for two results).
      // Measured and dropped: a quarter or a half of the exponentials as cubics on the FMA pipe, to relieve
      // the special-function unit (8,192-token prompt: 524 us without, 646 and 746 us with), and the two
      // heads taking turns at the exponentials (554 us): the softmax threads are short of issue slots and of
      // latency to hide, not of the unit.
      const float nsub = -sub;
      const f32x2 sc2 = pack2(scale_log2, scale_log2), ns2 = pack2(nsub, nsub);
      f32x2 sum2 = pack2(0.f, 0.f);
#pragma unroll
      for (int c0 = 0; c0 < kTK; c0 += 64) {
        uint32_t packed[32];
#pragma unroll
        for (int e = 0; e < 64; e += 2) {
          const f32x2 t = fma2(pack2(__uint_as_float(v[c0 + e]), __uint_as_float(v[c0 + e + 1])), sc2, ns2);
          float t0, t1;
          unpack2(t, t0, t1);
          const float a = ex2(t0), c = ex2(t1);
          sum2 = add2(sum2, pack2(a, c));
          const __nv_bfloat162 hh = __floats2bfloat162_rn(a, c);
          packed[e >> 1] = *reinterpret_cast<const uint32_t*>(&hh);
        }
        tc_st32(tmem_sx + lane_addr + (c0 >> 1), packed);   // P over the S that is in registers now
      }
      tc_wait_st();
      float ps0, ps1;
      unpack2(sum2, ps0, ps1);
      l = l * corr + (ps0 + ps1);
      tc_fence_before();
      mbar_arrive(bar_pr);
    }
    if (alive) {
      alive = mbar_wait(bar_pv, (n_tiles - 1) & 1);
      tc_fence_after();
    }
    if (!alive && lane == 0) set_status(status, CCB_ST_WAIT_TIMEOUT);
    pdl_trigger();
    if (alive) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = out + ((size_t)(row_begin + q_first + row) * nq + h) * HD;
#pragma unroll 1
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t v[32];
        tc_ld32(tmem_ox + lane_addr + c0, v);
        tc_wait_ld();
        if (row < rows_here) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint32_t p4[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(v[e + 2 * u]) * inv,
                                                              __uint_as_float(v[e + 2 * u + 1]) * inv);
              p4[u] = *reinterpret_cast<const uint32_t*>(&hh);
            }
            *reinterpret_cast<uint4*>(orow + c0 + e) = make_uint4(p4[0], p4[1], p4[2], p4[3]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

template <int NH>
int launch(const void* q, const void* k_cache, const void* v_cache, void* out, const int* cu_q, const int* pos0,
           const int* block_table, int bt_stride, int entry0, int n_entries, int max_new, int n_tokens, int nq,
           int nkv, int page_size, int num_pages, int window, float scale, int* status, cudaStream_t stream) {
  constexpr int HD = 64 * NH;
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  CUtensorMap tmQ, tmK, tmV;
  const unsigned long long cache_rows = (unsigned long long)num_pages * nkv * page_size;
  if (!ccb_tensor_map_2d(q, n_tokens, (unsigned long long)nq * HD, (unsigned long long)nq * HD, 64, 128, &tmQ) ||
      !ccb_tensor_map_2d(k_cache, cache_rows, HD, HD, 64, page_size, &tmK) ||
      !ccb_tensor_map_2d(v_cache, cache_rows, HD, HD, 64, page_size, &tmV))
    return CCB_REFUSE_ARG;
  if (NH == 2 && (nq / nkv) % 2 == 0 && !g_ccb_prefill_single_head) {
    // head size 128, groups of an even number of q heads: two heads of a group share a block and its key and
    // value tiles (with head size 64 the products are half as long and one head a block is faster: 46 us
    // against 55 us for a 2,048-token prompt of 16 heads)
    const size_t smem2 = (size_t)(2 + 2 * kKvStages) * NH * 128 * 128 + 20 * 8 + 1024;
    static bool configured2 = false;
    if (!configured2) {
      cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_pair_kernel<NH>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
      if (e != cudaSuccess) return (int)e;
      configured2 = true;
    }
    dim3 grid2(nq / 2, (max_new + kTQ - 1) / kTQ, n_entries);
    ccb_launch(attention_prefill_tc_pair_kernel<NH>, grid2, kPairThreads, smem2, stream, tmQ, tmK, tmV,
               (__nv_bfloat16*)out, cu_q, pos0, block_table, bt_stride, entry0, nq, nkv, page_size, page_shift,
               num_pages, window, scale * 1.4426950408889634f, status);
    return ccb_launch_status();
  }
  const size_t smem = (size_t)(1 + 2 * kKvStages) * NH * 128 * 128 + 20 * 8 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<NH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(nq, (max_new + kTQ - 1) / kTQ, n_entries);
  ccb_launch(attention_prefill_tc_kernel<NH>, grid, kTcThreads, smem, stream, tmQ, tmK, tmV, (__nv_bfloat16*)out, cu_q,
             pos0, block_table, bt_stride, entry0, nq, nkv, page_size, page_shift, num_pages, window,
             scale * 1.4426950408889634f, status);
  return ccb_launch_status();
}

}  // namespace

// As ccb_attention_prefill_mma; n_tokens = rows of q / out.  bfloat16, head size 64 or 128, page size a power
// of two from 8 to 128; anything else is refused (CCB_REFUSE_SIZE) and belongs to the other kernels.
CCB_API int ccb_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                     const int* cu_q, const int* pos0, const int* block_table, int bt_stride,
                                     int entry0, int n_entries, int max_new, int n_tokens, int nq, int nkv, int hd,
                                     int page_size, int num_pages, int window, float scale, int* status,
                                     cudaStream_t stream) {
  if (n_entries <= 0 || max_new <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || bt_stride <= 0 || n_entries > 65535 || nq > 65535 || page_size < 8 ||
      page_size > 128 || (page_size & (page_size - 1)) != 0 ||
      ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
        reinterpret_cast<uintptr_t>(out)) & 15) != 0)
    return CCB_REFUSE_SIZE;
  if (hd == 128)
    return launch<2>(q, k_cache, v_cache, out, cu_q, pos0, block_table, bt_stride, entry0, n_entries, max_new,
                     n_tokens, nq, nkv, page_size, num_pages, window, scale, status, stream);
  if (hd == 64)
    return launch<1>(q, k_cache, v_cache, out, cu_q, pos0, block_table, bt_stride, entry0, n_entries, max_new,
                     n_tokens, nq, nkv, page_size, num_pages, window, scale, status, stream);
  return CCB_REFUSE_SIZE;
}

// 1: one q head per block even where two heads of a group could share one (for measurements and tests); 0: the default
CCB_API int ccb_attention_prefill_tc_single_head(int on) {
  g_ccb_prefill_single_head = on ? 1 : 0;
  return 0;
}
