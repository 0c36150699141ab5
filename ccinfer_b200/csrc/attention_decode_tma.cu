// Decode attention on tensor cores with TMA page loads (bfloat16, head size 64 or 128, page size a power of
// two from 8 to 64): the same computation as attention_decode_mma_kernel (single query tokens over paged keys,
// the group's q heads as the 16 rows of an m16n8k16 tile, four warps each taking 16 of a tile's 64 keys, online
// softmax, split key range merged afterwards; 7QiC/ccInfer: src/kernel/attention/decode_attn.cu:417-473).
//
// What differs is how keys and values reach shared memory.  There a tile costs 2,048 16-byte cp.async copies
// issued by all threads, and the load/store path is what holds the kernel (mio / lg throttle stalls).  Here
// two more warps are the producers, one for keys and one for values: one lane per page issues
// cp.async.bulk.tensor boxes of one page of one kv head (page_size rows x 64 columns, 128-byte swizzle) - 16
// copies a tile at page size 16 - signalled by one mbarrier per stage; pages a tile reaches but the request
// does not hold are replaced by its last page (their keys are masked).  Every mbarrier wait is bounded.
#include "common.cuh"
#include "mma_common.cuh"
#include "tc_common.cuh"
#include "tma_host.h"
#include <math_constants.h>

using namespace ccb;

namespace {

constexpr int kTileKeys = 64;
constexpr int kStages = 3;
constexpr int kMinSplitTiles = 4;   // tiles a split should have before another block is worth its start-up
constexpr int kComputeThreads = 128;
constexpr int kThreads = 192;  // four compute warps and two producer warps (keys, values)
constexpr int kHalfBytes = kTileKeys * 128;  // 64 rows x 64 columns of bfloat16

// byte address of 16-byte chunk `chunk` (of the whole head) of row `row`: halves of 64 columns, rows 128 bytes
// apart, chunks XOR-swizzled by the row as the TMA unit wrote them
__device__ __forceinline__ uint32_t tile_addr(uint32_t tile, int row, int chunk) {
  return tile + (chunk >> 3) * kHalfBytes + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

// What the fused form takes instead of finished queries: the rows of the q|k|v product as they left it.  The
// kernel then does what qk_norm_rope_kv_write does for these single-token rows (7QiC/ccInfer:
// src/model/qwen3/qwen3_model.cpp:189-244): per-head RMSNorm and rotate-half rotation of the group's queries
// in every block; in the block whose key range ends at the row's position also the new key and value, which
// it writes to their page and adds to the attention as one more partial result (the copy of that page in
// shared memory was made before the write, so the position is masked there).
struct FusedQkv {
  const __nv_bfloat16* qkv;   // [rows, (nq + 2 nkv) * HD]: q heads, k heads, v heads
  int stride;                 // elements between rows
  const float* q_w;           // [HD] weights of the per-head norms, or null
  const float* k_w;
  float eps;
  const float* inv_freq;      // [HD / 2] rotation frequencies, or null
  __nv_bfloat16* k_cache;     // where the new key and value go; null when the cache belongs to another layer
  __nv_bfloat16* v_cache;     // (that layer has written this position already)
};

// (cos, sin) of position * inv_freq[i], or (1, 0) without rotation
__device__ __forceinline__ float2 angle_cs(const float* inv_freq, float fpos, int i) {
  if (inv_freq == nullptr) return make_float2(1.f, 0.f);
  float sn, cs;
  sincosf(fpos * inv_freq[i], &sn, &cs);
  return make_float2(cs, sn);
}

template <int HD, bool FUSED>
__global__ void __launch_bounds__(kThreads)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                            const __nv_bfloat16* __restrict__ q, const FusedQkv fq,
                            __nv_bfloat16* __restrict__ out,
                            float* __restrict__ part_acc, float* __restrict__ part_ml,
                            const int* __restrict__ positions, const int* __restrict__ entry_of_token,
                            const int* __restrict__ block_table, int bt_stride, int n_entries, int row0, int nq,
                            int nkv, int page_size, int page_shift, int num_pages, int window, float scale,
                            int num_splits, int* __restrict__ counters, int* status) {
  // The kernel after this one is let in only when this one ends: a product that came in while the last
  // blocks were still merging made the pair slower (measured), not faster.
  // The fused form may itself come in early (programmatic dependent launch): the cached keys and values it
  // copies were written by earlier steps and the step's tables long before, so the producer warps fill
  // their stages while the q|k|v product before this kernel still runs; the compute warps wait for that
  // product before they touch its rows.  Otherwise the key of the row's own position is in a page that
  // the kernel before this one wrote: everybody waits first.
  const bool early = FUSED && fq.k_cache != nullptr;
  if (!early) ccb::pdl_wait();
  constexpr int NH = HD / 64;
  constexpr int KS = HD / 16;
  constexpr int TILE_BYTES = NH * kHalfBytes;        // one K or V tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* k_sm = smem;                               // [stages][tile]
  uint8_t* v_sm = k_sm + kStages * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_sm + kStages * TILE_BYTES);
  const uint32_t bar0 = s32(bars), empty0 = s32(bars + kStages);   // per stage: "has landed", "has been read"
  __nv_bfloat16* q_sm = reinterpret_cast<__nv_bfloat16*>(bars + 8);   // [16][HD]: the group's queries (fused form)
  float2* cs_sm = reinterpret_cast<float2*>(q_sm + 16 * HD);          // [HD / 2]: (cos, sin) of the row's angles
  float* qw_sm = reinterpret_cast<float*>(cs_sm + HD / 2);            // [HD]: the queries' norm weights

  const int G = nq / nkv;
  const int gchunks = (G + 15) / 16;
  const int r = blockIdx.x, t = row0 + r;
  const int kvh = blockIdx.y / gchunks, gc = blockIdx.y - kvh * gchunks;
  const int split = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int h0 = kvh * G + gc * 16;
  const int n_heads = min(16, G - gc * 16);

  const int b = entry_of_token[t];
  const int p = positions[t];
  const bool padded = b < 0 || b >= n_entries || p < 0;
  // The row's tiles and how many of the grid's splits get some.  A split is worth a block only from a few
  // tiles on: with a short context the first eff_splits splits take kMinSplitTiles tiles each and the
  // others have nothing to do (the grid is sized without knowing the context).  Where the last block
  // merges, they leave at once and are not waited for (measured at one row and 2,048 keys with a grid of
  // 32 splits: 12.1 us when all 32 took a tile and were merged, as against 10.6 us with a grid of 8).
  const int j0 = (!padded && window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int first_tile = j0 / kTileKeys, last_tile = (padded ? 0 : p) / kTileKeys;
  const int n_tiles = last_tile - first_tile + 1;
  const int eff_splits = padded ? 1 : min(num_splits, max(1, (n_tiles + kMinSplitTiles - 1) / kMinSplitTiles));
  if (counters != nullptr && split >= eff_splits) return;
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar0 + 8 * s, 2);     // the two producer warps
      mbar_init(empty0 + 8 * s, 4);   // the four compute warps
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (FUSED && !padded && tid < HD / 2) cs_sm[tid] = angle_cs(fq.inv_freq, (float)p, tid);   // one angle a thread
  // weights do not wait for the kernel before this one: they are in shared memory when the queries arrive
  if (FUSED && !padded && fq.q_w != nullptr && tid < HD) qw_sm[tid] = fq.q_w[tid];
  __syncthreads();
  if (early && warp < 4) ccb::pdl_wait();

  float o[2 * KS][4];
#pragma unroll
  for (int i = 0; i < 2 * KS; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
  bool owner = false;   // fused form: this block's key range ends at the row's own position

  if (!padded) {
    // q as A fragments: rows = heads of the group (zero beyond n_heads); the producer warp has none
    uint32_t qa[KS][4];
    if (warp < 4 && !FUSED) {
      const __nv_bfloat16* q0 = q + ((size_t)t * nq + h0 + gid) * HD;
      const __nv_bfloat16* q1 = q0 + (size_t)8 * HD;
      const bool v0 = gid < n_heads, v1 = gid + 8 < n_heads;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const int c = ks * 16 + 2 * tig;
        qa[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + c) : 0u;
        qa[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + c) : 0u;
        qa[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + c + 8) : 0u;
        qa[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + c + 8) : 0u;
      }
    }
    if (warp < 4 && FUSED) {
      // Raw queries -> norm -> rotation -> fragments.  A lane holds, of rows gid and gid + 8, the columns
      // 16 ks + 2 tig (+ 0, 1, 8, 9): the four lanes of a quad hold a whole head between them, and the
      // partners of a rotation (columns i and i + HD / 2) sit in the same lane, KS / 2 steps apart.
#pragma unroll
      for (int rh = 0; rh < 2; ++rh) {
        const bool valid = gid + 8 * rh < n_heads;
        const __nv_bfloat16* src = fq.qkv + (size_t)t * fq.stride + (size_t)(h0 + gid + 8 * rh) * HD;
        float x[KS][4];
        float ss = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          const int c = ks * 16 + 2 * tig;
          const float2 lo = valid ? __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + c))
                                  : make_float2(0.f, 0.f);
          const float2 hi = valid ? __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + c + 8))
                                  : make_float2(0.f, 0.f);
          x[ks][0] = lo.x; x[ks][1] = lo.y; x[ks][2] = hi.x; x[ks][3] = hi.y;
          ss += lo.x * lo.x + lo.y * lo.y + hi.x * hi.x + hi.y * hi.y;
        }
        if (fq.q_w != nullptr) {
          ss += __shfl_xor_sync(0xffffffffu, ss, 1);
          ss += __shfl_xor_sync(0xffffffffu, ss, 2);
          const float inv = 1.0f / sqrtf(ss / (float)HD + fq.eps);
#pragma unroll
          for (int ks = 0; ks < KS; ++ks) {
            const int c = ks * 16 + 2 * tig;
            x[ks][0] *= inv * qw_sm[c];
            x[ks][1] *= inv * qw_sm[c + 1];
            x[ks][2] *= inv * qw_sm[c + 8];
            x[ks][3] *= inv * qw_sm[c + 9];
          }
        }
        if (valid || rh == 0) {   // (the angles are only worth computing for rows that exist)
#pragma unroll
          for (int ks = 0; ks < KS / 2; ++ks) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int i = ks * 16 + 2 * tig + (j & 1) + 8 * (j >> 1);
              const float2 cs = cs_sm[i];
              const float a = x[ks][j], bb = x[ks + KS / 2][j];
              x[ks][j] = a * cs.x - bb * cs.y;
              x[ks + KS / 2][j] = bb * cs.x + a * cs.y;
            }
          }
        }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          qa[ks][rh] = pack_bf16(x[ks][0], x[ks][1]);
          qa[ks][2 + rh] = pack_bf16(x[ks][2], x[ks][3]);
        }
      }
      if (warp == 0) {   // the same queries for the warp that adds the new key at the end
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          const int c = ks * 16 + 2 * tig;
          *reinterpret_cast<uint32_t*>(q_sm + gid * HD + c) = qa[ks][0];
          *reinterpret_cast<uint32_t*>(q_sm + (gid + 8) * HD + c) = qa[ks][1];
          *reinterpret_cast<uint32_t*>(q_sm + gid * HD + c + 8) = qa[ks][2];
          *reinterpret_cast<uint32_t*>(q_sm + (gid + 8) * HD + c + 8) = qa[ks][3];
        }
      }
    }
    const int* bt = block_table + (size_t)b * bt_stride;
    const int per_split = (n_tiles + eff_splits - 1) / eff_splits;
    const int my_first = first_tile + split * per_split;
    const int my_tiles = min(my_first + per_split, last_tile + 1) - my_first;
    const int pages_per_tile = kTileKeys >> page_shift;
    const int lp_last = p >> page_shift;
    // the fused form adds position p itself from the product's row, not from the (stale) copy of its page
    const int p_seen = (FUSED && fq.k_cache != nullptr) ? p - 1 : p;
    owner = FUSED && fq.k_cache != nullptr && last_tile >= my_first && last_tile < my_first + my_tiles;

    // producer warps (4: keys, 5: values): lane pg copies page pg of the tile (NH boxes); lane 0 arrives at the
    // stage's barrier with the warp's share of the bytes.  Every box is an instruction of its own that costs
    // its warp about 130 cycles: one warp for both operands was close to setting the pace at full bandwidth.
    auto issue = [&](int tile, int stage) {
      if (lane == 0) mbar_expect_tx(bar0 + 8 * stage, TILE_BYTES);
      __syncwarp();
      if (lane < pages_per_tile) {
        const int lp = ((tile * kTileKeys) >> page_shift) + lane;
        int page = (lp <= lp_last && lp < bt_stride) ? bt[lp] : -1;
        if (page < 0 || page >= num_pages) {
          // A page the tile reaches but no query of the row reads (before the window, beyond the position)
          // is replaced by one that certainly exists and its keys are masked.  One that holds a visible key
          // must be there: its absence is reported, not papered over.
          const int k_lo = lp << page_shift;
          if (k_lo <= p_seen && k_lo + page_size - 1 >= j0) set_status(status, CCB_ST_BAD_PAGE);
          page = bt[lp_last];
        }
        if (page < 0 || page >= num_pages) {
          set_status(status, CCB_ST_BAD_PAGE);
          page = 0;
        }
        const int grow = (page * nkv + kvh) * page_size;
        const uint32_t off = (uint32_t)(lane * page_size) * 128u;
        uint8_t* dst = (warp == 4 ? k_sm : v_sm) + stage * TILE_BYTES;
        const CUtensorMap* tm = warp == 4 ? &tmK : &tmV;
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) tma_load_2d(s32(dst + hf * kHalfBytes) + off, tm, hf * 64, grow, bar0 + 8 * stage);
      }
    };

    // The producers run ahead of the compute warps, held back only by the stages; nobody meets at a block-wide
    // barrier inside the loop: a compute warp waits for its tile to land and, when it has read it, says so.
    if (warp >= 4) {
      for (int j = 0; j < my_tiles; ++j) {
        const int st = j % kStages;
        int ok = 1;
        if (lane == 0) ok = mbar_wait(empty0 + 8 * st, ((j / kStages) & 1) ^ 1) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          if (lane == 0) set_status(status, CCB_ST_WAIT_TIMEOUT);
          break;
        }
        // the compute warps read the stage through the generic proxy, the copies write it through the async
        // proxy: the mbarrier orders the threads, this fence the proxies
        fence_async_smem();
        issue(my_first + j, st);
      }
    }
    for (int it = 0; warp < 4 && it < my_tiles; ++it) {
      const int st = it % kStages;
      if (!mbar_wait(bar0 + 8 * st, (it / kStages) & 1)) {
        if (lane == 0) set_status(status, CCB_ST_WAIT_TIMEOUT);
        break;
      }
      const uint32_t ks_ = s32(k_sm + st * TILE_BYTES);
      const uint32_t vs_ = s32(v_sm + st * TILE_BYTES);

      // S[16 heads, 16 keys of this warp] = Q K^T
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      {
        const int krow = warp * 16 + (lane & 7) + 8 * (lane >> 4);
        const int kchunk = (lane >> 3) & 1;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          uint32_t b00, b01, b10, b11;
          ldmatrix_x4(b00, b01, b10, b11, tile_addr(ks_, krow, 2 * ks + kchunk));
          mma_bf16_16816(s[0], qa[ks], b00, b01);
          mma_bf16_16816(s[1], qa[ks], b10, b11);
        }
      }
      // mask, online softmax (rows gid and gid + 8)
      const int jbase = (my_first + it) * kTileKeys + warp * 16 + 2 * tig;
      float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
      for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = jbase + nb * 8 + e;
          const bool vis = j >= j0 && j <= p_seen;
          s[nb][e] = vis ? s[nb][e] * scale : -CUDART_INF_F;
          s[nb][2 + e] = vis ? s[nb][2 + e] * scale : -CUDART_INF_F;
          mx0 = fmaxf(mx0, s[nb][e]);
          mx1 = fmaxf(mx1, s[nb][2 + e]);
        }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      // a row that has seen no key yet keeps max -inf: its probabilities are 0 and nothing is rescaled
      const float c0 = mn0 == -CUDART_INF_F ? 1.f : __expf(m0 - mn0);
      const float c1 = mn1 == -CUDART_INF_F ? 1.f : __expf(m1 - mn1);
      const float sub0 = mn0 == -CUDART_INF_F ? 0.f : mn0, sub1 = mn1 == -CUDART_INF_F ? 0.f : mn1;
      m0 = mn0;
      m1 = mn1;
      float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
      for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          s[nb][e] = __expf(s[nb][e] - sub0);          // exp(-inf) = 0 for masked keys
          s[nb][2 + e] = __expf(s[nb][2 + e] - sub1);
          ps0 += s[nb][e];
          ps1 += s[nb][2 + e];
        }
      l0 = l0 * c0 + ps0;   // per-lane partial sums; the four lanes of a row are added at the end
      l1 = l1 * c1 + ps1;
#pragma unroll
      for (int i = 0; i < 2 * KS; ++i) {
        o[i][0] *= c0; o[i][1] *= c0;
        o[i][2] *= c1; o[i][3] *= c1;
      }
      // O += P V
      uint32_t pa[4];
      pa[0] = pack_bf16(s[0][0], s[0][1]);
      pa[1] = pack_bf16(s[0][2], s[0][3]);
      pa[2] = pack_bf16(s[1][0], s[1][1]);
      pa[3] = pack_bf16(s[1][2], s[1][3]);
      {
        const int vrow = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
        const int vchunk = lane >> 4;
#pragma unroll
        for (int nn = 0; nn < KS; ++nn) {
          uint32_t b00, b01, b10, b11;
          ldmatrix_x4_trans(b00, b01, b10, b11, tile_addr(vs_, vrow, 2 * nn + vchunk));
          mma_bf16_16816(o[2 * nn], pa, b00, b01);
          mma_bf16_16816(o[2 * nn + 1], pa, b10, b11);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * st);   // this warp has read the stage
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  }
  __syncthreads();  // every copy has landed and every warp is done with the tiles: reuse the memory

  float* o_s = reinterpret_cast<float*>(smem);  // [4 warps + the new key][16 rows][HD]
  float* m_s = o_s + 5 * 16 * HD;                   // [5][16]
  float* l_s = m_s + 80;
  const int n_part = owner ? 5 : 4;
  if (FUSED && warp == 4 && owner) {
    // The row's own key and value, from the product's row: norm, rotation, rounding as the cache holds them;
    // into their page for the steps to come, and into the result as a fifth partial (one key: its score is
    // the maximum, its weight 1, its output the value).  A lane has HD / 32 consecutive columns; the partner
    // of a rotation is 16 lanes away.
    constexpr int CPL = HD / 32;
    const int col0 = lane * CPL;
    const __nv_bfloat16* krow = fq.qkv + (size_t)t * fq.stride + (size_t)(nq + kvh) * HD;
    const __nv_bfloat16* vrow = krow + (size_t)nkv * HD;
    float kx[CPL];
    __nv_bfloat16 vb[CPL];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
      kx[c] = __bfloat162float(krow[col0 + c]);
      vb[c] = vrow[col0 + c];
      ss += kx[c] * kx[c];
    }
    if (fq.k_w != nullptr) {
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)HD + fq.eps);
#pragma unroll
      for (int c = 0; c < CPL; ++c) kx[c] *= inv * fq.k_w[col0 + c];
    }
    const bool first_half = lane < 16;
    __nv_bfloat16 kb[CPL];
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
      const float other = __shfl_xor_sync(0xffffffffu, kx[c], 16);
      const int i = (col0 + c) & (HD / 2 - 1);
      const float2 cs = cs_sm[i];
      const float a = first_half ? kx[c] : other, bb = first_half ? other : kx[c];
      kb[c] = __float2bfloat16_rn(first_half ? a * cs.x - bb * cs.y : bb * cs.x + a * cs.y);
    }
    const int* bt = block_table + (size_t)b * bt_stride;
    const int lp = p >> page_shift;
    const int page = lp < bt_stride ? bt[lp] : -1;
    if (page < 0 || page >= num_pages) {
      if (lane == 0) set_status(status, CCB_ST_BAD_PAGE);
    } else if (gc == 0) {   // one block per kv head writes
      const size_t dst = (((size_t)page * nkv + kvh) * page_size + (p & (page_size - 1))) * HD + col0;
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        fq.k_cache[dst + c] = kb[c];
        fq.v_cache[dst + c] = vb[c];
      }
    }
    for (int hh = 0; hh < n_heads; ++hh) {
      float dot = 0.f;
#pragma unroll
      for (int c = 0; c < CPL; ++c) dot += __bfloat162float(q_sm[hh * HD + col0 + c]) * __bfloat162float(kb[c]);
      dot = warp_sum(dot);
      if (lane == 0) {
        m_s[4 * 16 + hh] = dot * scale;
        l_s[4 * 16 + hh] = 1.f;
      }
#pragma unroll
      for (int c = 0; c < CPL; ++c) o_s[(size_t)(4 * 16 + hh) * HD + col0 + c] = __bfloat162float(vb[c]);
    }
  }
  if (warp < 4) {
#pragma unroll
  for (int i = 0; i < 2 * KS; ++i) {
    const int d = i * 8 + 2 * tig;
    float* dst0 = o_s + ((size_t)(warp * 16 + gid)) * HD + d;
    float* dst1 = o_s + ((size_t)(warp * 16 + gid + 8)) * HD + d;
    dst0[0] = o[i][0]; dst0[1] = o[i][1];
    dst1[0] = o[i][2]; dst1[1] = o[i][3];
  }
  if (tig == 0) {
    m_s[warp * 16 + gid] = m0;
    m_s[warp * 16 + gid + 8] = m1;
    l_s[warp * 16 + gid] = l0;
    l_s[warp * 16 + gid + 8] = l1;
  }
  }
  __syncthreads();
  for (int idx = tid; idx < n_heads * HD; idx += kThreads) {
    const int row = idx / HD, d = idx - row * HD;
    float mm = -CUDART_INF_F;
    for (int w = 0; w < n_part; ++w) mm = fmaxf(mm, m_s[w * 16 + row]);
    float a = 0.f, ll = 0.f;
    if (mm != -CUDART_INF_F) {
      for (int w = 0; w < n_part; ++w) {
        const float f = __expf(m_s[w * 16 + row] - mm);
        a += o_s[(size_t)(w * 16 + row) * HD + d] * f;
        ll += l_s[w * 16 + row] * f;
      }
    }
    const int h = h0 + row;
    if (num_splits == 1) {
      out[((size_t)t * nq + h) * HD + d] = __float2bfloat16_rn(ll > 0.f ? a / ll : 0.f);
    } else {
      const size_t slot = ((size_t)r * nq + h) * num_splits + split;
      part_acc[slot * HD + d] = a;
      if (d == 0) {
        part_ml[slot * 2] = mm;
        part_ml[slot * 2 + 1] = ll;
      }
    }
  }
  if (num_splits == 1 || counters == nullptr) return;  // without counters a second kernel merges the splits
  // The block that arrives last at this (row, head group) merges the splits that had tiles, in ascending order whichever
  // block it is, so that no second kernel (and no gap before it) is needed.
  __shared__ int last_flag;
  __syncthreads();
  if (tid == 0) {
    __threadfence();  // cumulative: the whole block's partial results are visible before its count is
    int* c = counters + (size_t)r * gridDim.y + blockIdx.y;
    const int old = atomicAdd(c, 1);
    last_flag = old == eff_splits - 1;
    if (last_flag) *c = 0;  // ready for the next launch
    __threadfence();
  }
  __syncthreads();
  if (!last_flag) return;
  float* f_s = reinterpret_cast<float*>(smem);  // [16 heads][splits]: each split's weight, then 1 / sum
  float* inv_s = f_s + 16 * 64;
  // a warp per head, a lane per split (two beyond 32): every load of the head is in flight at once
  for (int hh = warp; hh < n_heads; hh += kThreads / 32) {
    const size_t base = ((size_t)r * nq + h0 + hh) * num_splits;
    const int s0 = lane, s1 = lane + 32;
    const float ma = s0 < eff_splits ? __ldcg(&part_ml[(base + s0) * 2]) : -CUDART_INF_F;
    const float mb = s1 < eff_splits ? __ldcg(&part_ml[(base + s1) * 2]) : -CUDART_INF_F;
    const float la = s0 < eff_splits ? __ldcg(&part_ml[(base + s0) * 2 + 1]) : 0.f;
    const float lb = s1 < eff_splits ? __ldcg(&part_ml[(base + s1) * 2 + 1]) : 0.f;
    const float mm = warp_max(fmaxf(ma, mb));
    const float fa = (mm == -CUDART_INF_F || s0 >= eff_splits) ? 0.f : __expf(ma - mm);
    const float fb = (mm == -CUDART_INF_F || s1 >= eff_splits) ? 0.f : __expf(mb - mm);
    if (s0 < eff_splits) f_s[hh * 64 + s0] = fa;
    if (s1 < eff_splits) f_s[hh * 64 + s1] = fb;
    const float ll = warp_sum(la * fa + lb * fb);  // a butterfly: the same order whichever block merges
    if (lane == 0) inv_s[hh] = ll > 0.f ? 1.f / ll : 0.f;
  }
  __syncthreads();
  for (int idx = tid; idx < n_heads * (HD / 4); idx += kThreads) {
    const int row = idx / (HD / 4), d = 4 * (idx - row * (HD / 4));
    const size_t base = ((size_t)r * nq + h0 + row) * num_splits;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int s = 0; s < eff_splits; ++s) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(&part_acc[(base + s) * HD + d]));
      const float f = f_s[row * 64 + s];
      a.x += v.x * f; a.y += v.y * f; a.z += v.z * f; a.w += v.w * f;
    }
    const float inv = inv_s[row];
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a.x * inv, a.y * inv), hi = __floats2bfloat162_rn(a.z * inv, a.w * inv);
    uint2 pk;
    pk.x = *reinterpret_cast<const uint32_t*>(&lo);
    pk.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(&out[((size_t)t * nq + h0 + row) * HD + d]) = pk;
  }
}

__global__ void attention_merge_bf16_kernel2(__nv_bfloat16* __restrict__ out, const float* __restrict__ part_acc,
                                            const float* __restrict__ part_ml, int row0, int nq, int hd,
                                            int num_splits) {
  ccb::pdl_begin();
  const int r = blockIdx.x, h = blockIdx.y;
  const size_t base = ((size_t)r * nq + h) * num_splits;
  __nv_bfloat16* o = out + ((size_t)(row0 + r) * nq + h) * hd;
  // Eight splits at a time: their maxima, sums and outputs are all asked for before any is used, and are
  // folded in ascending order into a running (maximum, sum, output), as the attention kernels do with keys.
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float mm = -CUDART_INF_F, ll = 0.f, a = 0.f;
    for (int s0 = 0; s0 < num_splits; s0 += 8) {
      float mv[8], lv[8], av[8];
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        const bool in = s0 + s < num_splits;
        mv[s] = in ? part_ml[(base + s0 + s) * 2] : -CUDART_INF_F;
        lv[s] = in ? part_ml[(base + s0 + s) * 2 + 1] : 0.f;
        av[s] = in ? part_acc[(base + s0 + s) * hd + d] : 0.f;
      }
      float mx = mm;
#pragma unroll
      for (int s = 0; s < 8; ++s) mx = fmaxf(mx, mv[s]);
      if (mx == -CUDART_INF_F) continue;
      const float keep = __expf(mm - mx);   // 0 while nothing has been seen
      ll *= keep;
      a *= keep;
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        const float f = __expf(mv[s] - mx);   // exp(-inf) = 0 for splits that saw no key or do not exist
        ll += lv[s] * f;
        a += av[s] * f;
      }
      mm = mx;
    }
    o[d] = __float2bfloat16_rn(ll > 0.f ? a / ll : 0.f);
  }
}

template <int HD, bool FUSED>
int launch(const void* q, const FusedQkv& fq, const void* k_cache, const void* v_cache, void* out, float* part_acc,
           float* part_ml,
           const int* positions, const int* entry_of_token, const int* block_table, int bt_stride, int n_entries,
           int row0, int n_rows, int nq, int nkv, int page_size, int num_pages, int window, float scale,
           int num_splits, int* counters, int* status, cudaStream_t stream) {
  const int G = nq / nkv, gchunks = (G + 15) / 16;
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  CUtensorMap tmK, tmV;
  const unsigned long long cache_rows = (unsigned long long)num_pages * nkv * page_size;
  if (!ccb_tensor_map_2d(k_cache, cache_rows, HD, HD, 64, page_size, &tmK) ||
      !ccb_tensor_map_2d(v_cache, cache_rows, HD, HD, 64, page_size, &tmV))
    return CCB_REFUSE_ARG;
  const size_t smem = (size_t)2 * kStages * (HD / 64) * kHalfBytes + 64 + 16 * HD * 2 + (HD / 2) * 8 + HD * 4 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_tma_kernel<HD, FUSED>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(n_rows, nkv * gchunks, num_splits);
  ccb_launch_ex(FUSED && fq.k_cache != nullptr, attention_decode_tma_kernel<HD, FUSED>, grid, kThreads, smem, stream,
                tmK, tmV, (const __nv_bfloat16*)q, fq, (__nv_bfloat16*)out, part_acc, part_ml, positions, entry_of_token, block_table, bt_stride, n_entries,
             row0, nq, nkv, page_size, page_shift, num_pages, window, scale, num_splits, counters, status);
  int rc = ccb_launch_status();
  if (rc != 0 || num_splits == 1 || counters != nullptr) return rc;
  ccb_launch(attention_merge_bf16_kernel2, dim3(n_rows, nq), 128, 0, stream, (__nv_bfloat16*)out, part_acc, part_ml,
             row0, nq, HD, num_splits);
  return ccb_launch_status();
}

}  // namespace

// As ccb_attention_decode_mma, for page sizes that are a power of two from 8 to 64 (others: CCB_REFUSE_SIZE).
// `counters` (optional): n_rows * kv_heads * ceil(group / 16) ints that are zero before the first launch and
// are left zero; with them the splits are merged by the attention kernel itself, without them by a second
// kernel.
CCB_API int ccb_attention_decode_tma(const void* q, const void* k_cache, const void* v_cache, void* out,
                                     float* part_acc, float* part_ml, const int* positions,
                                     const int* entry_of_token, const int* block_table, int bt_stride,
                                     int n_entries, int row0, int n_rows, int nq, int nkv, int hd, int page_size,
                                     int num_pages, int window, float scale, int num_splits, int* counters,
                                     int* status, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || bt_stride <= 0 || num_splits <= 0 || num_splits > 64 ||
      page_size < 8 || page_size > 64 || (page_size & (page_size - 1)) != 0 ||
      ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15) != 0)
    return CCB_REFUSE_SIZE;
  if (num_splits > 1 && (part_acc == nullptr || part_ml == nullptr)) return CCB_REFUSE_ARG;
  const FusedQkv none = {};
  if (hd == 128)
    return launch<128, false>(q, none, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token,
                              block_table, bt_stride, n_entries, row0, n_rows, nq, nkv, page_size, num_pages, window,
                              scale, num_splits, counters, status, stream);
  if (hd == 64)
    return launch<64, false>(q, none, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token,
                             block_table, bt_stride, n_entries, row0, n_rows, nq, nkv, page_size, num_pages, window,
                             scale, num_splits, counters, status, stream);
  return CCB_REFUSE_SIZE;
}

// The same attention for rows that bring ONE new token each, straight from the q|k|v product: qkv[t, :] holds
// nq query heads, then nkv key heads, then nkv value heads (row stride qkv_stride).  The kernel applies the
// per-head norms (q_w, k_w: [hd] floats or null) and the rotate-half rotation (inv_freq: [hd / 2] or null)
// at positions[t], writes the row's key and value to their page (write_kv != 0; with 0 the cache belongs to
// another layer that has written the position already) and attends over positions <= positions[t].
// qk_norm_rope_kv_write is not needed for such rows.
CCB_API int ccb_attention_decode_tma_fused(const void* qkv, int qkv_stride, void* k_cache, void* v_cache, void* out,
                                           float* part_acc, float* part_ml, const int* positions,
                                           const int* entry_of_token, const int* block_table, int bt_stride,
                                           int n_entries, int row0, int n_rows, int nq, int nkv, int hd,
                                           int page_size, int num_pages, int window, float scale, int num_splits,
                                           const float* q_w, const float* k_w, float eps, const float* inv_freq,
                                           int write_kv, int* counters, int* status, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || bt_stride <= 0 || num_splits <= 0 || num_splits > 64 ||
      page_size < 8 || page_size > 64 || (page_size & (page_size - 1)) != 0 || (qkv_stride & 1) ||
      qkv_stride < (nq + (write_kv ? 2 * nkv : 0)) * hd ||
      ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(qkv) & 3) != 0)
    return CCB_REFUSE_SIZE;
  if (qkv == nullptr || (num_splits > 1 && (part_acc == nullptr || part_ml == nullptr))) return CCB_REFUSE_ARG;
  FusedQkv fq;
  fq.qkv = (const __nv_bfloat16*)qkv;
  fq.stride = qkv_stride;
  fq.q_w = q_w;
  fq.k_w = k_w;
  fq.eps = eps;
  fq.inv_freq = inv_freq;
  fq.k_cache = write_kv ? (__nv_bfloat16*)k_cache : nullptr;
  fq.v_cache = write_kv ? (__nv_bfloat16*)v_cache : nullptr;
  if (hd == 128)
    return launch<128, true>(nullptr, fq, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token,
                             block_table, bt_stride, n_entries, row0, n_rows, nq, nkv, page_size, num_pages, window,
                             scale, num_splits, counters, status, stream);
  if (hd == 64)
    return launch<64, true>(nullptr, fq, k_cache, v_cache, out, part_acc, part_ml, positions, entry_of_token,
                            block_table, bt_stride, n_entries, row0, n_rows, nq, nkv, page_size, num_pages, window,
                            scale, num_splits, counters, status, stream);
  return CCB_REFUSE_SIZE;
}
