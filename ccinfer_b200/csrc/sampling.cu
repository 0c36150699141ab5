// Greedy, temperature, top-k and top-p sampling over float logits, one parameter set per row.
//
// Greedy: argmax, ties to the lowest id (7QiC/ccInfer: src/kernel/sampling/sample.cu:32, 51-52).
// Temperature (the reference carries temperature and seed in its SamplingParams,
// src/base/types.h:54-60, but samples greedily only): the Gumbel-max draw
//   token = argmax_v( logit_v / T + G_v ),  G_v = -log(-log u_v),
// which is an exact draw from softmax(logits / T).  u_v is word v % 4 of
// Philox4x32-10 with counter (v / 4, output index, 0, 0) and key (seed, 0), so a
// request's draw depends on its seed and on how many tokens it has produced,
// never on the batch it shares a step with.
// top-k / top-p (named by the reference's SamplingParams and request fields, src/base/types.h:54-60,
// src/http/http_server.cpp:529-555, which refuses them): the draw is restricted to the logits at or above a
// threshold.  top-k: the k-th largest logit.  top-p, within the top-k set: the largest threshold whose set
// still holds a share p of the set's probability at the row's temperature (the smallest set of most probable
// tokens that reaches p; ties at the threshold are all kept).  Both thresholds are found exactly over the
// order-preserving integer image of the floats, by a 256-way search of four levels, each one pass over the
// row into integer bins (see Search below).
#include "common.cuh"
#include <math_constants.h>

namespace {

constexpr int kSampleThreads = 512;

__device__ __forceinline__ void philox4(uint32_t c0, uint32_t c1, uint32_t k0, uint32_t* out) {
  uint32_t c[4] = {c0, c1, 0u, 0u};
  uint32_t k[2] = {k0, 0u};
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k[0], n2 = hi0 ^ c[3] ^ k[1];
    c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
    k[0] += 0x9E3779B9u;
    k[1] += 0xBB67AE85u;
  }
  out[0] = c[0]; out[1] = c[1]; out[2] = c[2]; out[3] = c[3];
}

__device__ __forceinline__ float gumbel_of(uint32_t r) {
  const float u = ((float)(r >> 9) + 0.5f) * (1.0f / 8388608.0f);  // exact: 24 significant bits
  return -logf(-logf(u));
}

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
  return v > bv || (v == bv && i < bi);
}

// Every logit of the row once; a thread asks for eight of its logits before it looks at the first.  The
// bodies of the loops below branch and add atomically, which keeps the compiler from overlapping the loads
// by itself: with one load in flight per thread a pass over 150,000 logits took 29 us, most of a top-p
// draw's 0.4 ms.
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* __restrict__ row, int V, F f) {
  constexpr int U = 8;
  int v = threadIdx.x;
  for (; v + (U - 1) * kSampleThreads < V; v += U * kSampleThreads) {
    float l[U];
#pragma unroll
    for (int u = 0; u < U; ++u) l[u] = row[v + u * kSampleThreads];
#pragma unroll
    for (int u = 0; u < U; ++u) f(v + u * kSampleThreads, l[u]);
  }
  for (; v < V; v += kSampleThreads) f(v, row[v]);
}

// order-preserving image of a float in the unsigned integers; NaN counts as the smallest value
__device__ __forceinline__ uint32_t float_key(float f) {
  if (f != f) return 0u;
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// ---------------------------------------------------------------------------------------------
// Thresholds of top-k and top-p: the largest key T such that the logits with key >= T number at least k
// (top-k), or hold at least the wanted probability mass (top-p).  Found exactly by a 256-way search: the
// range of keys that still holds T is cut into 256 equal bins, one pass over the row adds every logit of
// the range to its bin (counts, or masses in 2^-40 fixed point: integer sums do not depend on the order
// of the atomic additions, so the result is the same in every run), warp 0 walks the bins from the top
// until the target is reached, and the search goes on inside that bin: four levels from 2^32 keys to one.
// The first range is [smallest key, largest key], so the bins follow the spread of the row's logits and
// few lanes of a warp meet at the same bin.
// ---------------------------------------------------------------------------------------------
constexpr int kBins = 256;

struct Search {
  uint32_t hist_lo[kBins], hist_hi[kBins];   // a bin's sum: 2^32 hist_hi + hist_lo
  uint32_t bin_kmin[kBins], bin_kmax[kBins]; // first level of top-p: the keys that fell into a bin
  uint32_t lo;                  // keys [lo, lo + 2^wl) still hold the threshold,
  uint32_t limit;               // and none above this one
  int wl;
  unsigned long long above;     // count or mass of the keys above the range
  unsigned long long target;
  uint32_t ured[2 * (kSampleThreads / 32)];
};

// One level: `value(logit, key)` is what a logit adds (0: nothing).  The range is cut into up to 256 bins of
// 2^shift keys (a shift, not a division, per logit).  With share >= 0 the target is first set to that
// share of everything added (the first level of top-p).  Afterwards the range is the bin in which
// `above + bins from the top` reaches the target.
template <typename F>
__device__ void search_level(Search& S, const float* __restrict__ row, int V, double share, F value) {
  for (int i = threadIdx.x; i < kBins; i += kSampleThreads) S.hist_lo[i] = S.hist_hi[i] = 0u;
  __syncthreads();
  const uint32_t lo = S.lo;
  const int wl = S.wl, shift = wl > 8 ? wl - 8 : 0;
  const uint32_t limit = S.limit;
  const unsigned long long width = 1ull << wl;
  for_each_logit(row, V, [&](int v, float l) {
    const uint32_t key = float_key(l);
    const unsigned long long off = (unsigned long long)key - lo;
    if (key >= lo && off < width && key <= limit) {
      const unsigned long long q = value(l, key);
      if (q) {
        // two native 32-bit additions with the carry taken over by hand: integer sums, so the order in
        // which the lanes arrive does not matter (64-bit shared-memory atomics are compare-and-swap loops)
        const int b = (int)(off >> shift);
        const uint32_t ql = (uint32_t)q, qh = (uint32_t)(q >> 32);
        const uint32_t old = atomicAdd(&S.hist_lo[b], ql);
        const uint32_t carry = old > 0xffffffffu - ql ? 1u : 0u;
        if (qh + carry) atomicAdd(&S.hist_hi[b], qh + carry);
      }
    }
  });
  __syncthreads();
  if (threadIdx.x < 32) {  // warp 0: lane i owns bins 8 i .. 8 i + 7; walk from the top
    const int lane = threadIdx.x;
    constexpr int PER = kBins / 32;
    auto bin_sum = [&](int b) { return ((unsigned long long)S.hist_hi[b] << 32) + S.hist_lo[b]; };
    unsigned long long mine = 0ull;
#pragma unroll
    for (int j = 0; j < PER; ++j) mine += bin_sum(lane * PER + j);
    unsigned long long higher = 0ull, all = 0ull;  // the lanes above this one; every lane
    for (int l = 31; l >= 0; --l) {
      const unsigned long long x = __shfl_sync(0xffffffffu, mine, l);
      all += x;
      if (l > lane) higher += x;
    }
    unsigned long long tgt = S.target;
    if (share >= 0.0) {
      tgt = (unsigned long long)ceil(share * (double)(all + S.above));
      if (tgt < 1ull) tgt = 1ull;
    }
    __syncwarp();
    const unsigned long long acc0 = S.above + higher;
    if (acc0 < tgt && acc0 + mine >= tgt) {  // the target is reached inside this lane's bins
      unsigned long long acc = acc0;
      int b = lane * PER + PER - 1;
      for (; b > lane * PER; --b) {
        if (acc + bin_sum(b) >= tgt) break;
        acc += bin_sum(b);
      }
      S.above = acc;
      S.lo = lo + ((uint32_t)b << shift);
      S.wl = shift;
      S.target = tgt;
    }
  }
  __syncthreads();
}

// First level of top-p.  Bins of equal width in the logit's VALUE (not in its key: keys go by exponent, so
// equal key ranges put most of a row's logits into a handful of bins, and additions of different values
// to one shared-memory word are done one after another: 0.3 ms for 150,000 logits).  The bin of a logit is
// a non-decreasing function of its value, so the bins still cut the keys into ranges in order; which keys
// a bin holds is noted while it is filled (smallest and largest key: integer minima and maxima, the same
// in every run).  Sets the target to the share p of all the mass and narrows the range to the bin where
// the mass counted from the top reaches it.
template <typename F>
__device__ void first_level_by_value(Search& S, const float* __restrict__ row, int V, float p, float l_lo, float l_hi,
                                     uint32_t key_lo, F value) {
  for (int i = threadIdx.x; i < kBins; i += kSampleThreads) {
    S.hist_lo[i] = S.hist_hi[i] = 0u;
    S.bin_kmin[i] = 0xffffffffu;
    S.bin_kmax[i] = 0u;
  }
  __syncthreads();
  const float scale = (float)kBins / (l_hi - l_lo);
  for_each_logit(row, V, [&](int v, float l) {
    const uint32_t key = float_key(l);
    if (key < key_lo) return;
    const unsigned long long q = value(l, key);
    int b = (int)((l - l_lo) * scale);
    b = b < 0 ? 0 : (b > kBins - 1 ? kBins - 1 : b);
    atomicMin(&S.bin_kmin[b], key);
    atomicMax(&S.bin_kmax[b], key);
    if (q) {
      const uint32_t ql = (uint32_t)q, qh = (uint32_t)(q >> 32);
      const uint32_t old = atomicAdd(&S.hist_lo[b], ql);
      const uint32_t carry = old > 0xffffffffu - ql ? 1u : 0u;
      if (qh + carry) atomicAdd(&S.hist_hi[b], qh + carry);
    }
  });
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    constexpr int PER = kBins / 32;
    auto bin_sum = [&](int b) { return ((unsigned long long)S.hist_hi[b] << 32) + S.hist_lo[b]; };
    unsigned long long mine = 0ull;
#pragma unroll
    for (int j = 0; j < PER; ++j) mine += bin_sum(lane * PER + j);
    unsigned long long higher = 0ull, all = 0ull;
    for (int l = 31; l >= 0; --l) {
      const unsigned long long x = __shfl_sync(0xffffffffu, mine, l);
      all += x;
      if (l > lane) higher += x;
    }
    unsigned long long tgt = (unsigned long long)ceil((double)p * (double)all);
    if (tgt < 1ull) tgt = 1ull;
    __syncwarp();
    if (higher < tgt && higher + mine >= tgt) {
      unsigned long long acc = higher;
      int b = lane * PER + PER - 1;
      for (; b > lane * PER; --b) {
        if (acc + bin_sum(b) >= tgt) break;
        acc += bin_sum(b);
      }
      S.above = acc;
      S.lo = S.bin_kmin[b];
      S.limit = S.bin_kmax[b];   // the power-of-two range below may reach into the next bin's keys
      S.wl = 0;
      while ((1ull << S.wl) < (unsigned long long)S.bin_kmax[b] - S.bin_kmin[b] + 1ull) ++S.wl;
      S.target = tgt;
    }
  }
  __syncthreads();
}

// bits of the smallest power of two that holds n keys
__device__ __forceinline__ int width_log2(unsigned long long n) {
  int wl = 0;
  while ((1ull << wl) < n) ++wl;
  return wl;
}

// The smallest key that a logit must have to be drawn (0: every logit).
__device__ uint32_t draw_threshold(const float* __restrict__ row, int V, int k, float p, float inv_t, Search& S) {
  // the row's smallest and largest key
  uint32_t kmin = 0xffffffffu, kmax = 0u;
  for_each_logit(row, V, [&](int, float l) {
    const uint32_t key = float_key(l);
    kmin = min(kmin, key);
    kmax = max(kmax, key);
  });
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    kmin = min(kmin, __shfl_xor_sync(0xffffffffu, kmin, o));
    kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) {
    S.ured[2 * (threadIdx.x >> 5)] = kmin;
    S.ured[2 * (threadIdx.x >> 5) + 1] = kmax;
  }
  __syncthreads();
  for (int w = 0; w < kSampleThreads / 32; ++w) {
    kmin = min(kmin, S.ured[2 * w]);
    kmax = max(kmax, S.ured[2 * w + 1]);
  }
  __syncthreads();
  uint32_t thr = 0u;
  if (k > 0 && k < V) {  // the k-th largest key
    if (threadIdx.x == 0) {
      S.lo = kmin;
      S.limit = 0xffffffffu;
      S.wl = width_log2((unsigned long long)kmax - kmin + 1ull);
      S.above = 0ull;
      S.target = (unsigned long long)k;
    }
    __syncthreads();
    for (int level = 0; level < 5 && S.wl > 0; ++level)   // at most four levels; the limit is a safeguard
      search_level(S, row, V, -1.0, [](float, uint32_t) { return 1ull; });
    thr = S.lo;
    __syncthreads();
  }
  if (p < 1.f) {
    const float m = __uint_as_float((kmax & 0x80000000u) ? (kmax & 0x7fffffffu) : ~kmax);  // the largest logit
    const uint32_t floor_key = thr;  // masses are those of the top-k set
    auto mass = [&](float l, uint32_t key) -> unsigned long long {
      if (key < floor_key) return 0ull;
      return (unsigned long long)(__expf((l - m) * inv_t) * 1099511627776.0f);  // 2^40
    };
    const uint32_t key_lo = max(kmin, floor_key);
    const float l_lo = __uint_as_float((key_lo & 0x80000000u) ? (key_lo & 0x7fffffffu) : ~key_lo);
    if (key_lo >= kmax) {
      thr = key_lo;  // one value only
    } else if (m - l_lo < 3.0e38f) {
      first_level_by_value(S, row, V, p, l_lo, m, key_lo, mass);
      for (int level = 0; level < 5 && S.wl > 0; ++level) search_level(S, row, V, -1.0, mass);
      thr = max(S.lo, floor_key);
    } else {  // infinite logits: bins by key all the way
      if (threadIdx.x == 0) {
        S.lo = key_lo;
        S.limit = 0xffffffffu;
        S.wl = width_log2((unsigned long long)kmax - key_lo + 1ull);
        S.above = 0ull;
        S.target = 1ull;
      }
      __syncthreads();
      for (int level = 0; level < 5 && (level == 0 || S.wl > 0); ++level)
        search_level(S, row, V, level == 0 ? (double)p : -1.0, mass);
      thr = max(S.lo, floor_key);
    }
    __syncthreads();
  }
  return thr;
}

__global__ void __launch_bounds__(kSampleThreads)
sample_rows_kernel(const float* __restrict__ logits, size_t ld, int* __restrict__ tokens,
                   const float* __restrict__ temperature, const unsigned* __restrict__ seed,
                   const int* __restrict__ out_index, const int* __restrict__ top_k,
                   const float* __restrict__ top_p, int V, const int* __restrict__ slot_of_row,
                   int* __restrict__ by_slot, int n_slots) {
  ccb::pdl_begin();
  __shared__ float sv[kSampleThreads];
  __shared__ int si[kSampleThreads];
  __shared__ Search search;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * ld;
  const float temp = temperature ? temperature[r] : 0.f;
  float bv = -CUDART_INF_F;
  int bi = 0x7fffffff;
  if (temp > 0.f) {
    const float inv_t = 1.0f / temp;
    const uint32_t sd = seed[r], oi = (uint32_t)out_index[r];
    const int k = top_k ? top_k[r] : 0;
    const float p = top_p ? top_p[r] : 1.f;
    const uint32_t thr = (k > 0 || p < 1.f) ? draw_threshold(row, V, k, p, inv_t, search) : 0u;
    // four consecutive logits share one call of the generator
    auto draw4 = [&](int g, const float* l, int n) {
      bool any = thr == 0u;
      for (int i = 0; i < n && !any; ++i) any = float_key(l[i]) >= thr;
      if (!any) return;
      uint32_t rnd[4];
      philox4((uint32_t)g, oi, sd, rnd);
      for (int i = 0; i < n; ++i) {
        if (thr != 0u && float_key(l[i]) < thr) continue;
        const float z = l[i] * inv_t + gumbel_of(rnd[i]);
        if (better(z, 4 * g + i, bv, bi)) { bv = z; bi = 4 * g + i; }
      }
    };
    const int groups = V >> 2;
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
      constexpr int U = 4;  // groups a thread asks for at once
      int g = threadIdx.x;
      for (; g + (U - 1) * kSampleThreads < groups; g += U * kSampleThreads) {
        float4 x[U];
#pragma unroll
        for (int u = 0; u < U; ++u) x[u] = reinterpret_cast<const float4*>(row)[g + u * kSampleThreads];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const float l[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
          draw4(g + u * kSampleThreads, l, 4);
        }
      }
      for (; g < groups; g += kSampleThreads) {
        const float4 x = reinterpret_cast<const float4*>(row)[g];
        const float l[4] = {x.x, x.y, x.z, x.w};
        draw4(g, l, 4);
      }
    } else {
      for (int g = threadIdx.x; g < groups; g += kSampleThreads) {
        const float l[4] = {row[4 * g], row[4 * g + 1], row[4 * g + 2], row[4 * g + 3]};
        draw4(g, l, 4);
      }
    }
    if (threadIdx.x == 0 && (V & 3)) {  // the last, short group
      float l[4] = {0.f, 0.f, 0.f, 0.f};
      for (int i = 0; i < (V & 3); ++i) l[i] = row[4 * groups + i];
      draw4(groups, l, V & 3);
    }
  } else {
    for_each_logit(row, V, [&](int v, float z) {
      if (better(z, v, bv, bi)) { bv = z; bi = v; }
    });
  }
  sv[threadIdx.x] = bv;
  si[threadIdx.x] = bi;
  __syncthreads();
  for (int s = kSampleThreads / 2; s > 0; s >>= 1) {
    if (threadIdx.x < s && better(sv[threadIdx.x + s], si[threadIdx.x + s], sv[threadIdx.x], si[threadIdx.x])) {
      sv[threadIdx.x] = sv[threadIdx.x + s];
      si[threadIdx.x] = si[threadIdx.x + s];
    }
    __syncthreads();
  }
  // a row of NaNs or -inf only leaves the sentinel: report id 0 as the reference's kernel does
  if (threadIdx.x == 0) {
    const int tok = si[0] == 0x7fffffff ? 0 : si[0];
    tokens[r] = tok;
    // also kept per request slot, where the next step's embedding finds it without a round trip to the host
    if (slot_of_row != nullptr) {
      const int s = slot_of_row[r];
      if (s >= 0 && s < n_slots) by_slot[s] = tok;
    }
  }
}

}  // namespace

// top_k (int [R], 0 = off) and top_p (float [R], >= 1 = off) may be null; they apply to rows with a
// temperature above zero.
CCB_API int ccb_sample_rows(const float* logits, long long ld, int* tokens, const float* temperature,
                            const unsigned* seed, const int* out_index, const int* top_k, const float* top_p, int R,
                            int V, const int* slot_of_row, int* by_slot, int n_slots, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0 || ld < V) return CCB_REFUSE_SIZE;
  if (temperature != nullptr && (seed == nullptr || out_index == nullptr)) return CCB_REFUSE_ARG;
  if (slot_of_row != nullptr && (by_slot == nullptr || n_slots <= 0)) return CCB_REFUSE_ARG;
  if ((top_k != nullptr || top_p != nullptr) && temperature == nullptr) return CCB_REFUSE_ARG;
  ccb_launch(sample_rows_kernel, R, kSampleThreads, 0, stream, logits, (size_t)ld, tokens, temperature, seed, out_index,
             top_k, top_p, V, slot_of_row, by_slot, n_slots);
  return ccb_launch_status();
}
