// Greedy and temperature sampling over float logits, one parameter set per row.
//
// Greedy: argmax, ties to the lowest id (7QiC/ccInfer: src/kernel/sampling/sample.cu:32, 51-52).
// Temperature (the reference carries temperature and seed in its SamplingParams,
// src/base/types.h:54-60, but samples greedily only): the Gumbel-max draw
//   token = argmax_v( logit_v / T + G_v ),  G_v = -log(-log u_v),
// which is an exact draw from softmax(logits / T).  u_v comes from
// Philox4x32-10 with counter (v, output index, 0, 0) and key (seed, 0), so a
// request's draw depends on its seed and on how many tokens it has produced,
// never on the batch it shares a step with.
#include "common.cuh"
#include <math_constants.h>

namespace {

constexpr int kSampleThreads = 512;

__device__ __forceinline__ uint32_t philox_first_word(uint32_t c0, uint32_t c1, uint32_t k0) {
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
  return c[0];
}

__device__ __forceinline__ float gumbel(uint32_t v, uint32_t out_index, uint32_t seed) {
  const uint32_t r = philox_first_word(v, out_index, seed);
  const float u = ((float)(r >> 9) + 0.5f) * (1.0f / 8388608.0f);  // exact: 24 significant bits
  return -logf(-logf(u));
}

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
  return v > bv || (v == bv && i < bi);
}

__global__ void __launch_bounds__(kSampleThreads)
sample_rows_kernel(const float* __restrict__ logits, size_t ld, int* __restrict__ tokens,
                   const float* __restrict__ temperature, const unsigned* __restrict__ seed,
                   const int* __restrict__ out_index, int V, const int* __restrict__ slot_of_row,
                   int* __restrict__ by_slot, int n_slots) {
  ccb::pdl_begin();
  __shared__ float sv[kSampleThreads];
  __shared__ int si[kSampleThreads];
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * ld;
  const float temp = temperature ? temperature[r] : 0.f;
  float bv = -CUDART_INF_F;
  int bi = 0x7fffffff;
  if (temp > 0.f) {
    const float inv_t = 1.0f / temp;
    const uint32_t sd = seed[r], oi = (uint32_t)out_index[r];
    for (int v = threadIdx.x; v < V; v += kSampleThreads) {
      const float z = row[v] * inv_t + gumbel((uint32_t)v, oi, sd);
      if (better(z, v, bv, bi)) { bv = z; bi = v; }
    }
  } else {
    for (int v = threadIdx.x; v < V; v += kSampleThreads) {
      const float z = row[v];
      if (better(z, v, bv, bi)) { bv = z; bi = v; }
    }
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

CCB_API int ccb_sample_rows(const float* logits, long long ld, int* tokens, const float* temperature,
                            const unsigned* seed, const int* out_index, int R, int V, const int* slot_of_row,
                            int* by_slot, int n_slots, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0 || ld < V) return CCB_REFUSE_SIZE;
  if (temperature != nullptr && (seed == nullptr || out_index == nullptr)) return CCB_REFUSE_ARG;
  if (slot_of_row != nullptr && (by_slot == nullptr || n_slots <= 0)) return CCB_REFUSE_ARG;
  ccb_launch(sample_rows_kernel, R, kSampleThreads, 0, stream, logits, (size_t)ld, tokens, temperature, seed, out_index, V,
             slot_of_row, by_slot, n_slots);
  return ccb_launch_status();
}
