// Random weights on the device: out[i] = std * z_i (+ 1 for norm weights), z ~ N(0, 1).
//
// 7QiC/ccInfer has no random-weights mode (it loads bfloat16 checkpoints only,
// src/model/qwen3/qwen3_weights.cpp:49-51); this one exists so that a model of any size can be made from a
// configuration and a seed, on the device where 65 GB of weights cannot come from a host generator in
// reasonable time.
//
// The stream is defined by integers and by single IEEE operations only, so that the host version
// (ccinfer_b200/weights/random_init.py, NumPy) gives the same bits:
//   words  = Philox4x32-10(counter = (g lo, g hi, tensor key lo, tensor key hi), key = (seed lo, seed hi)),
//            g = i / 4: one call serves the four consecutive elements 4g .. 4g + 3
//   pair   (words 0, 1) -> elements 4g, 4g + 1; (words 2, 3) -> elements 4g + 2, 4g + 3   (Box-Muller)
//   u      = ((w >> 9) + 0.5) / 2^23                         exact, in (0, 1)
//   ln u   = e ln 2 + ln m, u = m 2^e with m in (sqrt(1/2), sqrt 2]: s = (m - 1) / (m + 1),
//            ln m = 2 s + 2 s (s^2/3 + s^4/5 + s^6/7 + s^8/9 + s^10/11), Horner, every product and sum rounded
//   r      = sqrt(-2 ln u)
//   angle  : k = w' >> 8 (24 bits); octant o = k >> 21; x = ((k & 0x1FFFFF) + 0.5) / 2^21 * (pi / 4);
//            sin x and cos x by their Taylor polynomials on (0, pi/4); the octant places (cos, sin) on the circle
//   z      = r cos, r sin
// __fmul_rn and friends are never contracted into fused multiply-adds, which the host does not have.
#include "common.cuh"

namespace {

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                              uint32_t k1, uint32_t* out) {
  uint32_t c[4] = {c0, c1, c2, c3};
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
    c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c[0]; out[1] = c[1]; out[2] = c[2]; out[3] = c[3];
}

__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }

// two standard normal values from two 32-bit words
__device__ __forceinline__ void normal_pair(uint32_t wa, uint32_t wb, float& z0, float& z1) {
  const float u = mul(add((float)(wa >> 9), 0.5f), 1.0f / 8388608.0f);
  const uint32_t bits = __float_as_uint(u);
  int e = (int)(bits >> 23) - 127;
  float m = __uint_as_float((bits & 0x7FFFFFu) | 0x3F800000u);
  if (m > 1.41421354f) {
    m = mul(m, 0.5f);
    e += 1;
  }
  const float s = __fdiv_rn(__fsub_rn(m, 1.0f), add(m, 1.0f));
  const float s2 = mul(s, s);
  float poly = 1.0f / 11.0f;
  poly = add(mul(poly, s2), 1.0f / 9.0f);
  poly = add(mul(poly, s2), 1.0f / 7.0f);
  poly = add(mul(poly, s2), 1.0f / 5.0f);
  poly = add(mul(poly, s2), 1.0f / 3.0f);
  poly = mul(poly, s2);
  const float two_s = mul(2.0f, s);
  const float ln_m = add(two_s, mul(two_s, poly));
  const float ln_u = add(mul((float)e, 0.693147182f), ln_m);
  const float r = __fsqrt_rn(mul(-2.0f, ln_u));

  const uint32_t k = wb >> 8;
  const uint32_t oct = k >> 21;
  const float x = mul(mul(add((float)(k & 0x1FFFFFu), 0.5f), 1.0f / 2097152.0f), 0.785398185f);
  const float x2 = mul(x, x);
  float ps = 1.0f / 362880.0f;
  ps = add(mul(ps, x2), -1.0f / 5040.0f);
  ps = add(mul(ps, x2), 1.0f / 120.0f);
  ps = add(mul(ps, x2), -1.0f / 6.0f);
  const float sn = add(x, mul(mul(x, x2), ps));
  float pc = -1.0f / 3628800.0f;
  pc = add(mul(pc, x2), 1.0f / 40320.0f);
  pc = add(mul(pc, x2), -1.0f / 720.0f);
  pc = add(mul(pc, x2), 1.0f / 24.0f);
  pc = add(mul(pc, x2), -0.5f);
  const float cs = add(1.0f, mul(x2, pc));
  // (cos, sin) of a direction in octant `oct`: swapped in the odd octants, signs by quadrant
  const bool swap = ((oct + 1u) >> 1) & 1u;          // octants 1, 2, 5, 6
  float c = swap ? sn : cs, sv = swap ? cs : sn;
  if (oct >= 2u && oct <= 5u) c = -c;
  if (oct >= 4u) sv = -sv;
  z0 = mul(r, c);
  z1 = mul(r, sv);
}

template <typename T>
__global__ void __launch_bounds__(256)
init_random_kernel(T* __restrict__ out, long long numel, uint32_t seed_lo, uint32_t seed_hi, uint32_t key_lo,
                   uint32_t key_hi, float std, int add_one) {
  const long long groups = (numel + 3) / 4;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < groups;
       g += (long long)gridDim.x * blockDim.x) {
    uint32_t w[4];
    philox4x32_10((uint32_t)(g & 0xFFFFFFFFll), (uint32_t)(g >> 32), key_lo, key_hi, seed_lo, seed_hi, w);
    float z[4];
    normal_pair(w[0], w[1], z[0], z[1]);
    normal_pair(w[2], w[3], z[2], z[3]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float v = mul(z[i], std);
      if (add_one) v = add(v, 1.0f);
      const long long at = 4 * g + i;
      if (at < numel) out[at] = ccb::from_f32<T>(v);
    }
  }
}

}  // namespace

// out[numel] (float or bfloat16, rounded once from float) = std * z (+ 1 with add_one); the stream is that of
// (seed, key): key is the tensor's own 64-bit number (the loader derives it from the tensor's name).
CCB_API int ccb_init_random(void* out, long long numel, int dtype, unsigned long long seed,
                            unsigned long long key, float std, int add_one, void* stream) {
  if (numel < 0) return CCB_REFUSE_SIZE;
  if (numel == 0) return 0;
  if (out == nullptr) return CCB_REFUSE_ARG;
  const long long groups = (numel + 3) / 4;
  const int blocks = (int)((groups + 255) / 256 < 148 * 16 ? (groups + 255) / 256 : 148 * 16);
  const uint32_t s_lo = (uint32_t)(seed & 0xFFFFFFFFull), s_hi = (uint32_t)(seed >> 32);
  const uint32_t k_lo = (uint32_t)(key & 0xFFFFFFFFull), k_hi = (uint32_t)(key >> 32);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == CCB_F32)
    ccb_launch(init_random_kernel<float>, dim3(blocks), dim3(256), 0, st, (float*)out, numel, s_lo, s_hi, k_lo,
               k_hi, std, add_one);
  else if (dtype == CCB_BF16)
    ccb_launch(init_random_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, st, (__nv_bfloat16*)out, numel, s_lo,
               s_hi, k_lo, k_hi, std, add_one);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}
