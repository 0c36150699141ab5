// bfloat16 matrix product on the 5th-generation tensor cores: C[M, N] = A[M, K] * W[N, K]^T.
//
// Blackwell-native: operand tiles travel global -> shared memory by TMA (cp.async.bulk.tensor, 128-byte
// swizzle), one elected thread issues tcgen05.mma (M = 128, K = 16 per instruction) with the accumulator in
// tensor memory, tcgen05.commit signals mbarriers, and four epilogue warps read the accumulator back with
// tcgen05.ld.  Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer (and TMEM owner), warps 2..5 = epilogue.
// (7QiC/ccInfer runs this product in cuBLAS, src/backend/cuda/cuda_backend.cpp:82-108.)
//
// Two orientations of the same kernel, both operands K-major as they are stored:
//   normal (M > 64):  tile rows = 128 tokens, tile columns = BN = 256 features.
//   swapped (M <= 64, decode): tile rows = 128 FEATURES (the weight matrix is the M side), tile columns =
//       the 16/32/64 tokens.  The product is then a stream of W through TMA; to give every SM a share, K is
//       cut into `splits` slices that run as separate blocks.  Each block writes its float partial tile to
//       scratch; the block that arrives last at the tile's counter adds the slices in ascending order (a
//       fixed order, so the result does not depend on which block was last) and writes C.
//
// Every wait on an mbarrier is bounded: after kWaitLimit failed polls the thread records
// CCB_ST_WAIT_TIMEOUT in the status word and leaves its loop; the block still reaches its teardown, frees
// its tensor memory and returns.
#include "common.cuh"
#include <cuda.h>
#include <cudaTypedefs.h>
#include <map>
#include <mutex>
#include <tuple>

#include "tc_common.cuh"
#include "tma_host.h"

using namespace ccb;

namespace {

constexpr int BM = 128;           // tile rows (TMEM lanes)
constexpr int BK = 64;            // k elements per stage: one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int kThreadsTc = 192;

// instruction descriptor: float accumulate, bfloat16 x bfloat16, both K-major, M = 128, N = n
__host__ __device__ constexpr uint32_t instr_desc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

template <typename TOut> __device__ __forceinline__ void store16(TOut* dst, const uint32_t* v, int n_valid);
template <> __device__ __forceinline__ void store16<float>(float* dst, const uint32_t* v, int n_valid) {
  if (n_valid >= 16 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      reinterpret_cast<uint4*>(dst)[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
    for (int i = 0; i < n_valid; ++i) dst[i] = __uint_as_float(v[i]);
  }
}
template <>
__device__ __forceinline__ void store16<__nv_bfloat16>(__nv_bfloat16* dst, const uint32_t* v, int n_valid) {
  if (n_valid >= 16 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    uint32_t p[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
      p[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    reinterpret_cast<uint4*>(dst)[0] = make_uint4(p[0], p[1], p[2], p[3]);
    reinterpret_cast<uint4*>(dst)[1] = make_uint4(p[4], p[5], p[6], p[7]);
  } else {
    for (int i = 0; i < n_valid; ++i) dst[i] = __float2bfloat16_rn(__uint_as_float(v[i]));
  }
}

// The factor of an RMSNorm that has no kernel of its own: token t of the result is multiplied by
// 1 / sqrt(sum_p ssq_in[t * parts + p] / dim + eps), p < parts, before the activation if there is one (the
// product before this one left bf16(h * w_norm) as the tokens and the partial sums of h^2; see gemm_fewrows.cu).
// Swapped products of at most 16 tokens without split-K only.  ssq_in == null: off.
struct CcbRowScale {
  const float* ssq_in;
  int parts;
  float dim, eps;
};

// ---------------------------------------------------------------------------------------------
// rowsA / rowsB: valid rows of the matrices behind tmA (tile 128) and tmB (tile BN).
// SWAP = false: C[rowA, rowB];  SWAP = true: C[rowB, rowA] (A = weights, B = tokens), with split-K.
// ---------------------------------------------------------------------------------------------
template <int BN, int STAGES, bool SWAP, typename TOut>
__global__ void __launch_bounds__(kThreadsTc, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, TOut* __restrict__ C,
               int ldc, int rowsA, int rowsB, int K, int splits, float* __restrict__ partial,
               int* __restrict__ counters, int swiglu, const CcbRowScale rs, int* status) {
  __shared__ float s_scale[16];
  constexpr int B_STAGE_BYTES = BN * BK * 2;
  constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + STAGES * B_STAGE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
  int* last_flag = reinterpret_cast<int*>(tmem_slot + 1);
  const uint32_t full0 = s32(bars), empty0 = s32(bars + STAGES), tfull = s32(bars + 2 * STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tileA = blockIdx.x, tileB = blockIdx.y, split = blockIdx.z;
  const int kb_total = (K + BK - 1) / BK;
  const int per = (kb_total + splits - 1) / splits;
  const int kb0 = split * per;
  const int nkb = min(kb0 + per, kb_total) - kb0;  // the host makes every slice non-empty

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(tfull, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // the whole warp allocates the accumulator's columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer ----
      // The weight operand does not depend on the kernel before this one: its first copies start at once
      // and run while that kernel finishes; the token operand waits for it (programmatic dependent launch).
      const int pre = min(nkb, STAGES);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(full0 + 8 * i, A_STAGE_BYTES + B_STAGE_BYTES);
        if (SWAP)
          tma_load_2d(s32(sA + i * A_STAGE_BYTES), &tmA, (kb0 + i) * BK, tileA * BM, full0 + 8 * i);
        else
          tma_load_2d(s32(sB + i * B_STAGE_BYTES), &tmB, (kb0 + i) * BK, tileB * BN, full0 + 8 * i);
      }
      pdl_wait();
      pdl_trigger();
      for (int i = 0; i < pre; ++i) {
        if (SWAP)
          tma_load_2d(s32(sB + i * B_STAGE_BYTES), &tmB, (kb0 + i) * BK, tileB * BN, full0 + 8 * i);
        else
          tma_load_2d(s32(sA + i * A_STAGE_BYTES), &tmA, (kb0 + i) * BK, tileA * BM, full0 + 8 * i);
      }
      for (int i = pre; i < nkb; ++i) {
        const int s = i % STAGES, ph = (i / STAGES) & 1;
        if (!mbar_wait(empty0 + 8 * s, ph ^ 1)) {
          set_status(status, CCB_ST_WAIT_TIMEOUT);
          break;
        }
        mbar_expect_tx(full0 + 8 * s, A_STAGE_BYTES + B_STAGE_BYTES);
        tma_load_2d(s32(sA + s * A_STAGE_BYTES), &tmA, (kb0 + i) * BK, tileA * BM, full0 + 8 * s);
        tma_load_2d(s32(sB + s * B_STAGE_BYTES), &tmB, (kb0 + i) * BK, tileB * BN, full0 + 8 * s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---- MMA issuer ----
      constexpr uint32_t idesc = instr_desc(BN);
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES, ph = (i / STAGES) & 1;
        if (!mbar_wait(full0 + 8 * s, ph)) {
          set_status(status, CCB_ST_WAIT_TIMEOUT);
          break;
        }
        tc_fence_after();
        const uint64_t da = smem_desc(s32(sA + s * A_STAGE_BYTES));
        const uint64_t db = smem_desc(s32(sB + s * B_STAGE_BYTES));
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          tc_mma(tmem_base, da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        tc_commit(empty0 + 8 * s);  // arrives when these products no longer read the stage
      }
      tc_commit(tfull);  // arrives when the accumulator is complete
    }
  } else {  // ---- epilogue: warp q reads TMEM lanes 32 q .. 32 q + 31 ----
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const bool scaled = SWAP && BN == 16 && rs.ssq_in != nullptr;
    if (scaled) {  // while the products run: the factor of each token, partial sums in the order of their blocks
      pdl_wait();
      for (int tok = q; tok < 16; tok += 4) {
        const float ss = tok < rowsB ? row_ssq(rs.ssq_in + (size_t)tok * rs.parts, rs.parts, lane) : 0.f;
        if (lane == 0) s_scale[tok] = 1.0f / sqrtf(ss / rs.dim + rs.eps);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    const bool ok = mbar_wait(tfull, 0);
    if (!ok && lane == 0) set_status(status, CCB_ST_WAIT_TIMEOUT);
    tc_fence_after();
    const int ga = tileA * BM + row;  // row of the A-side matrix
    if (ok) {
      if (!SWAP) {
        TOut* crow = C + (size_t)ga * ldc + (size_t)tileB * BN;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          uint32_t v[16];
          tc_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + c0, v);
          tc_wait_ld();
          const int n_valid = min(16, rowsB - (tileB * BN + c0));
          if (ga < rowsA && n_valid > 0) store16<TOut>(crow + c0, v, n_valid);
        }
      } else if (BN == 16 && swiglu) {
        // The weight rows come in blocks of 64 gate rows followed by the 64 up rows of the same channels:
        // lanes 0..63 of this tile hold gate, lanes 64..127 up.  The up half goes through shared memory
        // (the stages are idle: every product has completed), the gate half computes silu(g) * u and
        // writes C[token, 64 tileA + lane]: the activation, without a round trip of gate|up through memory.
        float* xch = reinterpret_cast<float*>(sA);  // [64][17]
        uint32_t v[16];
        tc_ld16(tmem_base + ((uint32_t)(q * 32) << 16), v);
        tc_wait_ld();
        if (q >= 2) {
#pragma unroll
          for (int j = 0; j < 16; ++j) xch[(row - 64) * 17 + j] = __uint_as_float(v[j]);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (q < 2 && tileA * BM + 64 + row < rowsA) {
          const int ch = tileA * 64 + row;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (j < rowsB) {
              float g = __uint_as_float(v[j]), u = xch[row * 17 + j];
              if (scaled) g *= s_scale[j], u *= s_scale[j];
              C[(size_t)j * ldc + ch] = from_f32<TOut>(g / (1.f + __expf(-g)) * u);
            }
          }
        }
      } else if (splits == 1) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          uint32_t v[16];
          tc_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + c0, v);
          tc_wait_ld();
          if (ga < rowsA) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int t = tileB * BN + c0 + j;
              if (t < rowsB) C[(size_t)t * ldc + ga] = from_f32<TOut>(__uint_as_float(v[j]) * (scaled ? s_scale[j] : 1.f));
            }
          }
        }
      } else {
        // this slice's partial tile -> scratch [split][token][feature]
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          uint32_t v[16];
          tc_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + c0, v);
          tc_wait_ld();
          if (ga < rowsA) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int t = tileB * BN + c0 + j;
              if (t < rowsB) partial[((size_t)split * rowsB + t) * rowsA + ga] = __uint_as_float(v[j]);
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
        if (threadIdx.x == 64) {
          __threadfence();  // cumulative: the whole block's partial sums are visible before its count is
          const int old = atomicAdd(&counters[tileA * gridDim.y + tileB], 1);
          *last_flag = (old == splits - 1) ? 1 : 0;
          if (old == splits - 1) counters[tileA * gridDim.y + tileB] = 0;  // ready for the next launch
          __threadfence();
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*last_flag) {
          const int t_begin = tileB * BN, t_end = min(rowsB, tileB * BN + BN);
          const size_t slice = (size_t)rowsB * rowsA;
          if ((rowsA & 3) == 0 && (ldc & 3) == 0) {
            // a warp per token, a lane per four features: the slices of a token arrive as 16-byte loads
            // that are all in flight at once, and are added in ascending order (a fixed order)
            const int f = tileA * BM + 4 * lane;
            if (f < rowsA) {  // rowsA % 4 == 0: the four features are all inside
#pragma unroll 2
              for (int t = t_begin + q; t < t_end; t += 4) {
                const float* src = partial + (size_t)t * rowsA + f;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
                for (int s0 = 0; s0 < splits; s0 += 8) {
                  float4 v[8];
#pragma unroll
                  for (int s = 0; s < 8; ++s)
                    v[s] = s0 + s < splits ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)(s0 + s) * slice))
                                           : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                  for (int s = 0; s < 8; ++s) {  // slices beyond `splits` are exact zeros
                    acc.x += v[s].x;
                    acc.y += v[s].y;
                    acc.z += v[s].z;
                    acc.w += v[s].w;
                  }
                }
                TOut* dst = C + (size_t)t * ldc + f;
                if constexpr (sizeof(TOut) == 4) {
                  *reinterpret_cast<float4*>(dst) = acc;
                } else {
                  const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y);
                  const __nv_bfloat162 hi = __floats2bfloat162_rn(acc.z, acc.w);
                  uint2 pk;
                  pk.x = *reinterpret_cast<const uint32_t*>(&lo);
                  pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                  *reinterpret_cast<uint2*>(dst) = pk;
                }
              }
            }
          } else if (ga < rowsA) {  // odd widths: a thread per feature
#pragma unroll 1
            for (int t = t_begin; t < t_end; ++t) {
              float acc = 0.f;
              for (int s = 0; s < splits; ++s) acc += __ldcg(&partial[(size_t)s * slice + (size_t)t * rowsA + ga]);
              C[(size_t)t * ldc + ga] = from_f32<TOut>(acc);
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

}  // namespace

// tensor maps are cached by (pointer, rows, columns, row stride, box, swizzle): weights and the engine's scratch
// buffers keep their addresses for the life of the process
static std::mutex g_mu;
static std::map<std::tuple<const void*, unsigned long long, unsigned long long, unsigned long long, unsigned, unsigned, int>,
                CUtensorMap> g_maps;

static bool tensor_map_2d(const void* ptr, unsigned long long rows, unsigned long long cols, unsigned long long ld,
                          unsigned box_cols, unsigned box_rows, bool swizzle128, CUtensorMap* out) {
  const auto key = std::make_tuple(ptr, rows, cols, ld, box_cols, box_rows, swizzle128 ? 1 : 0);
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return true;
  }
  auto fn = encode_fn();
  if (fn == nullptr) return false;
  CUtensorMap tm;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps[key] = tm;
  *out = tm;
  return true;
}

bool ccb_tensor_map_2d(const void* ptr, unsigned long long rows, unsigned long long cols, unsigned long long ld,
                       unsigned box_cols, unsigned box_rows, CUtensorMap* out) {
  return tensor_map_2d(ptr, rows, cols, ld, box_cols, box_rows, true, out);
}

bool ccb_tensor_map_2d_plain(const void* ptr, unsigned long long rows, unsigned long long cols, unsigned long long ld,
                             unsigned box_cols, unsigned box_rows, CUtensorMap* out) {
  return tensor_map_2d(ptr, rows, cols, ld, box_cols, box_rows, false, out);
}

namespace {

bool tensor_map(const void* ptr, int rows, int K, int ld, int box_rows, CUtensorMap* out) {
  return ccb_tensor_map_2d(ptr, rows, K, ld, BK, box_rows, out);
}

template <int BN, int STAGES, bool SWAP, typename TOut>
int launch_tc(const CUtensorMap& tmA, const CUtensorMap& tmB, void* C, int ldc, int rowsA, int rowsB, int K,
              int splits, float* partial, int* counters, int* status, cudaStream_t stream, int swiglu = 0,
              const CcbRowScale& rs = CcbRowScale{}) {
  constexpr size_t smem = (size_t)STAGES * (A_STAGE_BYTES + BN * BK * 2) + (2 * STAGES + 1) * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, SWAP, TOut>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((rowsA + BM - 1) / BM, (rowsB + BN - 1) / BN, splits);
  ccb_launch_ex(true, gemm_tc_kernel<BN, STAGES, SWAP, TOut>, grid, kThreadsTc, smem, stream, 
      tmA, tmB, (TOut*)C, ldc, rowsA, rowsB, K, splits, partial, counters, swiglu, rs, status);
  return ccb_launch_status();
}

template <typename TOut>
int dispatch(void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldc, int splits,
             float* partial, int* counters, int* status, cudaStream_t stream) {
  CUtensorMap tmW, tmX;
  if (M <= 64) {  // swapped: weights are the 128-row side
    const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    if (!tensor_map(W, N, K, ldw, BM, &tmW) || !tensor_map(A, M, K, lda, bn, &tmX)) return CCB_REFUSE_ARG;
    if (bn == 16)
      return launch_tc<16, 6, true, TOut>(tmW, tmX, C, ldc, N, M, K, splits, partial, counters, status, stream);
    if (bn == 32)
      return launch_tc<32, 6, true, TOut>(tmW, tmX, C, ldc, N, M, K, splits, partial, counters, status, stream);
    return launch_tc<64, 4, true, TOut>(tmW, tmX, C, ldc, N, M, K, splits, partial, counters, status, stream);
  }
  if (!tensor_map(A, M, K, lda, BM, &tmX) || !tensor_map(W, N, K, ldw, 256, &tmW)) return CCB_REFUSE_ARG;
  return launch_tc<256, 4, false, TOut>(tmX, tmW, C, ldc, M, N, K, 1, nullptr, nullptr, status, stream);
}

}  // namespace

// splits > 1 only with M <= 64; then `partial` holds splits * M * N floats and `counters`
// ceil(N / 128) ints that are zero before the first launch (the kernel leaves them zero).
// K and the row strides must be multiples of 8 elements, the bases 16-byte aligned.
CCB_API int ccb_gemm_tc_bf16(void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldc,
                             int out_dtype, int splits, float* partial, int* counters, int* status,
                             cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (out_dtype != CCB_F32 && out_dtype != CCB_BF16) return CCB_REFUSE_DTYPE;
  if (K <= 0 || (K & 7) || lda < K || ldw < K || ldc < N || (lda & 7) || (ldw & 7) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
    return CCB_REFUSE_SIZE;
  const int kb_total = (K + BK - 1) / BK;
  if (splits < 1 || splits > 16 || splits > kb_total || (splits > 1 && (M > 64 || partial == nullptr || counters == nullptr)))
    return CCB_REFUSE_ARG;
  if (splits > 1) {  // every slice must hold at least one k block
    const int per = (kb_total + splits - 1) / splits;
    if ((splits - 1) * per >= kb_total) return CCB_REFUSE_ARG;
  }
  if (out_dtype == CCB_F32)
    return dispatch<float>(C, A, W, M, N, K, lda, ldw, ldc, splits, partial, counters, status, stream);
  return dispatch<__nv_bfloat16>(C, A, W, M, N, K, lda, ldw, ldc, splits, partial, counters, status, stream);
}

// act[M, F] = silu(A W_gate^T) * (A W_up^T) in one kernel, for M <= 16 tokens.  W [2F, K] holds the rows in
// blocks: 64 gate rows, then the 64 up rows of the same channels (F a multiple of 64), so that one 128-row
// tile of the tensor-core product owns matching gate and up channels.  The products are accumulated in
// float and the activation is rounded once (7QiC/ccInfer rounds gate and up to bfloat16 first:
// src/model/qwen3/qwen3_model.cpp:325-370, src/kernel/mlp/silu_mul.cu:24-28).
static int tc_swiglu(void* act, const void* A, const void* W, int M, int F, int K, int lda, int ldw, int ld_act,
                     const CcbRowScale& rs, int* status, cudaStream_t stream) {
  if (M <= 0 || F <= 0) return 0;
  if (M > 16 || (F & 63)) return CCB_REFUSE_SIZE;
  if (K <= 0 || (K & 7) || lda < K || ldw < K || ld_act < F || (lda & 7) || (ldw & 7) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
    return CCB_REFUSE_SIZE;
  CUtensorMap tmW, tmX;
  if (!tensor_map(W, 2 * F, K, ldw, BM, &tmW) || !tensor_map(A, M, K, lda, 16, &tmX)) return CCB_REFUSE_ARG;
  return launch_tc<16, 6, true, __nv_bfloat16>(tmW, tmX, act, ld_act, 2 * F, M, K, 1, nullptr, nullptr, status, stream, 1, rs);
}

CCB_API int ccb_gemm_tc_swiglu_bf16(void* act, const void* A, const void* W, int M, int F, int K, int lda, int ldw,
                                    int ld_act, int* status, cudaStream_t stream) {
  return tc_swiglu(act, A, W, M, F, K, lda, ldw, ld_act, CcbRowScale{}, status, stream);
}

// The same with the factor of a norm for every token (see CcbRowScale).
CCB_API int ccb_gemm_tc_swiglu_scaled_bf16(void* act, const void* A, const void* W, int M, int F, int K, int lda,
                                           int ldw, int ld_act, const float* ssq_in, int parts, float dim, float eps,
                                           int* status, cudaStream_t stream) {
  if (ssq_in == nullptr || parts <= 0 || !(dim > 0.f)) return CCB_REFUSE_ARG;
  return tc_swiglu(act, A, W, M, F, K, lda, ldw, ld_act, CcbRowScale{ssq_in, parts, dim, eps}, status, stream);
}
