// bfloat16 matrix product for many rows with TWO SMs on one tile: C[M, N] = A[M, K] * W[N, K]^T.
//
// One SM cannot feed its tensor core at full rate with both operands in shared memory: a product of
// 128 x 256 x 16 reads 12 KB in its 128 cycles while the copies that refill the stages write as much again,
// and shared memory delivers 128 bytes a cycle (a persistent kernel with one block per tile of 128 x 256
// stopped at 74 % of the tensor pipe: 303 us for 2,048 x 24,576 x 4,096 against the library's 263).
// Here a cluster of two blocks works on a tile of 256 rows x 256 features (tcgen05 cta_group::2): each
// block holds 128 of the rows (its A half) and 128 of the features (its B half), the leader's one thread
// issues products of M = 256 that read both blocks' shared memory and accumulate in both blocks' tensor
// memory, so every SM reads and writes half as much per product (259 us for the same product).
// One cluster per pair of SMs walks over the tiles (row tiles fastest, so that the clusters running at one
// time share a few weight tiles in L2); the TMA producers and the MMA issuer run on from one tile into the
// next, so the ring of six stages never drains and tensor maps and tensor memory are set up once; the
// accumulator has two buffers of 256 columns: while the epilogue warps read one out, convert and store it,
// the products of the next tile fill the other.
// SWIGLU: the weight rows come in blocks of 64 gate rows and the 64 up rows of the same channels; a thread
// holds a row's 256 accumulator columns, so silu(gate) * up needs no exchange: the tile writes 128 outputs.
//
// Who tells whom (all mbarriers, every wait bounded):
//   full[s]       both blocks' copies of stage s have landed     the copies of BOTH blocks count their bytes on the
//                                                                leader's barrier (cp.async.bulk.tensor cta_group::2)
//   empty[s]      the products no longer read the stage          leader's tcgen05.commit, multicast to both blocks
//   tfull[b]      accumulator b is complete                      leader's tcgen05.commit, multicast to both blocks
//   tempty[b]     accumulator b has been read out                four epilogue warps of each block -> leader (8 arrivals)
// (7QiC/ccInfer runs this product in cuBLAS, src/backend/cuda/cuda_backend.cpp:82-108.)
#include "common.cuh"
#include <cuda.h>

#include "tc_common.cuh"
#include "tma_host.h"

using namespace ccb;

namespace {

constexpr int PBM = 128;          // rows per block (TMEM lanes); the pair's tile has 256
constexpr int PBN = 256;          // features per tile; each block loads 128 of them
constexpr int PBK = 64;
constexpr int PSTAGES = 6;
constexpr int P_A_BYTES = PBM * PBK * 2;          // 16 KB
constexpr int P_B_BYTES = (PBN / 2) * PBK * 2;    // 16 KB
constexpr int kPairGemmThreads = 192;
constexpr int PACC = 2;           // accumulators of 256 columns in tensor memory

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address, in the cluster's shared window, of `local_addr` inside block `rank`
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kWaitLimit; ++i)
    if (mbar_try_wait_cluster(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void tc_mma2(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives, once the products issued so far are complete, at the barrier at this offset in BOTH blocks
__device__ __forceinline__ void tc_commit2(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(mask)
               : "memory");
}

// A tile copy into THIS block's shared memory whose bytes are counted on a barrier of the pair's leader
// (`bar_cluster`: an address in the cluster's shared window).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* tm, int c0, int c1, uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tm), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}

template <typename TOut> __device__ __forceinline__ void pstore16(TOut* dst, const uint32_t* v, int n_valid);
template <> __device__ __forceinline__ void pstore16<float>(float* dst, const uint32_t* v, int n_valid) {
  if (n_valid >= 16 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      reinterpret_cast<uint4*>(dst)[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (i < n_valid) dst[i] = __uint_as_float(v[i]);
  }
}
template <>
__device__ __forceinline__ void pstore16<__nv_bfloat16>(__nv_bfloat16* dst, const uint32_t* v, int n_valid) {
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
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (i < n_valid) dst[i] = __float2bfloat16_rn(__uint_as_float(v[i]));
  }
}

template <bool SWIGLU, typename TOut>
__global__ void __launch_bounds__(kPairGemmThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    TOut* __restrict__ C, int ldc, int rowsA, int rowsB, int K, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + PSTAGES * P_A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + PSTAGES * P_B_BYTES);
  const uint32_t full0 = s32(bars), empty0 = s32(bars + PSTAGES), tfull0 = s32(bars + 2 * PSTAGES),
                 tempty0 = s32(bars + 2 * PSTAGES + 2);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * PSTAGES + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int tiles_m = (rowsA + 2 * PBM - 1) / (2 * PBM), tiles_n = (rowsB + PBN - 1) / PBN;
  const int n_tiles = tiles_m * tiles_n;
  const int nkb = (K + PBK - 1) / PBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PSTAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < PACC; ++b) {
      mbar_init(tfull0 + 8 * b, 1);
      mbar_init(tempty0 + 8 * b, 8);   // four epilogue warps of each block
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // a warp of EACH block of the pair allocates: the columns are taken in both
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"((uint32_t)(PACC * PBN))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // both blocks' barriers exist before anybody signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer: this block's half of A (rows) and of B (features) ----
      pdl_wait();
      pdl_trigger();
      int it = 0;
      bool alive = true;
      for (int t = pair; t < n_tiles && alive; t += n_pairs) {
        const int tm = t % tiles_m, tn = t / tiles_m;
        const int a_row = tm * 2 * PBM + (int)rank * PBM, b_row = tn * PBN + (int)rank * (PBN / 2);
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % PSTAGES, ph = (it / PSTAGES) & 1;
          if (!mbar_wait_cluster(empty0 + 8 * s, ph ^ 1)) {
            set_status(status, CCB_ST_WAIT_TIMEOUT);
            alive = false;
            break;
          }
          // the leader expects the bytes of both blocks; the peer's may even land first (the count goes below
          // zero for a moment, the phase cannot complete before the leader's arrival)
          const uint32_t bar = map_to_rank(full0 + 8 * s, 0);
          if (leader) mbar_expect_tx(full0 + 8 * s, 2 * (P_A_BYTES + P_B_BYTES));
          tma_load_2d_pair(s32(sA + s * P_A_BYTES), &tmA, kb * PBK, a_row, bar);
          tma_load_2d_pair(s32(sB + s * P_B_BYTES), &tmB, kb * PBK, b_row, bar);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {  // ---- MMA issuer (the leader's): products of M = 256 over both blocks ----
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(PBN >> 3) << 17) |
                                 ((uint32_t)((2 * PBM) >> 4) << 24);
      int it = 0, local = 0;
      bool alive = true;
      for (int t = pair; t < n_tiles && alive; t += n_pairs, ++local) {
        const int buf = local % PACC;
        if (!mbar_wait_cluster(tempty0 + 8 * buf, ((local / PACC) & 1) ^ 1)) {
          set_status(status, CCB_ST_WAIT_TIMEOUT);
          break;
        }
        tc_fence_after();
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % PSTAGES, ph = (it / PSTAGES) & 1;
          if (!mbar_wait_cluster(full0 + 8 * s, ph)) {
            set_status(status, CCB_ST_WAIT_TIMEOUT);
            alive = false;
            break;
          }
          tc_fence_after();
          const uint64_t da = smem_desc(s32(sA + s * P_A_BYTES));
          const uint64_t db = smem_desc(s32(sB + s * P_B_BYTES));
#pragma unroll
          for (int k = 0; k < PBK / 16; ++k)
            tc_mma2(tmem_base + buf * PBN, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit2(empty0 + 8 * s);
        }
        if (alive) tc_commit2(tfull0 + 8 * buf);
      }
    }
  } else {  // ---- epilogue: this block's 128 rows of the tile, all 256 features ----
    const int q = warp & 3;
    const int row = q * 32 + lane;
    int local = 0;
    for (int t = pair; t < n_tiles; t += n_pairs, ++local) {
      const int tm = t % tiles_m, tn = t / tiles_m;
      const int buf = local % PACC;
      if (!mbar_wait_cluster(tfull0 + 8 * buf, (local / PACC) & 1)) {
        if (lane == 0) set_status(status, CCB_ST_WAIT_TIMEOUT);
        break;
      }
      tc_fence_after();
      const int ga = tm * 2 * PBM + (int)rank * PBM + row;
      const uint32_t taddr = tmem_base + buf * PBN + ((uint32_t)(q * 32) << 16);
      if (!SWIGLU) {
        TOut* crow = C + (size_t)ga * ldc + (size_t)tn * PBN;
#pragma unroll 1
        for (int c0 = 0; c0 < PBN; c0 += 32) {
          uint32_t v[32];
          tc_ld32(taddr + c0, v);
          tc_wait_ld();
          if (ga < rowsA) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int n_valid = min(16, rowsB - (tn * PBN + c0 + 16 * h));
              if (n_valid > 0) pstore16<TOut>(crow + c0 + 16 * h, v + 16 * h, n_valid);
            }
          }
        }
      } else {
        TOut* crow = C + (size_t)ga * ldc + (size_t)tn * (PBN / 2);
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
#pragma unroll 1
          for (int c0 = 0; c0 < 64; c0 += 32) {
            uint32_t g[32], u[32];
            tc_ld32(taddr + half * 128 + c0, g);
            tc_ld32(taddr + half * 128 + 64 + c0, u);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float gv = __uint_as_float(g[j]);
              g[j] = __float_as_uint(gv / (1.f + __expf(-gv)) * __uint_as_float(u[j]));
            }
            if (ga < rowsA) {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int n_valid = min(16, rowsB / 2 - (tn * (PBN / 2) + half * 64 + c0 + 16 * h));
                if (n_valid > 0) pstore16<TOut>(crow + half * 64 + c0 + 16 * h, g + 16 * h, n_valid);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {   // this warp's quarter of this block's accumulator is free again: the leader counts eight
        if (leader) mbar_arrive(tempty0 + 8 * buf);
        else mbar_arrive_remote(map_to_rank(tempty0 + 8 * buf, 0));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // nobody leaves while the other block may still signal it or read its shared memory
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(PACC * PBN)) : "memory");
  }
}

template <bool SWIGLU, typename TOut>
int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, void* C, int ldc, int M, int N, int K, int sms, int* status,
                cudaStream_t stream) {
  constexpr size_t smem = (size_t)PSTAGES * (P_A_BYTES + P_B_BYTES) + (2 * PSTAGES + 4) * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<SWIGLU, TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = ((M + 2 * PBM - 1) / (2 * PBM)) * ((N + PBN - 1) / PBN);
  int pairs = sms / 2;
  if (pairs > tiles) pairs = tiles;
  if (pairs < 1) pairs = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(kPairGemmThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<SWIGLU, TOut>, tmA, tmB, (TOut*)C, ldc, M, N, K, status);
  return ccb_launch_status();
}

}  // namespace

// C[M, N] = A[M, K] W[N, K]^T (bfloat16 operands, bfloat16 or float result), a pair of SMs per 256 x 256 tile.
// swiglu: W [N = 2F, K] in blocks of 64 gate and 64 up rows (F a multiple of 64), C [M, F] = silu(gate) * up.
// K and the row strides are multiples of 8 elements, the bases 16-byte aligned.
CCB_API int ccb_gemm_tc_pair_bf16(void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldc,
                                  int out_dtype, int swiglu, int sms, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (out_dtype != CCB_F32 && out_dtype != CCB_BF16) return CCB_REFUSE_DTYPE;
  if (K <= 0 || (K & 7) || lda < K || ldw < K || ldc < (swiglu ? N / 2 : N) || (lda & 7) || (ldw & 7) || sms < 2 ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) || (swiglu && (N & 127)))
    return CCB_REFUSE_SIZE;
  CUtensorMap tmX, tmW;
  if (!ccb_tensor_map_2d(A, M, K, lda, PBK, PBM, &tmX) || !ccb_tensor_map_2d(W, N, K, ldw, PBK, PBN / 2, &tmW))
    return CCB_REFUSE_ARG;
  if (swiglu) {
    if (out_dtype != CCB_BF16) return CCB_REFUSE_DTYPE;
    return launch_pair<true, __nv_bfloat16>(tmX, tmW, C, ldc, M, N, K, sms, status, stream);
  }
  if (out_dtype == CCB_F32) return launch_pair<false, float>(tmX, tmW, C, ldc, M, N, K, sms, status, stream);
  return launch_pair<false, __nv_bfloat16>(tmX, tmW, C, ldc, M, N, K, sms, status, stream);
}
