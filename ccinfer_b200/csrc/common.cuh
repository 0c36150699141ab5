// Shared device helpers of the ccinfer_b200 kernels (sm_100a).
//
// Every kernel family is instantiated for two element types: float (the true
// 32-bit path) and __nv_bfloat16 (the serving path).  Arithmetic is always
// done in float; only loads and stores see the storage type.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <utility>

#define CCB_API extern "C" __attribute__((visibility("default")))

// dtype codes of the C interface
enum { CCB_F32 = 0, CCB_BF16 = 1 };

// bits of the device status word (set by kernels, never cleared by them)
enum {
  CCB_ST_BAD_TOKEN = 1,   // token id outside [0, vocab)
  CCB_ST_BAD_SLOT = 2,    // cache slot outside the pool
  CCB_ST_BAD_PAGE = 4,    // block-table entry outside the pool where a key was needed
  CCB_ST_BAD_ROW = 8,     // row index outside the batch
  CCB_ST_WAIT_TIMEOUT = 16  // a bounded mbarrier wait gave up
};

namespace ccb {

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of kThreads (a multiple of 32, at most 1024) in a fixed
// order: lanes by butterfly, then the warps' partial sums one after another.
// Every thread gets the result.  `red` holds at least 32 floats.
template <int kThreads>
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();  // red may still be read from an earlier call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w) total += red[w];
  return total;
}

// Programmatic dependent launch.  A kernel launched with the attribute may start while its predecessor in
// the stream still runs; `pdl_wait` blocks until the predecessor has completed and its writes are visible,
// `pdl_trigger` lets the successor start early in turn.  Without the attribute both are no-ops.
// Every kernel calls pdl_begin() (or the two halves, with read-only prefetching of weights in between)
// before it touches memory that another kernel may have written.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Kernels without weights to prefetch: wait for the predecessor, then let the successor start (a product
// then streams its first weight tiles while this kernel runs).  The order matters: a kernel that let its
// successor in BEFORE its predecessor had finished would put three kernels on the device at once, and a
// product's blocks, resident but waiting, would keep the predecessor's last blocks from being scheduled.
__device__ __forceinline__ void pdl_begin() {
  pdl_wait();
  pdl_trigger();
}

// Sum of a row of `n` partial sums by one warp, every lane with the result; the order of the additions is
// fixed (by lane, then a shuffle tree).  The loads are asked for together, not one after the other's use.
__device__ __forceinline__ float row_ssq(const float* row, int n, int lane) {
  float ss = 0.f;
  if ((n & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const float4* row4 = reinterpret_cast<const float4*>(row);
#pragma unroll 4
    for (int p = lane; p < (n >> 2); p += 32) {
      const float4 v = __ldcg(row4 + p);
      ss += (v.x + v.y) + (v.z + v.w);
    }
  } else {
#pragma unroll 4
    for (int p = lane; p < n; p += 32) ss += __ldcg(row + p);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  return ss;
}

__device__ __forceinline__ void set_status(int* status, int bit) {
  if (status != nullptr) atomicOr(status, bit);
}

}  // namespace ccb

// Host side: every launcher returns the CUDA error code of its launch (0 = ok)
// or a negative number for an argument it refuses.
#define CCB_REFUSE_SIZE (-2)
#define CCB_REFUSE_DTYPE (-3)
#define CCB_REFUSE_ARG (-4)

static inline int ccb_launch_status() { return (int)cudaGetLastError(); }

// One switch for the whole library (ccb_set_pdl): launch kernels with programmatic stream serialization.
extern int g_ccb_pdl;

// `early`: this kernel gains from starting before its predecessor has finished (it prefetches weights).
template <typename... KArgs, typename... Args>
static inline void ccb_launch_ex(bool early, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (g_ccb_pdl && (early || g_ccb_pdl > 1)) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);  // the error is read by ccb_launch_status()
}

template <typename... KArgs, typename... Args>
static inline void ccb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  ccb_launch_ex(false, kernel, grid, block, smem, stream, static_cast<Args&&>(args)...);
}
