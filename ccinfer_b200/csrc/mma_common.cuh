// Warp-level tensor-core and asynchronous-copy primitives shared by the bfloat16 attention kernels.
//
// mma.sync.m16n8k16 (bf16 x bf16 -> float) fragment layout, lane = 4 * gid + tig:
//   A (16 x 16, row):  a0 = (row gid,     cols 2 tig, 2 tig + 1)    a1 = (row gid + 8, same cols)
//                      a2 = (row gid,     cols 2 tig + 8, + 9)      a3 = (row gid + 8, cols 2 tig + 8, + 9)
//   B (16 x 8, col):   b0 = (k 2 tig, 2 tig + 1; n gid)             b1 = (k 2 tig + 8, + 9; n gid)
//   C (16 x 8):        c0, c1 = (row gid, cols 2 tig, + 1)          c2, c3 = (row gid + 8, same cols)
// ldmatrix.x4 reads four 8 x 8 matrices of 16-bit elements; lane i gives the address of row i % 8 of
// matrix i / 8, and register j of a lane holds (row gid, cols 2 tig, + 1) of matrix j, or with .trans
// (rows 2 tig, + 1; col gid).
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace ccb {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte asynchronous copy global -> shared; when !valid nothing is read and zeros are written
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                                  uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// Shared-memory tile of rows of HD bfloat16, 16-byte chunks XOR-swizzled by the row so that the eight
// rows an ldmatrix reads fall into different banks.  HD is a power of two >= 64.
template <int HD> __device__ __forceinline__ int swz(int row, int chunk) {
  return row * HD + ((chunk ^ (row & 7)) << 3);
}

}  // namespace ccb
