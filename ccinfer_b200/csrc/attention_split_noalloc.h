// ccb_attention_split_noalloc: split-KV paged attention that allocates nothing.
//
// This entry point has no counterpart in 7QiC/ccInfer; it exists for users of this library whose code
// must not, or cannot, allocate device memory at the moment they need attention:
//   * a serving process that has handed ALL device memory to its own pools at start-up (weights, cache
//     pages), so that any later cudaMalloc would simply fail;
//   * a latency-critical decode loop in which an allocation call is forbidden because it synchronises the
//     whole device and may take milliseconds;
//   * a plug-in running under a host framework's allocator lock, where calling back into an allocator
//     (the framework's or CUDA's) can deadlock or fragment the framework's pool.
// Such callers still own their inputs and outputs and pass them in; only the kernel's scratch memory (the
// partial results of the key-range splits) is the library's business, and here it is a fixed array inside
// the library image instead of a buffer the caller has to provide.
//
// Same arguments and result as ccb_attention_split without the two scratch pointers.
//
// Limits and rules:
//   * n_rows * nq * num_splits * (hd + 2) must not exceed CCB_NOALLOC_SCRATCH_FLOATS (512 Ki floats =
//     2 MiB); more is refused with CCB_REFUSE_NOALLOC_TOO_LARGE and nothing is launched.  With
//     num_splits == 1 no scratch is used and any size goes.
//   * Every GPU that loads the library holds the 2 MiB array until the process exits.
//   * The FIRST call on a device looks up the array's device address (cudaGetSymbolAddress, checked); make
//     that first call during set-up, before any stream capture begins.  Later calls only launch kernels.
//   * It calls no cudaMalloc, cudaFree or any allocating library routine.
//   * All calls share the one array, which keeps the last call's contents.  Nothing in it has to start at
//     zero: each launch writes every slot it later reads.  Two calls that overlap on the GPU (different
//     streams, or the same call from two threads) race on the array; serialise them on one stream.
#pragma once

#include <cuda_runtime.h>

#define CCB_NOALLOC_SCRATCH_FLOATS (512 * 1024)
#define CCB_REFUSE_NOALLOC_TOO_LARGE (-5)

extern "C" __attribute__((visibility("default"))) int ccb_attention_split_noalloc(
    const void* q, const void* k_cache, const void* v_cache, void* out, const int* positions,
    const int* entry_of_token, const int* block_table, int bt_stride, int n_entries, int row0, int n_rows, int nq,
    int nkv, int hd, int page_size, int num_pages, int window, float scale, int num_splits, int dtype, int* status,
    cudaStream_t stream);
