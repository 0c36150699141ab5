// Host-side tensor maps for TMA (cuTensorMapEncodeTiled through the runtime's driver entry point).
#pragma once

#include <cuda.h>

// A cached map of a row-major bfloat16 matrix [rows, cols] with row stride `ld` elements (a multiple of 8),
// 16-byte aligned base, box = box_cols x box_rows elements (box_cols * 2 bytes <= 128), 128-byte swizzle,
// out-of-range elements read as zero.  False if the driver refuses the description.
bool ccb_tensor_map_2d(const void* ptr, unsigned long long rows, unsigned long long cols, unsigned long long ld,
                       unsigned box_cols, unsigned box_rows, CUtensorMap* out);

// The same without a swizzle: the box lies in shared memory as box_rows rows of box_cols elements (up to 256).
bool ccb_tensor_map_2d_plain(const void* ptr, unsigned long long rows, unsigned long long cols, unsigned long long ld,
                             unsigned box_cols, unsigned box_rows, CUtensorMap* out);
