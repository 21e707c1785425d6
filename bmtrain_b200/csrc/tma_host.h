// Host-side helper shared by the tensor-core kernels: cached cuTensorMapEncodeTiled for 16-bit element tensors.
#pragma once
#include <cuda.h>
#include <stdint.h>

// 4-D map with dims {inner, rows, nb0, nb1}; `ld`, `bs0`, `bs1` are the element strides of dims 1..3 (multiples of 8,
// base pointer 16-byte aligned).  128-byte swizzle, zero fill outside the tensor.  Returns 0, or a negative code
// (-10 driver entry point missing, -11 alignment, -12 encode failed).
int bmt_tma_map_4d(CUtensorMap* out, const void* ptr, int dtype, int64_t inner, int64_t rows, int64_t ld, int64_t nb0, int64_t bs0,
                   int64_t nb1, int64_t bs1, int box_inner, int box_rows);
