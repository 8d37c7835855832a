// Host-side TMA tensor maps for row-major bf16 matrices (shared by the tcgen05 kernels).
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace s1 {
// Tensor map of a row-major bf16 matrix [rows, cols] whose rows are row_stride elements apart
// (a multiple of 8), read in boxes of [box_rows, 64 columns] with the 128-byte swizzle. Rows and
// columns outside the matrix read as zero. Maps are cached by their arguments. False when the
// driver entry point is missing or refuses the arguments (base not 16-byte aligned, ...).
bool tensor_map_2d(const void* ptr, uint64_t rows, uint64_t cols, uint64_t row_stride, uint32_t box_rows,
                   CUtensorMap* out);
// The same without swizzle: boxes of [box_rows, box_cols] (box_cols * 2 bytes a multiple of 16, at
// most 256 columns) land densely packed, row after row.
bool tensor_map_2d_plain(const void* ptr, uint64_t rows, uint64_t cols, uint64_t row_stride, uint32_t box_rows,
                         uint32_t box_cols, CUtensorMap* out);
}  // namespace s1
