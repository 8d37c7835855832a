// Device helpers of the host executor (init.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace s1 {
// kind 0: mean + std * N(0,1); kind 1: uniform in [mean, mean + std). n bf16 values.
int fill_bf16(void* out, size_t n, uint64_t seed, float mean, float std, int kind, cudaStream_t st);
// out[s] = x[ends[s] - 1] for rows of D bf16 (D % 8 == 0); ends on the device.
int gather_rows(const void* x, const int* ends_device, void* out, int nseq, int D, cudaStream_t st);
// Copies `packs` 16-byte pieces from src to dst + row0[i] * row_packs for each of n <= 16 rows i:
// one block of rows (the conv tail of a prefix) in front of every continuation of a pack.
int spread_block(void* dst, size_t row_packs, const int* row0, int n, const void* src, size_t packs, cudaStream_t st);
}  // namespace s1
