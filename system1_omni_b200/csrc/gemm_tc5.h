// Internal interface of the tcgen05 GEMM engine (gemm_tc5.cu), used by gemm.cu.
#pragma once
#include <cuda_runtime.h>

// True when the tcgen05 kernel can run this problem: K a multiple of 8 (16-byte rows for the
// TMA tensor maps) and at least 64, x and w 16-byte aligned.
bool s1_gemm_tc5_supported(const void* x, const void* w, const void* y, int M, int N, int K, int ldy);
// Queues y [M, N] (rows of ldy) = x [M, K] * w [N, K]^T on `stream`. Returns 0, a cudaError_t
// or CS1_ERR_TENSOR_MAP.
int s1_gemm_tc5(const void* x, const void* w, void* y, int M, int N, int K, int ldy, cudaStream_t stream);
