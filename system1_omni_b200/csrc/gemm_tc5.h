// Internal interface of the tcgen05 GEMM engine (gemm_tc5.cu), used by gemm.cu.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

// Device memory a GEMM handle lends the engine for K-split problems: float32 partial tiles
// and one counter per (tile, block of the pair). The counters must be zero when a launch
// starts; the kernel leaves them zero. Two launches that may overlap on the GPU must not
// share it (one handle serves one stream, as in the reference).
struct S1GemmScratch {
    void* partials;
    size_t partial_bytes;
    int* counters;
    int counter_slots;
};

// True when the tcgen05 kernel can run this problem: K a multiple of 8 (16-byte rows for the
// TMA tensor maps) and at least 64, x and w 16-byte aligned.
bool s1_gemm_tc5_supported(const void* x, const void* w, const void* y, int M, int N, int K, int ldy);
// Queues y [M, N] (rows of ldy) = x [M, K] * w [N, K]^T on `stream`. scratch may be null (no
// K split is used then). Returns 0, a cudaError_t or CS1_ERR_TENSOR_MAP.
int s1_gemm_tc5(const void* x, const void* w, void* y, int M, int N, int K, int ldy, const S1GemmScratch* scratch,
                cudaStream_t stream);

// y [M, N] (rows of ldy) = bf16(x w^T + bias), bias [N] bf16 added to the float32 sum before the one
// rounding; whole tiles on the single-block kernel, any M. Same support rule and return codes.
int s1_gemm_tc5_bias(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, int ldy,
                     cudaStream_t stream);

// The MLP's first half in one kernel: act [M, I] (rows of ld) = silu(x w[0:I]^T) * (x w[I:2I]^T),
// each projection rounded to bf16 before the activation (bit-identical to the GEMM followed
// by the SiLU-multiply operator). Needs more than 128 rows (the pair kernel).
bool s1_gemm_tc5_swiglu_supported(const void* x, const void* w, int M, int I, int K);
int s1_gemm_tc5_swiglu(const void* x, const void* w, void* act, int M, int I, int K, int ld, cudaStream_t stream);
