// y [M, N] (rows of ldy) = x [M, K] * w [N, K]^T in bf16 with float32 accumulation: every
// projection of the decoder (reference entry: src/backends/cuda/qwen3_5/gemm.cu:103-135, where
// it is a cuBLASLt call). One engine: the tcgen05 kernels of gemm_tc5.cu take every problem
// whose rows TMA can address (K a multiple of 8 and at least 64, 16-byte aligned operands); the
// few that it cannot - ragged K, unaligned views, the float32 product of unmerged LoRA factors
// - run on the plain CUDA-core kernel below. No vendor library is linked.
#include <cuda_runtime.h>
#include <stdlib.h>

#include "common.cuh"
#include "cs1_ops.h"
#include "gemm_tc5.h"
#include "s1_executor.h"

namespace s1 {
namespace {

constexpr int COUNTER_SLOTS = 16384;
constexpr size_t PARTIAL_BYTES = (size_t)48 << 20;

// What cs1_gemm_create hands back: scratch the tcgen05 kernel's shared-tile schedules use
// (float32 partial tiles and one counter per tile and block of a pair). The caller's
// workspace_bytes is the reference's cuBLASLt workspace and has no use here.
struct Gemm {
    int* counters = nullptr;
    void* partials = nullptr;
    size_t partial_bytes = 0;
};

S1GemmScratch scratch_of(Gemm* g) { return S1GemmScratch{g->partials, g->partial_bytes, g->counters, COUNTER_SLOTS}; }

__device__ __forceinline__ float as_f32(float x) { return x; }
__device__ __forceinline__ float as_f32(bf16 x) { return f32(x); }
__device__ __forceinline__ void put(float* p, float v) { *p = v; }
__device__ __forceinline__ void put(bf16* p, float v) { *p = to_bf16(v); }

// The plain product for what the tensor-core path cannot address: a block computes a 64 x 64
// tile of y from 16-wide slices of x and w staged in shared memory as float32, a thread a 4 x 4
// corner of it, summing over k in order with float32 FMAs (no TF32, no reordering), bias (bf16,
// nullable) added to the float32 sum before the one rounding. Any sizes, any alignment.
constexpr int ST = 64, SK = 16;
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
    gemm_plain_kernel(const TI* __restrict__ x, const TI* __restrict__ w, const bf16* __restrict__ bias, TO* __restrict__ y,
                      int M, int N, int K, int ldy) {
    grid_dep_trigger();
    __shared__ float xs[SK][ST + 4], wsm[SK][ST + 4];
    const int m0 = blockIdx.y * ST, n0 = blockIdx.x * ST;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4] = {};
    grid_dep_sync();
    for (int k0 = 0; k0 < K; k0 += SK) {
        for (int i = threadIdx.x; i < ST * SK; i += 256) {
            const int r = i / SK, kk = i % SK;
            xs[kk][r] = (m0 + r < M && k0 + kk < K) ? as_f32(x[(size_t)(m0 + r) * K + k0 + kk]) : 0.f;
            wsm[kk][r] = (n0 + r < N && k0 + kk < K) ? as_f32(w[(size_t)(n0 + r) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < SK; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                a[i] = xs[kk][ty * 4 + i];
                b[i] = wsm[kk][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) put(y + (size_t)m * ldy + n, acc[i][j] + (bias ? f32(bias[n]) : 0.f));
        }
}

template <typename TI, typename TO>
int gemm_plain(const TI* x, const TI* w, const bf16* bias, TO* y, int M, int N, int K, int ldy, cudaStream_t st) {
    const dim3 grid((N + ST - 1) / ST, (M + ST - 1) / ST);
    return launch_dep(gemm_plain_kernel<TI, TO>, grid, 256, 0, st, x, w, bias, y, M, N, K, ldy);
}

}  // namespace
}  // namespace s1

using namespace s1;

extern "C" void* cs1_gemm_create(size_t workspace_bytes) {
    (void)workspace_bytes;
    Gemm* g = new Gemm();
    // counters of the tcgen05 kernel's shared-tile schedules; zero between launches
    if (cudaMalloc(reinterpret_cast<void**>(&g->counters), COUNTER_SLOTS * sizeof(int)) != cudaSuccess ||
        cudaMemset(g->counters, 0, COUNTER_SLOTS * sizeof(int)) != cudaSuccess) {
        if (g->counters) cudaFree(g->counters);
        cudaGetLastError();
        delete g;
        return nullptr;
    }
    // Room for two 256 x 256 float32 partial tiles per block pair (37 MiB on 148 SMs). Without
    // it (allocation refused) the kernel keeps to whole tiles.
    if (cudaMalloc(&g->partials, PARTIAL_BYTES) == cudaSuccess)
        g->partial_bytes = PARTIAL_BYTES;
    else
        cudaGetLastError();
    return g;
}

extern "C" void cs1_gemm_destroy(void* gemm) {
    Gemm* g = static_cast<Gemm*>(gemm);
    if (!g) return;
    if (g->counters) cudaFree(g->counters);
    if (g->partials) cudaFree(g->partials);
    delete g;
}

extern "C" int cs1_gemm(void* gemm, const void* x, const void* w, void* y, int M, int N, int K, int ldy,
                        void* stream) {
    Gemm* g = static_cast<Gemm*>(gemm);
    if (!g || M < 0 || N <= 0 || K <= 0 || ldy < N) return cudaErrorInvalidValue;
    if (M == 0) return cudaSuccess;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (s1_gemm_tc5_supported(x, w, y, M, N, K, ldy)) {
        const S1GemmScratch scratch = scratch_of(g);
        return s1_gemm_tc5(x, w, y, M, N, K, ldy, &scratch, st);
    }
    return gemm_plain(static_cast<const bf16*>(x), static_cast<const bf16*>(w), nullptr, static_cast<bf16*>(y), M, N, K, ldy, st);
}

// cs1_gemm without the K-split path: every row's sum runs over K in one fixed order, whatever M is.
extern "C" int s1_gemm_unsplit(void* gemm, const void* x, const void* w, void* y, int M, int N, int K, int ldy,
                               void* stream) {
    if (!gemm || M < 0 || N <= 0 || K <= 0 || ldy < N) return cudaErrorInvalidValue;
    if (M == 0) return cudaSuccess;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (s1_gemm_tc5_supported(x, w, y, M, N, K, ldy)) return s1_gemm_tc5(x, w, y, M, N, K, ldy, nullptr, st);
    return gemm_plain(static_cast<const bf16*>(x), static_cast<const bf16*>(w), nullptr, static_cast<bf16*>(y), M, N, K, ldy, st);
}

// 1 if cs1_gemm runs this problem on the tcgen05 kernels, 0 if on the plain kernel.
extern "C" int s1_gemm_engine(void* gemm, const void* x, const void* w, int M, int N, int K) {
    return gemm && s1_gemm_tc5_supported(x, w, nullptr, M, N, K, N) ? 1 : 0;
}

// The MLP's first half as one kernel on the tcgen05 engine: act [M, I] (rows of ld) =
// silu(x w[0:I]^T) * (x w[I:2I]^T), bit-identical to cs1_gemm into a [M, 2 I] buffer followed by
// cs1_silu_mul. Returns CS1_ERR_UNSUPPORTED when the pair kernel cannot take the problem (at most
// 128 rows, K not a multiple of 8); the caller then runs the two operators.
extern "C" int s1_gemm_swiglu(void* gemm, const void* x, const void* w, void* act, int M, int I, int K, int ld,
                              void* stream) {
    if (!gemm || M < 0 || I <= 0 || K <= 0 || ld < I) return cudaErrorInvalidValue;
    if (M == 0) return cudaSuccess;
    if (!s1_gemm_tc5_swiglu_supported(x, w, M, I, K)) return CS1_ERR_UNSUPPORTED;
    return s1_gemm_tc5_swiglu(x, w, act, M, I, K, ld, static_cast<cudaStream_t>(stream));
}

// Engine-pinned entry points for the GEMM benchmark and the parity tests.
extern "C" int s1_gemm_tcgen05(void* gemm, const void* x, const void* w, void* y, int M, int N, int K, int ldy,
                               void* stream) {
    if (M < 0 || N <= 0 || K <= 0 || ldy < N) return cudaErrorInvalidValue;
    if (M == 0) return cudaSuccess;
    if (!s1_gemm_tc5_supported(x, w, y, M, N, K, ldy)) return CS1_ERR_UNSUPPORTED;
    Gemm* g = static_cast<Gemm*>(gemm);  // null: no scratch, so no K split
    if (!g) return s1_gemm_tc5(x, w, y, M, N, K, ldy, nullptr, static_cast<cudaStream_t>(stream));
    const S1GemmScratch scratch = scratch_of(g);
    return s1_gemm_tc5(x, w, y, M, N, K, ldy, &scratch, static_cast<cudaStream_t>(stream));
}

extern "C" int s1_gemm_plain(void* gemm, const void* x, const void* w, void* y, int M, int N, int K, int ldy,
                             void* stream) {
    if (!gemm || M < 0 || N <= 0 || K <= 0 || ldy < N) return cudaErrorInvalidValue;
    if (M == 0) return cudaSuccess;
    return gemm_plain(static_cast<const bf16*>(x), static_cast<const bf16*>(w), nullptr, static_cast<bf16*>(y), M, N, K, ldy,
                      static_cast<cudaStream_t>(stream));
}

// ---- the vision tower's two GEMMs (gemm.cu:137-163 of the reference, library calls there) ----
// y [M, N] = bf16(x w^T + bias): the bias joins the float32 sum before the rounding.
extern "C" int cs1_vision_linear(void* gemm, const void* x, const void* w, const void* bias, void* y, int M, int N, int K,
                                 void* stream) {
    if (!gemm || !bias || !x || !w || !y || M <= 0 || N <= 0 || K <= 0) return cudaErrorInvalidValue;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (s1_gemm_tc5_supported(x, w, y, M, N, K, N)) return s1_gemm_tc5_bias(x, w, bias, y, M, N, K, N, st);
    return gemm_plain(static_cast<const bf16*>(x), static_cast<const bf16*>(w), static_cast<const bf16*>(bias),
                      static_cast<bf16*>(y), M, N, K, N, st);
}

// float32 in, float32 out, float32 arithmetic (unmerged LoRA factors; no TF32).
extern "C" int cs1_gemm_f32(void* gemm, const float* x, const float* w, float* y, int M, int N, int K, void* stream) {
    if (!gemm || !x || !w || !y || M <= 0 || N <= 0 || K <= 0) return cudaErrorInvalidValue;
    return gemm_plain(x, w, static_cast<const bf16*>(nullptr), y, M, N, K, N, static_cast<cudaStream_t>(stream));
}
