// Small device helpers of the host executor: the seeded generator for synthetic weights
// and the gather of each prompt's last-token row.
#include "common.cuh"
#include "exec_kernels.h"

namespace s1 {
namespace {

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
    x += 0x9e3779b97f4a7c15ull;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
    return x ^ (x >> 31);
}

// kind 0: mean + std * N(0,1) by Box-Muller; kind 1: uniform in [mean, mean + std).
__global__ void fill_kernel(bf16* out, size_t n, uint64_t seed, float mean, float std, int kind) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t r = splitmix64(seed ^ (i * 0xd1342543de82ef95ull));
    const float u1 = ((float)(r >> 40) + 0.5f) * (1.0f / 16777216.0f);
    const float u2 = ((float)((r >> 16) & 0xffffff) + 0.5f) * (1.0f / 16777216.0f);
    float v;
    if (kind == 0)
        v = mean + std * sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
    else
        v = mean + std * u1;
    out[i] = to_bf16(v);
}

__global__ void gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ ends, uint4* __restrict__ out,
                                   int packs) {
    grid_dep_trigger();
    grid_dep_sync();
    const size_t src = (size_t)(ends[blockIdx.x] - 1) * packs;
    const size_t dst = (size_t)blockIdx.x * packs;
    for (int i = threadIdx.x; i < packs; i += blockDim.x) out[dst + i] = x[src + i];
}

}  // namespace

int fill_bf16(void* out, size_t n, uint64_t seed, float mean, float std, int kind, cudaStream_t st) {
    if (n == 0) return 0;
    fill_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(static_cast<bf16*>(out), n, seed, mean, std, kind);
    return cudaGetLastError();
}

int gather_rows(const void* x, const int* ends_device, void* out, int nseq, int D, cudaStream_t st) {
    if (nseq == 0) return 0;
    gather_rows_kernel<<<nseq, 128, 0, st>>>(static_cast<const uint4*>(x), ends_device, static_cast<uint4*>(out),
                                             D / 8);
    return cudaGetLastError();
}

}  // namespace s1
