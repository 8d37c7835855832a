// Small device helpers of the host executor: the seeded generator for synthetic weights
// and the gather of each prompt's last-token row.
#include "common.cuh"
#include "exec_kernels.h"
#include "s1_executor.h"
#include "status.h"

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

struct SpreadRows {
    int row0[16];
};
__global__ void spread_block_kernel(uint4* __restrict__ dst, size_t row_packs, const __grid_constant__ SpreadRows rows,
                                    const uint4* __restrict__ src, size_t packs) {
    grid_dep_trigger();
    grid_dep_sync();
    uint4* out = dst + (size_t)rows.row0[blockIdx.y] * row_packs;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < packs; i += (size_t)gridDim.x * blockDim.x) out[i] = src[i];
}

__global__ void collect_status_kernel(const int* a, const int* b, const int* c, int* out) {
    out[0] = *a;
    out[1] = *b;
    out[2] = *c;
}

}  // namespace

int collect_status(int* out3_device, cudaStream_t st) {
    int *a = nullptr, *b = nullptr, *c = nullptr;
    cudaError_t e;
    if ((e = (cudaError_t)gemm_error_address(&a)) != cudaSuccess) return e;
    if ((e = (cudaError_t)attn_error_address(&b)) != cudaSuccess) return e;
    if ((e = (cudaError_t)gdn_error_address(&c)) != cudaSuccess) return e;
    collect_status_kernel<<<1, 1, 0, st>>>(a, b, c, out3_device);
    return cudaGetLastError();
}

int clear_status() {
    int* p[3] = {};
    cudaError_t e;
    if ((e = (cudaError_t)gemm_error_address(&p[0])) != cudaSuccess) return e;
    if ((e = (cudaError_t)attn_error_address(&p[1])) != cudaSuccess) return e;
    if ((e = (cudaError_t)gdn_error_address(&p[2])) != cudaSuccess) return e;
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) return e;
    for (int i = 0; i < 3; i++)
        if ((e = cudaMemset(p[i], 0, sizeof(int))) != cudaSuccess) return e;
    return cudaSuccess;
}

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

int spread_block(void* dst, size_t row_packs, const int* row0, int n, const void* src, size_t packs, cudaStream_t st) {
    if (n <= 0 || n > 16 || packs == 0) return n == 0 || packs == 0 ? 0 : (int)cudaErrorInvalidValue;
    SpreadRows rows{};
    for (int i = 0; i < n; i++) rows.row0[i] = row0[i];
    const unsigned bx = (unsigned)std::min<size_t>((packs + 255) / 256, 64);
    spread_block_kernel<<<dim3(bx, n), 256, 0, st>>>(static_cast<uint4*>(dst), row_packs, rows, static_cast<const uint4*>(src), packs);
    return cudaGetLastError();
}

}  // namespace s1

// The three device error words of the current device after waiting for all queued work
// (0 = no bounded wait gave up), cleared when any is set. Every out pointer is nullable.
extern "C" int s1_device_status(int* gemm, int* attention, int* gdn) {
    int* p[3] = {};
    cudaError_t e;
    if ((e = (cudaError_t)s1::gemm_error_address(&p[0])) != cudaSuccess) return e;
    if ((e = (cudaError_t)s1::attn_error_address(&p[1])) != cudaSuccess) return e;
    if ((e = (cudaError_t)s1::gdn_error_address(&p[2])) != cudaSuccess) return e;
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) return e;
    int v[3] = {};
    for (int i = 0; i < 3; i++)
        if ((e = cudaMemcpy(&v[i], p[i], sizeof(int), cudaMemcpyDeviceToHost)) != cudaSuccess) return e;
    if (v[0] | v[1] | v[2]) {
        const int rc = s1::clear_status();
        if (rc != 0) return rc;
    }
    if (gemm) *gemm = v[0];
    if (attention) *attention = v[1];
    if (gdn) *gdn = v[2];
    return 0;
}
