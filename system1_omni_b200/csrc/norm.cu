// RMSNorm variants: zero-centred RMSNorm, residual add fused with it, and the gated RMSNorm
// of the Gated DeltaNet output. One block per row with the row held in registers between
// the reduction and the scaling (each element is read from HBM once), 16-byte accesses,
// shuffle reductions; element-wise fallbacks cover odd widths and 2-byte-aligned pointers.
//
// Rounding follows src/backends/cuda/qwen3_5/norm.cu:10-99 of the reference.
#include "common.cuh"
#include "cs1_ops.h"

namespace s1 {
namespace {

constexpr int NORM_THREADS = 256;
constexpr int MAX_PACKS = 4;  // packs of 8 per thread held in registers: D <= 8192

// ADD: residual += delta first (rounded to bf16 and stored back).
template <bool ADD, int PACKS>
__global__ void __launch_bounds__(NORM_THREADS)
    rms_norm_packed_kernel(bf16* __restrict__ residual, const bf16* __restrict__ delta, const bf16* __restrict__ w,
                           bf16* __restrict__ out, int D, float eps) {
    __shared__ float scratch[32];
    grid_dep_trigger();
    grid_dep_sync();
    const size_t row = (size_t)blockIdx.x * D;
    const int packs = D / 8;
    float v[PACKS][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PACKS; i++) {
        const int p = threadIdx.x + i * NORM_THREADS;
        if (p < packs) {
            unpack8(ld16(residual + row + (size_t)p * 8), v[i]);
            if (ADD) {
                float d[8];
                unpack8(ld16_stream(delta + row + (size_t)p * 8), d);
#pragma unroll
                for (int e = 0; e < 8; e++) v[i][e] = v[i][e] + d[e];
                const uint4 r = pack8(v[i]);
                st16(residual + row + (size_t)p * 8, r);
                unpack8(r, v[i]);
            }
#pragma unroll
            for (int e = 0; e < 8; e++) ss += v[i][e] * v[i][e];
        }
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / D + eps);
#pragma unroll
    for (int i = 0; i < PACKS; i++) {
        const int p = threadIdx.x + i * NORM_THREADS;
        if (p < packs) {
            float wv[8];
            unpack8(ld16(w + (size_t)p * 8), wv);
#pragma unroll
            for (int e = 0; e < 8; e++) v[i][e] = v[i][e] * inv * (1.f + wv[e]);
            st16(out + row + (size_t)p * 8, pack8(v[i]));
        }
    }
}

template <bool ADD>
__global__ void __launch_bounds__(NORM_THREADS)
    rms_norm_scalar_kernel(bf16* __restrict__ residual, const bf16* __restrict__ delta, const bf16* __restrict__ w,
                           bf16* __restrict__ out, int D, float eps) {
    __shared__ float scratch[32];
    const size_t row = (size_t)blockIdx.x * D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float r = f32(residual[row + i]);
        if (ADD) {
            const bf16 rb = to_bf16(r + f32(delta[row + i]));
            residual[row + i] = rb;
            r = f32(rb);
        }
        ss += r * r;
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / D + eps);
    // each thread rereads only the elements it wrote
    for (int i = threadIdx.x; i < D; i += blockDim.x)
        out[row + i] = to_bf16(f32(residual[row + i]) * inv * (1.f + f32(w[i])));
}

template <bool ADD>
int launch_norm(void* residual, const void* delta, const void* w, void* out, int rows, int D, float eps,
                void* stream) {
    if (rows < 0 || D <= 0) return cudaErrorInvalidValue;
    if (rows == 0) return cudaSuccess;
    bf16* r = static_cast<bf16*>(residual);
    const bf16* d = static_cast<const bf16*>(delta);
    const bf16* wp = static_cast<const bf16*>(w);
    bf16* o = static_cast<bf16*>(out);
    const cudaStream_t st = as_stream(stream);
    const bool packed = D % 8 == 0 && D <= 8 * NORM_THREADS * MAX_PACKS && aligned16(residual) && aligned16(w) &&
                        aligned16(out) && (!ADD || aligned16(delta));
    if (packed) {
        const int per = (D / 8 + NORM_THREADS - 1) / NORM_THREADS;
        switch (per) {
            case 1: launch_dep_family(DEP_NORM, rms_norm_packed_kernel<ADD, 1>, rows, NORM_THREADS, 0, st, r, d, wp, o, D, eps); break;
            case 2: launch_dep_family(DEP_NORM, rms_norm_packed_kernel<ADD, 2>, rows, NORM_THREADS, 0, st, r, d, wp, o, D, eps); break;
            case 3: launch_dep_family(DEP_NORM, rms_norm_packed_kernel<ADD, 3>, rows, NORM_THREADS, 0, st, r, d, wp, o, D, eps); break;
            default: launch_dep_family(DEP_NORM, rms_norm_packed_kernel<ADD, 4>, rows, NORM_THREADS, 0, st, r, d, wp, o, D, eps); break;
        }
    } else {
        rms_norm_scalar_kernel<ADD><<<rows, NORM_THREADS, 0, st>>>(r, d, wp, o, D, eps);
    }
    return cudaGetLastError();
}

// Gated RMSNorm, D = 128: 16 lanes per (token, head) row, 8 values per lane.
// Each lane group takes GN_ROWS_PER_GROUP rows 16 apart and requests all of them before
// reducing, to keep eight 16-byte loads in flight per thread.
constexpr int GN_GROUPS = 16, GN_ROWS_PER_GROUP = 4;
constexpr int GN_ROWS_PER_BLOCK = GN_GROUPS * GN_ROWS_PER_GROUP;

__global__ void __launch_bounds__(GN_GROUPS * 16)
    gated_rms_norm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ z, int ldz, const bf16* __restrict__ w,
                          bf16* __restrict__ out, int rows, int H, float eps) {
    constexpr int D = 128;
    grid_dep_trigger();
    grid_dep_sync();
    const int group = threadIdx.x / 16, sub = threadIdx.x & 15;
    uint4 xv[GN_ROWS_PER_GROUP], zv[GN_ROWS_PER_GROUP];
    size_t base[GN_ROWS_PER_GROUP];
    bool live[GN_ROWS_PER_GROUP];
#pragma unroll
    for (int r = 0; r < GN_ROWS_PER_GROUP; r++) {
        const int row = blockIdx.x * GN_ROWS_PER_BLOCK + r * GN_GROUPS + group;
        live[r] = row < rows;
        const int rr = live[r] ? row : rows - 1;
        base[r] = (size_t)rr * D + sub * 8;
        xv[r] = ld16_stream(x + base[r]);
        zv[r] = ld16_stream(z + (size_t)(rr / H) * ldz + (size_t)(rr % H) * D + sub * 8);
    }
    float wv[8];
    unpack8(ld16(w + sub * 8), wv);
#pragma unroll
    for (int r = 0; r < GN_ROWS_PER_GROUP; r++) {
        float v[8], g[8];
        unpack8(xv[r], v);
        unpack8(zv[r], g);
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; e++) ss += v[e] * v[e];
        const float inv = rsqrtf(warp_sum<16>(ss) / D + eps);
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const float normed = rbf(v[e] * inv);
            const float scaled = rbf(wv[e] * normed);
            v[e] = scaled * silu_fast(g[e]);
        }
        if (live[r]) st16(out + base[r], pack8(v));
    }
}

__global__ void gated_rms_norm_scalar_kernel(const bf16* __restrict__ x, const bf16* __restrict__ z, int ldz,
                                             const bf16* __restrict__ w, bf16* __restrict__ out, int rows, int H,
                                             float eps) {
    constexpr int D = 128, PER = D / 32;
    const int row = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32, lane = threadIdx.x & 31;
    if (row >= rows) return;
    const size_t base = (size_t)row * D + lane * PER;
    const size_t zbase = (size_t)(row / H) * ldz + (size_t)(row % H) * D + lane * PER;
    float v[PER];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PER; i++) {
        v[i] = f32(x[base + i]);
        ss += v[i] * v[i];
    }
    const float inv = rsqrtf(warp_sum(ss) / D + eps);
#pragma unroll
    for (int i = 0; i < PER; i++) {
        const float normed = rbf(v[i] * inv);
        const float scaled = rbf(f32(w[lane * PER + i]) * normed);
        out[base + i] = to_bf16(scaled * silu_fast(f32(z[zbase + i])));
    }
}

}  // namespace
}  // namespace s1

using namespace s1;

extern "C" int cs1_rms_norm(const void* x, const void* w, void* out, int rows, int D, float eps, void* stream) {
    // the input is only read when ADD is false
    return launch_norm<false>(const_cast<void*>(x), nullptr, w, out, rows, D, eps, stream);
}

extern "C" int cs1_add_rms_norm(void* residual, const void* delta, const void* w, void* out, int rows, int D,
                                float eps, void* stream) {
    return launch_norm<true>(residual, delta, w, out, rows, D, eps, stream);
}

extern "C" int cs1_gated_rms_norm(const void* x, const void* z, int ldz, const void* w, void* out, int T, int H,
                                  int D, float eps, void* stream) {
    if (D != 128 || T < 0 || H < 0 || ldz < H * D) return cudaErrorInvalidValue;
    const long long rows = (long long)T * H;
    if (rows <= 0) return cudaSuccess;
    if (rows > 0x7fffffffLL) return cudaErrorInvalidValue;
    const bf16 *xp = static_cast<const bf16*>(x), *zp = static_cast<const bf16*>(z), *wp = static_cast<const bf16*>(w);
    if (ldz % 8 == 0 && aligned16(x) && aligned16(z) && aligned16(w) && aligned16(out)) {
        launch_dep_family(DEP_NORM, gated_rms_norm_kernel, (unsigned)((rows + GN_ROWS_PER_BLOCK - 1) / GN_ROWS_PER_BLOCK), GN_GROUPS * 16, 0,
                   as_stream(stream), xp, zp, ldz, wp, static_cast<bf16*>(out), (int)rows, H, eps);
    } else {
        gated_rms_norm_scalar_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, as_stream(stream)>>>(
            xp, zp, ldz, wp, static_cast<bf16*>(out), (int)rows, H, eps);
    }
    return cudaGetLastError();
}

// ---- per-head L2 norm, head dim 128 (the q / k normalisation of the delta rule as an operator of
// its own: inside cs1_gdn_prefill it is part of the chunk kernel, gdn_prefill.cu:170-203 of the
// reference; here it exists for the elementwise benchmark sweep and for checks) ----
namespace s1 {
namespace {
__global__ void __launch_bounds__(GN_GROUPS * 16)
    l2norm_heads_kernel(const bf16* __restrict__ x, bf16* __restrict__ out, int rows, float scale) {
    constexpr int D = 128;
    const int group = threadIdx.x / 16, sub = threadIdx.x & 15;
    uint4 xv[GN_ROWS_PER_GROUP];
    size_t base[GN_ROWS_PER_GROUP];
    bool live[GN_ROWS_PER_GROUP];
#pragma unroll
    for (int r = 0; r < GN_ROWS_PER_GROUP; r++) {
        const int row = blockIdx.x * GN_ROWS_PER_BLOCK + r * GN_GROUPS + group;
        live[r] = row < rows;
        base[r] = (size_t)(live[r] ? row : rows - 1) * D + sub * 8;
        xv[r] = ld16_stream(x + base[r]);
    }
#pragma unroll
    for (int r = 0; r < GN_ROWS_PER_GROUP; r++) {
        float v[8];
        unpack8(xv[r], v);
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; e++) ss += v[e] * v[e];
        const float inv = rsqrtf(warp_sum<16>(ss) + 1e-6f) * scale;
#pragma unroll
        for (int e = 0; e < 8; e++) v[e] *= inv;
        if (live[r]) st16(out + base[r], pack8(v));
    }
}
}  // namespace
}  // namespace s1

// out = bf16(x * rsqrt(sum x^2 + 1e-6) * scale) over rows of 128; x and out 16-byte aligned.
extern "C" int s1_l2norm_heads(const void* x, void* out, long long rows, float scale, void* stream) {
    if (rows < 0 || rows > 0x7fffffffLL) return cudaErrorInvalidValue;
    if (rows == 0) return cudaSuccess;
    if (!x || !out || !s1::aligned16(x) || !s1::aligned16(out)) return cudaErrorInvalidValue;
    s1::l2norm_heads_kernel<<<(unsigned)((rows + s1::GN_ROWS_PER_BLOCK - 1) / s1::GN_ROWS_PER_BLOCK), s1::GN_GROUPS * 16, 0,
                              s1::as_stream(stream)>>>(static_cast<const s1::bf16*>(x), static_cast<s1::bf16*>(out), (int)rows,
                                                       scale);
    return cudaGetLastError();
}
