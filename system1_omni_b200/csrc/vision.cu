// The vision-tower operators of the C ABI (single image, hidden 1024, 16 heads of 64; reference:
// src/backends/cuda/qwen3_5/ops.h:125-138, vision.cu). bf16 activations; normalisation, rotary
// and LoRA arithmetic in float32 with the reference's rounding points:
//   norm      LayerNorm, eps 1e-6, mean and variance in two passes, y = bf16((x - mean) inv w + b)
//   position  x += bf16(sum_j table[index_j] * weight_j) with separate float32 multiplies and adds
//   rope      q, k = bf16(x cos + (-/+ partner) sin), both products rounded before the add; head dim 64
//   gelu      erf or tanh form, in place;  add / bias / lora_add  one bf16 rounding after a float32 add
//   attention all n keys for every query (no mask but the sequence end), on the tcgen05 kernel
// Elementwise operators move 16 bytes per thread when pointers and sizes allow, else one element.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>

#include "attention_tc5.h"
#include "common.cuh"
#include "cs1_ops.h"

namespace s1 {
namespace {

constexpr int VT = 256;
constexpr int VD = 1024;  // hidden size of the tower: 16 heads of 64
inline unsigned vblocks(size_t n) { return (unsigned)((n + VT - 1) / VT); }

// ---- LayerNorm: one block per row ----
__global__ void __launch_bounds__(VT)
    vision_norm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const bf16* __restrict__ b,
                       bf16* __restrict__ y, int d) {
    __shared__ float scratch[32];
    const size_t off = (size_t)blockIdx.x * d;
    float sum = 0.f;
    for (int i = threadIdx.x; i < d; i += VT) sum += f32(x[off + i]);
    const float mean = block_sum(sum, scratch) / d;
    float var = 0.f;
    for (int i = threadIdx.x; i < d; i += VT) {
        const float a = f32(x[off + i]) - mean;
        var += a * a;
    }
    const float inv = rsqrtf(block_sum(var, scratch) / d + 1e-6f);
    for (int i = threadIdx.x; i < d; i += VT) y[off + i] = to_bf16((f32(x[off + i]) - mean) * inv * f32(w[i]) + f32(b[i]));
}

// The same for rows of 8 * VT elements at most, 16-byte aligned: the row stays in registers.
__global__ void __launch_bounds__(VT)
    vision_norm_packed_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const bf16* __restrict__ b,
                              bf16* __restrict__ y, int d) {
    __shared__ float scratch[32];
    const size_t off = (size_t)blockIdx.x * d;
    const int i0 = threadIdx.x * 8;
    const bool live = i0 < d;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (live) unpack8(ld16_stream(x + off + i0), v);
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < 8; e++) sum += v[e];
    const float mean = block_sum(sum, scratch) / d;
    float var = 0.f;
    if (live) {
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const float a = v[e] - mean;
            var += a * a;
        }
    }
    const float inv = rsqrtf(block_sum(var, scratch) / d + 1e-6f);
    if (live) {
        float wv[8], bv[8];
        unpack8(ld16(w + i0), wv);
        unpack8(ld16(b + i0), bv);
#pragma unroll
        for (int e = 0; e < 8; e++) v[e] = (v[e] - mean) * inv * wv[e] + bv[e];
        st16(y + off + i0, pack8(v));
    }
}

// ---- learned position embedding, bilinear from a 48 x 48 table: 8 channels per thread ----
__global__ void __launch_bounds__(VT)
    vision_position_kernel(bf16* __restrict__ x, const bf16* __restrict__ table, const int* __restrict__ indices,
                           const float* __restrict__ weights, size_t packs) {
    const size_t p = (size_t)blockIdx.x * VT + threadIdx.x;
    if (p >= packs) return;
    const size_t t = p / (VD / 8);
    const int d0 = (int)(p % (VD / 8)) * 8;
    float pos[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        float e[8];
        unpack8(ld16(table + (size_t)indices[t * 4 + j] * VD + d0), e);
        const float wj = weights[t * 4 + j];
#pragma unroll
        for (int c = 0; c < 8; c++) pos[c] = __fadd_rn(pos[c], __fmul_rn(e[c], wj));
    }
    float v[8];
    unpack8(ld16(x + t * VD + d0), v);
#pragma unroll
    for (int c = 0; c < 8; c++) v[c] = v[c] + rbf(pos[c]);
    st16(x + t * VD + d0, pack8(v));
}

// ---- rotary embedding of q and k out of the fused projection [n, 3072]: 8 channels per thread ----
__global__ void __launch_bounds__(VT)
    vision_rope_kernel(const bf16* __restrict__ qkv, const float* __restrict__ co, const float* __restrict__ si,
                       bf16* __restrict__ q, bf16* __restrict__ k, size_t packs) {
    const size_t p = (size_t)blockIdx.x * VT + threadIdx.x;
    if (p >= packs) return;
    const size_t t = p / (VD / 8);
    const int channel = (int)(p % (VD / 8)) * 8, d = channel % 64;
    const int partner = channel + (d < 32 ? 32 : -32);
    const float sign = d < 32 ? -1.f : 1.f;
    float c[8], s[8];
#pragma unroll
    for (int e = 0; e < 8; e++) {
        c[e] = co[t * 32 + d % 32 + e];
        s[e] = si[t * 32 + d % 32 + e];
    }
#pragma unroll
    for (int which = 0; which < 2; which++) {
        const bf16* src = qkv + t * (3 * VD) + which * VD;
        float a[8], b[8], y[8];
        unpack8(ld16(src + channel), a);
        unpack8(ld16(src + partner), b);
#pragma unroll
        for (int e = 0; e < 8; e++) y[e] = __fadd_rn(__fmul_rn(a[e], c[e]), __fmul_rn(sign * b[e], s[e]));
        st16((which == 0 ? q : k) + t * VD + channel, pack8(y));
    }
}

// ---- elementwise maps: F(bf16 value as float, element index) -> float, rounded once ----
template <typename F>
__global__ void __launch_bounds__(VT) map_packed_kernel(bf16* __restrict__ x, size_t packs, F f) {
    const size_t p = (size_t)blockIdx.x * VT + threadIdx.x;
    if (p >= packs) return;
    float v[8];
    unpack8(ld16(x + p * 8), v);
#pragma unroll
    for (int e = 0; e < 8; e++) v[e] = f(v[e], p * 8 + e);
    st16(x + p * 8, pack8(v));
}
template <typename F>
__global__ void __launch_bounds__(VT) map_scalar_kernel(bf16* __restrict__ x, size_t n, F f) {
    const size_t i = (size_t)blockIdx.x * VT + threadIdx.x;
    if (i < n) x[i] = to_bf16(f(f32(x[i]), i));
}
template <typename F>
int map_in_place(void* x, size_t n, bool packed_ok, void* stream, F f) {
    if (n == 0) return cudaSuccess;
    if (!x) return cudaErrorInvalidValue;
    if (packed_ok && n % 8 == 0 && aligned16(x))
        map_packed_kernel<<<vblocks(n / 8), VT, 0, as_stream(stream)>>>(static_cast<bf16*>(x), n / 8, f);
    else
        map_scalar_kernel<<<vblocks(n), VT, 0, as_stream(stream)>>>(static_cast<bf16*>(x), n, f);
    return cudaGetLastError();
}

__global__ void __launch_bounds__(VT) to_float_kernel(const bf16* __restrict__ x, float* __restrict__ out, size_t n) {
    const size_t i = (size_t)blockIdx.x * VT + threadIdx.x;
    if (i < n) out[i] = f32(x[i]);
}

}  // namespace
}  // namespace s1

using namespace s1;

extern "C" {

int cs1_vision_norm(const void* x, const void* w, const void* b, void* y, int rows, int d, void* stream) {
    if (rows <= 0 || d <= 0 || !x || !w || !b || !y) return cudaErrorInvalidValue;
    const bf16 *xp = static_cast<const bf16*>(x), *wp = static_cast<const bf16*>(w), *bp = static_cast<const bf16*>(b);
    if (d % 8 == 0 && d <= 8 * VT && aligned16(x) && aligned16(w) && aligned16(b) && aligned16(y))
        vision_norm_packed_kernel<<<rows, VT, 0, as_stream(stream)>>>(xp, wp, bp, static_cast<bf16*>(y), d);
    else
        vision_norm_kernel<<<rows, VT, 0, as_stream(stream)>>>(xp, wp, bp, static_cast<bf16*>(y), d);
    return cudaGetLastError();
}

int cs1_vision_position(void* x, const void* table, const int* indices, const float* weights, int n, void* stream) {
    if (n <= 0 || !x || !table || !indices || !weights || !aligned16(x) || !aligned16(table)) return cudaErrorInvalidValue;
    const size_t packs = (size_t)n * (VD / 8);
    vision_position_kernel<<<vblocks(packs), VT, 0, as_stream(stream)>>>(static_cast<bf16*>(x),
                                                                        static_cast<const bf16*>(table), indices, weights,
                                                                        packs);
    return cudaGetLastError();
}

int cs1_vision_rope(const void* qkv, const float* co, const float* si, void* q, void* k, int n, void* stream) {
    if (n <= 0 || !qkv || !co || !si || !q || !k || !aligned16(qkv) || !aligned16(q) || !aligned16(k))
        return cudaErrorInvalidValue;
    const size_t packs = (size_t)n * (VD / 8);
    vision_rope_kernel<<<vblocks(packs), VT, 0, as_stream(stream)>>>(static_cast<const bf16*>(qkv), co, si,
                                                                    static_cast<bf16*>(q), static_cast<bf16*>(k), packs);
    return cudaGetLastError();
}

// q, k [n, 1024]; v is a slice of the fused projection, rows 3072 elements apart (vision.cu:229-235).
int cs1_vision_attention(const void* q, const void* k, const void* v, void* out, int n, void* stream) {
    if (n <= 0 || !q || !k || !v || !out || !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out))
        return cudaErrorInvalidValue;
    return s1_attn_tc5_full64(static_cast<const bf16*>(q), static_cast<const bf16*>(k), static_cast<const bf16*>(v), 3 * VD,
                              static_cast<bf16*>(out), n, 16, 0.125f, as_stream(stream));
}

int cs1_vision_bias(void* x, const void* bias, size_t n, int d, void* stream) {
    if (d <= 0) return cudaErrorInvalidValue;
    if (n == 0) return cudaSuccess;
    if (!bias) return cudaErrorInvalidValue;
    const bf16* bp = static_cast<const bf16*>(bias);
    return map_in_place(x, n, true, stream, [bp, d] __device__(float a, size_t i) { return a + f32(bp[i % d]); });
}

int cs1_vision_gelu(void* x, size_t n, int exact, void* stream) {
    if (exact)
        return map_in_place(x, n, true, stream,
                            [] __device__(float a, size_t) { return 0.5f * a * (1.f + erff(a * 0.7071067811865475244f)); });
    return map_in_place(x, n, true, stream, [] __device__(float a, size_t) {
        return 0.5f * a * (1.f + tanhf(0.7978845608028654f * (a + 0.044715f * a * a * a)));
    });
}

int cs1_vision_add(void* x, const void* delta, size_t n, void* stream) {
    if (n == 0) return cudaSuccess;
    if (!delta) return cudaErrorInvalidValue;
    const bf16* dp = static_cast<const bf16*>(delta);
    return map_in_place(x, n, true, stream, [dp] __device__(float a, size_t i) { return a + f32(dp[i]); });
}

int cs1_vision_to_float(const void* x, float* out, size_t n, void* stream) {
    if (n == 0) return cudaSuccess;
    if (!x || !out) return cudaErrorInvalidValue;
    to_float_kernel<<<vblocks(n), VT, 0, as_stream(stream)>>>(static_cast<const bf16*>(x), out, n);
    return cudaGetLastError();
}

int cs1_vision_lora_add(void* x, const float* delta, size_t n, float scale, void* stream) {
    if (n == 0) return cudaSuccess;
    if (!delta) return cudaErrorInvalidValue;
    return map_in_place(x, n, true, stream,
                        [delta, scale] __device__(float a, size_t i) { return __fadd_rn(a, __fmul_rn(scale, delta[i])); });
}

}  // extern "C"
