// HBM-bound sidecars of the Gated DeltaNet and MLP blocks: embedding gather, causal
// depthwise conv1d + SiLU + q/k/v split, beta / log-decay gates, sigmoid gate, SiLU * up.
// All of them move 16 bytes per access when pointers and widths allow it and fall back to
// element-wise kernels otherwise (callers may pass 2-byte-aligned pointers).
//
// Rounding follows the reference kernels (src/backends/cuda/qwen3_5/elementwise.cu:11-87):
// every place the model stores a bf16 tensor is a round-to-nearest-even here.
#include "common.cuh"
#include "cs1_ops.h"

namespace s1 {
namespace {

constexpr int THREADS = 256;

inline unsigned blocks_for(size_t n, int per = THREADS) { return (unsigned)((n + per - 1) / per); }

// ---- embedding ----
__global__ void __launch_bounds__(128) embed_kernel(const int32_t* __restrict__ ids, const uint4* __restrict__ table,
                                                    uint4* __restrict__ out, int packs) {
    grid_dep_trigger();
    grid_dep_sync();
    const size_t t = blockIdx.x;
    const size_t id = (size_t)ids[t];
    const uint4* src = table + id * packs;
    uint4* dst = out + t * packs;
    for (int i = threadIdx.x; i < packs; i += blockDim.x) dst[i] = src[i];
}

// ---- causal depthwise conv (kernel 4) + SiLU + split ----
// One thread owns 8 adjacent channels and walks TT consecutive tokens with the three
// previous rows held in registers, so each input row is fetched once per token block
// (plus a 3-row halo) instead of four times.
constexpr int CONV_TT = 16;     // tokens per thread for long inputs
constexpr int CONV_TT_SHORT = 8; // up to CONV_SHORT_TOKENS tokens: twice the blocks, so that loads and arithmetic of different warps overlap
constexpr int CONV_SHORT_TOKENS = 2048;
constexpr int CONV_THREADS = 128;

template <int CONV_TT>
__device__ __forceinline__ void conv_block(const bf16* __restrict__ qkv, int ld, const bf16* __restrict__ w,
                                           bf16* __restrict__ q, bf16* __restrict__ k, bf16* __restrict__ v, int T,
                                           int key_dim, int value_dim) {
    const int packs = (2 * key_dim + value_dim) / 8;
    const int p = blockIdx.y * CONV_THREADS + threadIdx.x;
    if (p >= packs) return;
    const int c0 = p * 8;
    const int t0 = blockIdx.x * CONV_TT;

    // w is [channels][4]: 32 consecutive values for these 8 channels.
    float wf[8][4];
    {
        const uint4* wp = reinterpret_cast<const uint4*>(w + (size_t)c0 * 4);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float tmp[8];
            unpack8(wp[i], tmp);
#pragma unroll
            for (int e = 0; e < 8; e++) wf[(i * 8 + e) / 4][(i * 8 + e) % 4] = tmp[e];
        }
    }
    bf16* dst;
    int dld, dc;
    if (c0 < key_dim) {
        dst = q, dld = key_dim, dc = c0;
    } else if (c0 < 2 * key_dim) {
        dst = k, dld = key_dim, dc = c0 - key_dim;
    } else {
        dst = v, dld = value_dim, dc = c0 - 2 * key_dim;
    }

    // All rows of the block (and the 3-row halo) are requested before any arithmetic, so a
    // thread keeps 19 independent 16-byte loads in flight instead of one.
    uint4 rows[CONV_TT + 3];
#pragma unroll
    for (int i = 0; i < CONV_TT + 3; i++) {
        const int t = t0 - 3 + i;
        rows[i] = (t >= 0 && t < T) ? ld16_stream(qkv + (size_t)t * ld + c0) : make_uint4(0, 0, 0, 0);
    }
    float x0[8], x1[8], x2[8], x3[8];
    unpack8(rows[0], x0);
    unpack8(rows[1], x1);
    unpack8(rows[2], x2);
#pragma unroll
    for (int i = 0; i < CONV_TT; i++) {
        const int t = t0 + i;
        if (t >= T) break;
        unpack8(rows[i + 3], x3);
        float y[8];
#pragma unroll
        for (int e = 0; e < 8; e++) {
            // taps in order t-3 .. t; a missing tap contributes an exact zero
            float acc = fmaf(wf[e][0], x0[e], 0.f);
            acc = fmaf(wf[e][1], x1[e], acc);
            acc = fmaf(wf[e][2], x2[e], acc);
            acc = fmaf(wf[e][3], x3[e], acc);
            y[e] = silu_fast(rbf(acc));
        }
        st16(dst + (size_t)t * dld + dc, pack8(y));
#pragma unroll
        for (int e = 0; e < 8; e++) {
            x0[e] = x1[e];
            x1[e] = x2[e];
            x2[e] = x3[e];
        }
    }
}

template <int TT>
__global__ void __launch_bounds__(CONV_THREADS)
    gdn_conv_packed_kernel(const bf16* __restrict__ qkv, int ld, const bf16* __restrict__ w, bf16* __restrict__ q,
                           bf16* __restrict__ k, bf16* __restrict__ v, int T, int key_dim, int value_dim) {
    grid_dep_trigger();
    grid_dep_sync();
    conv_block<TT>(qkv, ld, w, q, k, v, T, key_dim, value_dim);
}

__global__ void gdn_conv_scalar_kernel(const bf16* __restrict__ qkv, int ld, const bf16* __restrict__ w,
                                       bf16* __restrict__ q, bf16* __restrict__ k, bf16* __restrict__ v, int T,
                                       int key_dim, int value_dim) {
    const int channels = 2 * key_dim + value_dim;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)T * channels) return;
    const int t = idx / channels, c = idx % channels;
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int s = t - 3 + j;
        if (s >= 0) acc = fmaf(f32(w[c * 4 + j]), f32(qkv[(size_t)s * ld + c]), acc);
    }
    const bf16 y = to_bf16(silu_fast(rbf(acc)));
    if (c < key_dim)
        q[(size_t)t * key_dim + c] = y;
    else if (c < 2 * key_dim)
        k[(size_t)t * key_dim + c - key_dim] = y;
    else
        v[(size_t)t * value_dim + c - 2 * key_dim] = y;
}

// ---- gates ----
__device__ __forceinline__ void gate_element(const bf16* __restrict__ b, const bf16* __restrict__ a, int ld,
                                             const bf16* __restrict__ A_log, const bf16* __restrict__ dt_bias,
                                             bf16* __restrict__ beta, float* __restrict__ g, int i, int H) {
    const int h = i % H;
    const size_t src = (size_t)(i / H) * ld + h;
    beta[i] = to_bf16(sigmoid(f32(b[src])));
    const float x = f32(a[src]) + f32(dt_bias[h]);
    const float sp = x > 20.f ? x : log1pf(expf(x));
    g[i] = -expf(f32(A_log[h])) * sp;
}

__global__ void gdn_gates_kernel(const bf16* __restrict__ b, const bf16* __restrict__ a, int ld,
                                 const bf16* __restrict__ A_log, const bf16* __restrict__ dt_bias,
                                 bf16* __restrict__ beta, float* __restrict__ g, int n, int H) {
    grid_dep_trigger();
    grid_dep_sync();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    gate_element(b, a, ld, A_log, dt_bias, beta, g, i, H);
}

// The convolution and the gates of one token range in one launch: both read the rows the input
// projection wrote. Blocks with blockIdx.y below conv_blocks are convolution blocks, the row of
// blocks after them computes the gates of the same CONV_TT tokens. Same arithmetic per element as
// the two kernels above.
template <int TT>
__global__ void __launch_bounds__(CONV_THREADS)
    gdn_conv_gates_kernel(const bf16* __restrict__ qkv, int ld, const bf16* __restrict__ w, bf16* __restrict__ q,
                          bf16* __restrict__ k, bf16* __restrict__ v, int T, int key_dim, int value_dim, int conv_blocks,
                          const bf16* __restrict__ b, const bf16* __restrict__ a, const bf16* __restrict__ A_log,
                          const bf16* __restrict__ dt_bias, bf16* __restrict__ beta, float* __restrict__ g, int H) {
    grid_dep_trigger();
    grid_dep_sync();
    if ((int)blockIdx.y < conv_blocks) {
        conv_block<TT>(qkv, ld, w, q, k, v, T, key_dim, value_dim);
        return;
    }
    const int first = blockIdx.x * TT * H;
    const int end = min((int)(blockIdx.x + 1) * TT, T) * H;
    for (int i = first + (int)threadIdx.x; i < end; i += CONV_THREADS) gate_element(b, a, ld, A_log, dt_bias, beta, g, i, H);
}

// The same for the sequences of a pack (blockIdx.z): sequence i is rows [row0[i], row0[i] + len[i])
// of every operand; the convolution of a sequence's first rows sees zeros before it, not the
// sequence packed in front of it.
struct ConvSeqs {
    int row0[16], len[16];
};
template <int TT>
__global__ void __launch_bounds__(CONV_THREADS)
    gdn_conv_gates_batch_kernel(const bf16* __restrict__ qkv, int ld, const bf16* __restrict__ w, bf16* __restrict__ q,
                                bf16* __restrict__ k, bf16* __restrict__ v, const __grid_constant__ ConvSeqs seqs, int key_dim,
                                int value_dim, int conv_blocks, const bf16* __restrict__ b, const bf16* __restrict__ a,
                                const bf16* __restrict__ A_log, const bf16* __restrict__ dt_bias, bf16* __restrict__ beta,
                                float* __restrict__ g, int H) {
    grid_dep_trigger();
    const int T = seqs.len[blockIdx.z];
    if ((int)blockIdx.x * TT >= T) return;
    const size_t r = (size_t)seqs.row0[blockIdx.z];
    grid_dep_sync();
    if ((int)blockIdx.y < conv_blocks) {
        conv_block<TT>(qkv + r * ld, ld, w, q + r * key_dim, k + r * key_dim, v + r * value_dim, T, key_dim, value_dim);
        return;
    }
    const int first = blockIdx.x * TT * H;
    const int end = min((int)(blockIdx.x + 1) * TT, T) * H;
    for (int i = first + (int)threadIdx.x; i < end; i += CONV_THREADS)
        gate_element(b + r * ld, a + r * ld, ld, A_log, dt_bias, beta + r * H, g + r * H, i, H);
}

// ---- x * sigmoid(gate) ----
__global__ void sigmoid_gate_kernel(bf16* __restrict__ x, const bf16* __restrict__ gate, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    x[i] = to_bf16(f32(x[i]) * rbf(sigmoid(f32(gate[i]))));
}

__global__ void sigmoid_gate_packed_kernel(uint4* __restrict__ x, const uint4* __restrict__ gate, size_t packs) {
    grid_dep_trigger();
    grid_dep_sync();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= packs) return;
    float xv[8], gv[8];
    unpack8(x[i], xv);
    unpack8(ld16_stream(gate + i), gv);
#pragma unroll
    for (int e = 0; e < 8; e++) xv[e] = xv[e] * rbf(sigmoid(gv[e]));
    x[i] = pack8(xv);
}

// ---- SwiGLU activation ----
__global__ void silu_mul_kernel(const bf16* __restrict__ gate_up, int ld, bf16* __restrict__ out, int I, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / I, j = i % I;
    const bf16* row = gate_up + t * ld;
    out[i] = to_bf16(rbf(silu_fast(f32(row[j]))) * f32(row[I + j]));
}

// Two packs per thread keep more loads in flight per warp.
__global__ void __launch_bounds__(THREADS)
    silu_mul_packed_kernel(const uint4* __restrict__ gate_up, int ld, uint4* __restrict__ out, int I, size_t n) {
    grid_dep_trigger();
    grid_dep_sync();
    const size_t base = ((size_t)blockIdx.x * blockDim.x) * 2 + threadIdx.x;
    uint4 g[2], u[2];
    size_t idx[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        idx[r] = base + (size_t)r * THREADS;
        if (idx[r] < n) {
            const size_t t = idx[r] / I, j = idx[r] % I;
            const uint4* row = gate_up + t * ld;
            g[r] = ld16_stream(row + j);
            u[r] = ld16_stream(row + I + j);
        }
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
        if (idx[r] < n) {
            float gv[8], uv[8];
            unpack8(g[r], gv);
            unpack8(u[r], uv);
#pragma unroll
            for (int e = 0; e < 8; e++) gv[e] = rbf(silu_fast(gv[e])) * uv[e];
            out[idx[r]] = pack8(gv);
        }
    }
}

}  // namespace
}  // namespace s1

using namespace s1;

extern "C" int cs1_embed(const int32_t* ids, const void* table, void* out, int T, int D, void* stream) {
    if (D % 8 != 0 || D <= 0) return cudaErrorInvalidValue;
    if (T <= 0) return cudaSuccess;
    if (!aligned16(table) || !aligned16(out)) return cudaErrorInvalidValue;
    launch_dep(embed_kernel, T, 128, 0, as_stream(stream), ids, static_cast<const uint4*>(table), static_cast<uint4*>(out),
               D / 8);
    return cudaGetLastError();
}

extern "C" int cs1_gdn_conv(const void* qkv, int ld, const void* w, void* q, void* k, void* v, int T, int key_dim,
                            int value_dim, void* stream) {
    if (T < 0 || key_dim < 0 || value_dim < 0 || ld < 2 * key_dim + value_dim) return cudaErrorInvalidValue;
    const int channels = 2 * key_dim + value_dim;
    const size_t n = (size_t)T * channels;
    if (n == 0) return cudaSuccess;
    const bool packed = key_dim % 8 == 0 && value_dim % 8 == 0 && ld % 8 == 0 && aligned16(qkv) && aligned16(w) &&
                        aligned16(q) && aligned16(k) && aligned16(v);
    if (packed) {
        const int tt = T <= CONV_SHORT_TOKENS ? CONV_TT_SHORT : CONV_TT;
        const dim3 grid((T + tt - 1) / tt, (channels / 8 + CONV_THREADS - 1) / CONV_THREADS);
        launch_dep(tt == CONV_TT ? gdn_conv_packed_kernel<CONV_TT> : gdn_conv_packed_kernel<CONV_TT_SHORT>, grid, CONV_THREADS, 0,
                   as_stream(stream), static_cast<const bf16*>(qkv), ld, static_cast<const bf16*>(w), static_cast<bf16*>(q),
                   static_cast<bf16*>(k), static_cast<bf16*>(v), T, key_dim, value_dim);
    } else {
        gdn_conv_scalar_kernel<<<blocks_for(n), THREADS, 0, as_stream(stream)>>>(
            static_cast<const bf16*>(qkv), ld, static_cast<const bf16*>(w), static_cast<bf16*>(q),
            static_cast<bf16*>(k), static_cast<bf16*>(v), T, key_dim, value_dim);
    }
    return cudaGetLastError();
}

extern "C" int cs1_gdn_gates(const void* b, const void* a, int ld, const void* A_log, const void* dt_bias,
                             void* beta, float* g, int T, int H, void* stream) {
    if (T < 0 || H < 0 || ld < H) return cudaErrorInvalidValue;
    const long long n = (long long)T * H;
    if (n == 0) return cudaSuccess;
    if (n > 0x7fffffffLL) return cudaErrorInvalidValue;
    launch_dep(gdn_gates_kernel, blocks_for((size_t)n), THREADS, 0, as_stream(stream), static_cast<const bf16*>(b),
               static_cast<const bf16*>(a), ld, static_cast<const bf16*>(A_log), static_cast<const bf16*>(dt_bias),
               static_cast<bf16*>(beta), g, (int)n, H);
    return cudaGetLastError();
}

extern "C" int s1_gdn_conv_gates(const void* qkv, int ld, const void* w, void* q, void* k, void* v, int T, int key_dim,
                                 int value_dim, const void* b, const void* a, const void* A_log, const void* dt_bias,
                                 void* beta, float* g, int H, void* stream) {
    if (T < 0 || key_dim < 0 || value_dim < 0 || H < 0 || ld < 2 * key_dim + value_dim || ld < H) return cudaErrorInvalidValue;
    const int channels = 2 * key_dim + value_dim;
    if (T == 0) return cudaSuccess;
    const bool packed = key_dim % 8 == 0 && value_dim % 8 == 0 && ld % 8 == 0 && aligned16(qkv) && aligned16(w) &&
                        aligned16(q) && aligned16(k) && aligned16(v);
    if (!packed || channels == 0 || H == 0 || (long long)T * H > 0x7fffffffLL) return CS1_ERR_UNSUPPORTED;
    const int conv_blocks = (channels / 8 + CONV_THREADS - 1) / CONV_THREADS;
    const int tt = T <= CONV_SHORT_TOKENS ? CONV_TT_SHORT : CONV_TT;
    const dim3 grid((T + tt - 1) / tt, conv_blocks + 1);
    launch_dep(tt == CONV_TT ? gdn_conv_gates_kernel<CONV_TT> : gdn_conv_gates_kernel<CONV_TT_SHORT>, grid, CONV_THREADS, 0,
               as_stream(stream), static_cast<const bf16*>(qkv), ld,
               static_cast<const bf16*>(w), static_cast<bf16*>(q), static_cast<bf16*>(k), static_cast<bf16*>(v), T, key_dim,
               value_dim, conv_blocks, static_cast<const bf16*>(b), static_cast<const bf16*>(a),
               static_cast<const bf16*>(A_log), static_cast<const bf16*>(dt_bias), static_cast<bf16*>(beta), g, H);
    return cudaGetLastError();
}

// s1_gdn_conv_gates for the sequences of one pack in one launch: every pointer is that of packed
// row 0 (b and a: the two gate columns of row 0); sequence i is rows [row0[i], row0[i] + len[i]).
// nseq <= 16, len[i] > 0. The same bits as one call per sequence; CS1_ERR_UNSUPPORTED likewise.
extern "C" int s1_gdn_conv_gates_batch(const void* qkv, int ld, const void* w, void* q, void* k, void* v, const int* row0,
                                       const int* len, int nseq, int key_dim, int value_dim, const void* b, const void* a,
                                       const void* A_log, const void* dt_bias, void* beta, float* g, int H, void* stream) {
    if (nseq <= 0 || nseq > 16 || !row0 || !len || key_dim < 0 || value_dim < 0 || H < 0 || ld < 2 * key_dim + value_dim || ld < H)
        return cudaErrorInvalidValue;
    const int channels = 2 * key_dim + value_dim;
    const bool packed = key_dim % 8 == 0 && value_dim % 8 == 0 && ld % 8 == 0 && aligned16(qkv) && aligned16(w) &&
                        aligned16(q) && aligned16(k) && aligned16(v);
    ConvSeqs seqs{};
    int longest = 0;
    for (int i = 0; i < nseq; i++) {
        if (row0[i] < 0 || len[i] <= 0) return cudaErrorInvalidValue;
        if ((long long)len[i] * H > 0x7fffffffLL) return CS1_ERR_UNSUPPORTED;
        seqs.row0[i] = row0[i];
        seqs.len[i] = len[i];
        longest = longest > len[i] ? longest : len[i];
    }
    if (!packed || channels == 0 || H == 0) return CS1_ERR_UNSUPPORTED;
    const int conv_blocks = (channels / 8 + CONV_THREADS - 1) / CONV_THREADS;
    const int tt = longest <= CONV_SHORT_TOKENS ? CONV_TT_SHORT : CONV_TT;
    const dim3 grid((longest + tt - 1) / tt, conv_blocks + 1, nseq);
    launch_dep(tt == CONV_TT ? gdn_conv_gates_batch_kernel<CONV_TT> : gdn_conv_gates_batch_kernel<CONV_TT_SHORT>, grid,
               CONV_THREADS, 0, as_stream(stream), static_cast<const bf16*>(qkv), ld, static_cast<const bf16*>(w),
               static_cast<bf16*>(q), static_cast<bf16*>(k), static_cast<bf16*>(v), seqs, key_dim, value_dim, conv_blocks,
               static_cast<const bf16*>(b), static_cast<const bf16*>(a), static_cast<const bf16*>(A_log),
               static_cast<const bf16*>(dt_bias), static_cast<bf16*>(beta), g, H);
    return cudaGetLastError();
}

extern "C" int cs1_sigmoid_gate(void* x, const void* gate, size_t n, void* stream) {
    if (n == 0) return cudaSuccess;
    if (n % 8 == 0 && aligned16(x) && aligned16(gate)) {
        launch_dep(sigmoid_gate_packed_kernel, blocks_for(n / 8), THREADS, 0, as_stream(stream), static_cast<uint4*>(x),
                   static_cast<const uint4*>(gate), n / 8);
    } else {
        sigmoid_gate_kernel<<<blocks_for(n), THREADS, 0, as_stream(stream)>>>(static_cast<bf16*>(x),
                                                                             static_cast<const bf16*>(gate), n);
    }
    return cudaGetLastError();
}

extern "C" int cs1_silu_mul(const void* gate_up, int ld, void* out, int T, int I, void* stream) {
    if (T < 0 || I < 0 || ld < 2 * I) return cudaErrorInvalidValue;
    const size_t n = (size_t)T * I;
    if (n == 0) return cudaSuccess;
    if (I % 8 == 0 && ld % 8 == 0 && aligned16(gate_up) && aligned16(out)) {
        launch_dep(silu_mul_packed_kernel, blocks_for(n / 8, 2 * THREADS), THREADS, 0, as_stream(stream),
                   static_cast<const uint4*>(gate_up), ld / 8, static_cast<uint4*>(out), I / 8, n / 8);
    } else {
        silu_mul_kernel<<<blocks_for(n), THREADS, 0, as_stream(stream)>>>(static_cast<const bf16*>(gate_up), ld,
                                                                         static_cast<bf16*>(out), I, n);
    }
    return cudaGetLastError();
}
