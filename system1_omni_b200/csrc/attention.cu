// Full-attention layers: q/k preparation (per-head RMSNorm, partial rotary embedding, gate
// split) and causal grouped-query flash attention with the sigmoid output gate fused into
// the epilogue, for head dims 128 and 256.
//
// The attention kernel keeps the online softmax and the output tile in registers
// (FlashAttention-2 schedule on mma.sync m16n8k16): one block takes 64 queries of one head,
// four warps of 16 rows, and walks the keys in double-buffered cp.async tiles. Probabilities
// are rounded to bf16 for P*V while the running sums stay float32, and the gated epilogue
// rounds both factors to bf16 before multiplying, which makes the fused result equal to
// attention followed by a separate gate pass bit for bit, and a windowed launch equal to
// the rows of a full launch (reference contract: src/backends/cuda/qwen3_5/attention.cu:84-233,
// tests/qwen3_5/kernels.rs:273-474,852-929).
#include <math.h>

#include "attention_tc5.h"
#include "common.cuh"
#include "cs1_ops.h"
#include "mma.cuh"

namespace s1 {
namespace {

// ---- q/k RMSNorm + rotary + gate split (attention.cu:19-71 of the reference) ----
// DH/8 lanes per (token, head), 8 consecutive dims per lane; the rotary partner of dim d
// (d +- half) lives half/8 lanes away.
template <int DH>
__global__ void __launch_bounds__(256)
    attn_prep_kernel(const bf16* __restrict__ qg, const bf16* __restrict__ kr, int ld, const bf16* __restrict__ qw,
                     const bf16* __restrict__ kw, const bf16* __restrict__ cos_t, const bf16* __restrict__ sin_t,
                     bf16* __restrict__ q, bf16* __restrict__ gate, bf16* __restrict__ k, long long total, int Hq,
                     int Hk, int half, float eps) {
    grid_dep_trigger();
    grid_dep_sync();
    constexpr int LANES = DH / 8;
    const int sub = threadIdx.x % LANES;
    long long unit = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / LANES;
    const bool live = unit < total;
    if (!live) unit = total - 1;
    const int heads = Hq + Hk;
    const int t = (int)(unit / heads), hh = (int)(unit % heads);
    const bool is_q = hh < Hq;
    const int h = is_q ? hh : hh - Hq;
    const bf16* src = is_q ? qg + (size_t)t * ld + (size_t)h * 2 * DH : kr + (size_t)t * ld + (size_t)h * DH;
    const bf16* w = is_q ? qw : kw;
    const int d0 = sub * 8;

    float x[8], wv[8];
    unpack8(ld16_stream(src + d0), x);
    unpack8(ld16(w + d0), wv);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) ss += x[i] * x[i];
    const float inv = rsqrtf(warp_sum<LANES>(ss) / DH + eps);
#pragma unroll
    for (int i = 0; i < 8; i++) x[i] = rbf(x[i] * inv * (1.f + wv[i]));

    const int rot = 2 * half;
    float y[8];
    float cs[8], sn[8];
    if (d0 < rot) {
        // half is a multiple of 8, so the 8 dims of a lane share one aligned table pack
        unpack8(ld16(cos_t + (size_t)t * half + d0 % half), cs);
        unpack8(ld16(sin_t + (size_t)t * half + d0 % half), sn);
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float partner = __shfl_xor_sync(0xffffffffu, x[i], half / 8);
        y[i] = x[i];
        if (d0 < rot) {
            const float r = d0 < half ? -partner : partner;
            y[i] = rbf(rbf(x[i] * cs[i]) + rbf(r * sn[i]));
        }
    }
    if (!live) return;
    if (is_q) {
        st16(q + ((size_t)t * Hq + h) * DH + d0, pack8(y));
        st16(gate + ((size_t)t * Hq + h) * DH + d0, ld16_stream(src + DH + d0));
    } else {
        st16(k + ((size_t)t * Hk + h) * DH + d0, pack8(y));
    }
}

// ---- flash attention ----
constexpr int BM = 64, FA_THREADS = 128;

template <int DH, int BN>
struct FaSmem {
    static constexpr int LDS = DH + 8;  // row stride in elements; 16 extra bytes keep ldmatrix conflict-free
    static constexpr int BYTES = (BM + 4 * BN) * LDS * 2;
};

template <int DH, int BN, bool GATED>
__global__ void __launch_bounds__(FA_THREADS)
    flash_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v, int ldv,
                 const bf16* __restrict__ gate, bf16* __restrict__ out, int T, int Hq, int Hk, float scale_log2,
                 int q_base, const bf16* __restrict__ kpre, const bf16* __restrict__ vpre, int ldvpre, int own_base) {
    // Rows are absolute positions. Keys and values of positions below own_base come from the
    // shared prefix buffers (kpre, vpre); q, gate, out, k and v hold the positions from own_base
    // on, indexed from zero. own_base = 0: everything in q, k, v (the plain and q_base entries).
    constexpr int LDS = FaSmem<DH, BN>::LDS;
    constexpr int NT = BN / 8;   // score tiles per warp row block
    constexpr int DT = DH / 8;   // output tiles
    extern __shared__ __align__(16) unsigned char smem[];
    bf16* qs = reinterpret_cast<bf16*>(smem);
    bf16* ks = qs + BM * LDS;           // [2][BN][LDS]
    bf16* vs = ks + 2 * BN * LDS;       // [2][BN][LDS]
    const int h = blockIdx.y, hk = h / (Hq / Hk);
    const int q0 = q_base + (gridDim.x - 1 - blockIdx.x) * BM;  // longest blocks first
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int g = lane / 4, t = lane % 4;
    const int row0 = q0 + warp * 16;

    constexpr int CPR = DH / 8;  // 16-byte chunks per row
    for (int c = tid; c < BM * CPR; c += FA_THREADS) {
        const int r = c / CPR, col = (c % CPR) * 8, row = q0 + r;
        cp_async16(qs + r * LDS + col, q + ((size_t)(min(row, T - 1) - own_base) * Hq + h) * DH + col, row < T);
    }
    const int kv_end = min(T, q0 + BM);
    const int ntiles = (kv_end + BN - 1) / BN;
    auto load_kv = [&](int tile, int stage) {
        const int k0 = tile * BN;
        bf16* kd = ks + stage * BN * LDS;
        bf16* vd = vs + stage * BN * LDS;
        for (int c = tid; c < BN * CPR; c += FA_THREADS) {
            const int r = c / CPR, col = (c % CPR) * 8, row = k0 + r;
            const bool ok = row < kv_end;
            const int rr = min(row, T - 1);
            if (rr < own_base) {
                cp_async16(kd + r * LDS + col, kpre + ((size_t)rr * Hk + hk) * DH + col, ok);
                cp_async16(vd + r * LDS + col, vpre + (size_t)rr * ldvpre + (size_t)hk * DH + col, ok);
            } else {
                cp_async16(kd + r * LDS + col, k + ((size_t)(rr - own_base) * Hk + hk) * DH + col, ok);
                cp_async16(vd + r * LDS + col, v + (size_t)(rr - own_base) * ldv + (size_t)hk * DH + col, ok);
            }
        }
    };
    load_kv(0, 0);
    cp_async_commit();

    float o[DT][4];
#pragma unroll
    for (int n = 0; n < DT; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int j = 0; j < ntiles; j++) {
        if (j + 1 < ntiles) {
            load_kv(j + 1, (j + 1) & 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const bf16* kt = ks + (j & 1) * BN * LDS;
        const bf16* vt = vs + (j & 1) * BN * LDS;
        const int k0 = j * BN;

        float s[NT][4];
#pragma unroll
        for (int n = 0; n < NT; n++) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < DH / 16; kk++) {
            uint32_t a[4];
            load_a_rm(a, qs, LDS, warp * 16, kk * 16, lane);
#pragma unroll
            for (int np = 0; np < NT / 2; np++) {
                uint32_t b[4];
                load_b_nk(b, kt, LDS, np * 16, kk * 16, lane);
                mma_bf16(s[2 * np], a, b[0], b[1]);
                mma_bf16(s[2 * np + 1], a, b[2], b[3]);
            }
        }
        // causal mask on tiles that reach past this warp's first row
        if (k0 + BN - 1 > row0) {
#pragma unroll
            for (int n = 0; n < NT; n++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int key = k0 + n * 8 + 2 * t + (e & 1);
                    const int row = row0 + g + (e >> 1) * 8;
                    if (key > row) s[n][e] = -INFINITY;
                }
            }
        }
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            float mx = -INFINITY;
#pragma unroll
            for (int n = 0; n < NT; n++) mx = fmaxf(mx, fmaxf(s[n][2 * r], s[n][2 * r + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float mn = fmaxf(m[r], mx * scale_log2);
            alpha[r] = exp2f(m[r] - mn);
            m[r] = mn;
            float sum = 0.f;
#pragma unroll
            for (int n = 0; n < NT; n++) {
                const float p0 = exp2f(s[n][2 * r] * scale_log2 - mn);
                const float p1 = exp2f(s[n][2 * r + 1] * scale_log2 - mn);
                s[n][2 * r] = p0;
                s[n][2 * r + 1] = p1;
                sum += p0 + p1;
            }
            l[r] = l[r] * alpha[r] + sum;
        }
#pragma unroll
        for (int n = 0; n < DT; n++) {
            o[n][0] *= alpha[0];
            o[n][1] *= alpha[0];
            o[n][2] *= alpha[1];
            o[n][3] *= alpha[1];
        }
#pragma unroll
        for (int kt2 = 0; kt2 < BN / 16; kt2++) {
            uint32_t a[4];
            a[0] = pack2(s[2 * kt2][0], s[2 * kt2][1]);
            a[1] = pack2(s[2 * kt2][2], s[2 * kt2][3]);
            a[2] = pack2(s[2 * kt2 + 1][0], s[2 * kt2 + 1][1]);
            a[3] = pack2(s[2 * kt2 + 1][2], s[2 * kt2 + 1][3]);
#pragma unroll
            for (int dp = 0; dp < DT / 2; dp++) {
                uint32_t b[4];
                load_b_kn(b, vt, LDS, kt2 * 16, dp * 16, lane);
                mma_bf16(o[2 * dp], a, b[0], b[1]);
                mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();  // every warp is done with this stage before it is refilled
    }

#pragma unroll
    for (int r = 0; r < 2; r++) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    const float inv[2] = {1.f / l[0], 1.f / l[1]};
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int row = row0 + g + r * 8;
        if (row >= T) continue;
        const size_t base = ((size_t)(row - own_base) * Hq + h) * DH + 2 * t;
#pragma unroll
        for (int n = 0; n < DT; n++) {
            float a = o[n][2 * r] * inv[r], b = o[n][2 * r + 1] * inv[r];
            if constexpr (GATED) {
                const uint32_t gw = *reinterpret_cast<const uint32_t*>(gate + base + n * 8);
                // attention -> bf16 store -> bf16 sigmoid -> multiply, without the store
                a = rbf(a) * rbf(sigmoid(__uint_as_float(gw << 16)));
                b = rbf(b) * rbf(sigmoid(__uint_as_float(gw & 0xffff0000u)));
            }
            *reinterpret_cast<uint32_t*>(out + base + n * 8) = pack2(a, b);
        }
    }
}

template <int DH, int BN, bool GATED>
int launch_flash(const bf16* q, const bf16* k, const bf16* v, int ldv, const bf16* gate, bf16* out, int T, int Hq,
                 int Hk, float scale, int q_base, cudaStream_t st, const bf16* kpre = nullptr,
                 const bf16* vpre = nullptr, int ldvpre = 0, int own_base = 0) {
    constexpr int BYTES = FaSmem<DH, BN>::BYTES;
    // Raise the dynamic shared memory limit once per device.
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 64) return cudaErrorInvalidDevice;
    if (!configured[dev]) {
        e = cudaFuncSetAttribute(flash_kernel<DH, BN, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, BYTES);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    constexpr float LOG2E = 1.4426950408889634f;
    const dim3 grid((T - q_base + BM - 1) / BM, Hq);
    flash_kernel<DH, BN, GATED><<<grid, FA_THREADS, BYTES, st>>>(q, k, v, ldv, gate, out, T, Hq, Hk, scale * LOG2E,
                                                                q_base, kpre, vpre, ldvpre, own_base);
    return cudaGetLastError();
}

template <bool GATED>
int attention_entry(const void* q, const void* k, const void* v, int ldv, const void* gate, void* out, int T, int Hq,
                    int Hk, int Dh, float scale, int q_base, void* stream) {
    if ((Dh != 128 && Dh != 256) || Hk <= 0 || Hq <= 0 || Hq % Hk != 0 || ldv % 8 != 0 || ldv < Hk * Dh || T < 0)
        return cudaErrorInvalidValue;
    if (q_base < 0 || q_base % BM || q_base > T) return cudaErrorInvalidValue;
    if (T == q_base) return cudaSuccess;
    if (GATED && gate == nullptr) return cudaErrorInvalidValue;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || (reinterpret_cast<uintptr_t>(out) & 3) ||
        (GATED && (reinterpret_cast<uintptr_t>(gate) & 3)))
        return cudaErrorInvalidValue;
    const bf16 *qp = static_cast<const bf16*>(q), *kp = static_cast<const bf16*>(k), *vp = static_cast<const bf16*>(v);
    const bf16* gp = static_cast<const bf16*>(gate);
    bf16* op = static_cast<bf16*>(out);
    // one kernel for every size, so that a window and the one-shot pass round alike
    if (s1_attn_tc5_enabled())
        return s1_attn_tc5(qp, kp, vp, ldv, GATED ? gp : nullptr, op, T, Hq, Hk, Dh, scale, q_base, nullptr, nullptr, 0, 0,
                           as_stream(stream));
    if (Dh == 256) return launch_flash<256, 32, GATED>(qp, kp, vp, ldv, gp, op, T, Hq, Hk, scale, q_base, as_stream(stream));
    return launch_flash<128, 64, GATED>(qp, kp, vp, ldv, gp, op, T, Hq, Hk, scale, q_base, as_stream(stream));
}

}  // namespace
}  // namespace s1

using namespace s1;

extern "C" int cs1_attn_prep(const void* qg, const void* kr, int ld, const void* qw, const void* kw, const void* cos,
                             const void* sin, void* q, void* gate, void* k, int T, int Hq, int Hk, int Dh, int half,
                             float eps, void* stream) {
    if (ld % 8 != 0 || T < 0 || Hq < 0 || Hk < 0) return cudaErrorInvalidValue;
    // the lane ^ (half / 8) partner exchange needs half a multiple of 8, half / 8 a power of two, 2 * half <= Dh
    if ((Dh != 128 && Dh != 256) || half <= 0 || half % 8 != 0 || 2 * half > Dh || ((half / 8) & (half / 8 - 1)))
        return cudaErrorInvalidValue;
    const long long total = (long long)T * (Hq + Hk);
    if (total == 0) return cudaSuccess;
    if (!aligned16(qg) || !aligned16(kr) || !aligned16(qw) || !aligned16(kw) || !aligned16(cos) || !aligned16(sin) ||
        !aligned16(q) || !aligned16(gate) || !aligned16(k))
        return cudaErrorInvalidValue;
    const int lanes = Dh / 8;
    const long long threads = total * lanes;
    const unsigned grid = (unsigned)((threads + 255) / 256);
    const bf16 *a0 = static_cast<const bf16*>(qg), *a1 = static_cast<const bf16*>(kr), *a2 = static_cast<const bf16*>(qw),
               *a3 = static_cast<const bf16*>(kw), *a4 = static_cast<const bf16*>(cos), *a5 = static_cast<const bf16*>(sin);
    if (Dh == 256)
        launch_dep(attn_prep_kernel<256>, grid, 256, 0, as_stream(stream), a0, a1, ld, a2, a3, a4, a5, static_cast<bf16*>(q),
                                                                   static_cast<bf16*>(gate), static_cast<bf16*>(k),
                                                                   total, Hq, Hk, half, eps);
    else
        launch_dep(attn_prep_kernel<128>, grid, 256, 0, as_stream(stream), a0, a1, ld, a2, a3, a4, a5, static_cast<bf16*>(q),
                                                                   static_cast<bf16*>(gate), static_cast<bf16*>(k),
                                                                   total, Hq, Hk, half, eps);
    return cudaGetLastError();
}

extern "C" int cs1_attention(const void* q, const void* k, const void* v, int ldv, void* out, int T, int Hq, int Hk,
                             int Dh, float scale, void* stream) {
    return attention_entry<false>(q, k, v, ldv, nullptr, out, T, Hq, Hk, Dh, scale, 0, stream);
}

extern "C" int cs1_attention_gated(const void* q, const void* k, const void* v, int ldv, const void* gate, void* out,
                                   int T, int Hq, int Hk, int Dh, float scale, void* stream) {
    return attention_entry<true>(q, k, v, ldv, gate, out, T, Hq, Hk, Dh, scale, 0, stream);
}

// Gated causal attention of a window that continues a shared prefix: positions
// [prefix_len, prefix_len + rows). q, gate, out [rows, Hq, Dh], k [rows, Hk, Dh] and v (row
// stride ldv) hold the window only; the prefix's post-prep keys [prefix_len, Hk, Dh] and values
// (row stride ldv_prefix) are read where they lie, so several windows can share one copy. Same
// tiles and arithmetic as cs1_attention_gated_prefix on the concatenated buffers (the
// reference restores the prefix rows into the scratch first, model.rs:1516-1523).
extern "C" int s1_attention_gated_shared_prefix(const void* q, const void* k, const void* v, int ldv, const void* gate,
                                                void* out, const void* k_prefix, const void* v_prefix, int ldv_prefix,
                                                int prefix_len, int rows, int Hq, int Hk, int Dh, float scale,
                                                void* stream) {
    if ((Dh != 128 && Dh != 256) || Hk <= 0 || Hq <= 0 || Hq % Hk != 0 || ldv % 8 != 0 || ldv < Hk * Dh ||
        ldv_prefix % 8 != 0 || ldv_prefix < Hk * Dh || rows < 0 || prefix_len < 0 || prefix_len % BM)
        return cudaErrorInvalidValue;
    if (rows == 0) return cudaSuccess;
    if (!q || !k || !v || !gate || !out || (prefix_len > 0 && (!k_prefix || !v_prefix))) return cudaErrorInvalidValue;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(k_prefix) || !aligned16(v_prefix) ||
        (reinterpret_cast<uintptr_t>(out) & 3) || (reinterpret_cast<uintptr_t>(gate) & 3))
        return cudaErrorInvalidValue;
    const bf16 *qp = static_cast<const bf16*>(q), *kp = static_cast<const bf16*>(k), *vp = static_cast<const bf16*>(v);
    const bf16 *kpre = static_cast<const bf16*>(k_prefix), *vpre = static_cast<const bf16*>(v_prefix);
    const bf16* gp = static_cast<const bf16*>(gate);
    bf16* op = static_cast<bf16*>(out);
    const int T = prefix_len + rows;
    if (s1_attn_tc5_enabled())
        return s1_attn_tc5(qp, kp, vp, ldv, gp, op, T, Hq, Hk, Dh, scale, prefix_len, kpre, vpre, ldv_prefix, prefix_len,
                           as_stream(stream));
    if (Dh == 256)
        return launch_flash<256, 32, true>(qp, kp, vp, ldv, gp, op, T, Hq, Hk, scale, prefix_len, as_stream(stream), kpre,
                                           vpre, ldv_prefix, prefix_len);
    return launch_flash<128, 64, true>(qp, kp, vp, ldv, gp, op, T, Hq, Hk, scale, prefix_len, as_stream(stream), kpre, vpre,
                                       ldv_prefix, prefix_len);
}

extern "C" int cs1_attention_gated_prefix(const void* q, const void* k, const void* v, int ldv, const void* gate,
                                          void* out, int T, int Hq, int Hk, int Dh, float scale, int q_base,
                                          void* stream) {
    return attention_entry<true>(q, k, v, ldv, gate, out, T, Hq, Hk, Dh, scale, q_base, stream);
}
