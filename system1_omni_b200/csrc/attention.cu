// Full-attention layers: q/k preparation (per-head RMSNorm, partial rotary embedding, gate
// split) and the entry points of causal grouped-query attention with the sigmoid output gate,
// for head dims 128 and 256. The attention itself is the tcgen05 kernel of attention_tc5.cu:
// probabilities are rounded to bf16 for P*V while the running sums stay float32, and the gated
// epilogue rounds both factors to bf16 before multiplying, which makes the fused result equal
// to attention followed by a separate gate pass bit for bit, and a windowed launch equal to the
// rows of a full launch (reference contract: src/backends/cuda/qwen3_5/attention.cu:84-233,
// tests/qwen3_5/kernels.rs:273-474,852-929).
#include <math.h>

#include "attention_tc5.h"
#include "common.cuh"
#include "cs1_ops.h"

namespace s1 {
namespace {

// ---- q/k RMSNorm + rotary + gate split (attention.cu:19-71 of the reference) ----
// DH/8 lanes per (token, head), 8 consecutive dims per lane; the rotary partner of dim d
// (d +- half) lives half/8 lanes away.
// The sequences of a pack for the batched form: sequence i is rows [row0[i], row0[i] + rows[i]) and
// its first row has position 0 of the tables it is given; rows outside every sequence are skipped.
// n = 0: one sequence, row t at position t.
struct PrepSeqs {
    int n;
    int row0[16], rows[16];
};

template <int DH>
__global__ void __launch_bounds__(256)
    attn_prep_kernel(const bf16* __restrict__ qg, const bf16* __restrict__ kr, int ld, const bf16* __restrict__ qw,
                     const bf16* __restrict__ kw, const bf16* __restrict__ cos_t, const bf16* __restrict__ sin_t,
                     bf16* __restrict__ q, bf16* __restrict__ gate, bf16* __restrict__ k, long long total, int Hq,
                     int Hk, int half, float eps, const __grid_constant__ PrepSeqs seqs) {
    grid_dep_trigger();
    grid_dep_sync();
    constexpr int LANES = DH / 8;
    const int sub = threadIdx.x % LANES;
    long long unit = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / LANES;
    bool live = unit < total;
    if (!live) unit = total - 1;
    const int heads = Hq + Hk;
    const int t = (int)(unit / heads), hh = (int)(unit % heads);
    int pos = t;  // the row's position in the rotary tables
    if (seqs.n > 0) {
        pos = -1;
        for (int i = 0; i < seqs.n; i++)
            if (t >= seqs.row0[i] && t < seqs.row0[i] + seqs.rows[i]) pos = t - seqs.row0[i];
        live = live && pos >= 0;
        pos = max(pos, 0);
    }
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
        unpack8(ld16(cos_t + (size_t)pos * half + d0 % half), cs);
        unpack8(ld16(sin_t + (size_t)pos * half + d0 % half), sn);
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

constexpr int BM = 64;  // a window starts on a multiple of 64 rows (the delta rule's chunk, model.rs:955-958)

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
    return s1_attn_tc5(qp, kp, vp, ldv, GATED ? gp : nullptr, op, T, Hq, Hk, Dh, scale, q_base, nullptr, nullptr, 0, 0,
                       as_stream(stream));
}

}  // namespace
}  // namespace s1

using namespace s1;

namespace {

int attn_prep_run(const void* qg, const void* kr, int ld, const void* qw, const void* kw, const void* cos, const void* sin,
                  void* q, void* gate, void* k, int T, int Hq, int Hk, int Dh, int half, float eps, const PrepSeqs& seqs,
                  void* stream) {
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
                   static_cast<bf16*>(gate), static_cast<bf16*>(k), total, Hq, Hk, half, eps, seqs);
    else
        launch_dep(attn_prep_kernel<128>, grid, 256, 0, as_stream(stream), a0, a1, ld, a2, a3, a4, a5, static_cast<bf16*>(q),
                   static_cast<bf16*>(gate), static_cast<bf16*>(k), total, Hq, Hk, half, eps, seqs);
    return cudaGetLastError();
}

}  // namespace

extern "C" int cs1_attn_prep(const void* qg, const void* kr, int ld, const void* qw, const void* kw, const void* cos,
                             const void* sin, void* q, void* gate, void* k, int T, int Hq, int Hk, int Dh, int half,
                             float eps, void* stream) {
    return attn_prep_run(qg, kr, ld, qw, kw, cos, sin, q, gate, k, T, Hq, Hk, Dh, half, eps, PrepSeqs{}, stream);
}

// cs1_attn_prep for the sequences of one pack in one launch: all pointers are those of packed row 0,
// T the packed rows in all; sequence i is rows [row0[i], row0[i] + rows[i]) and its first row takes
// the first row of the tables (cos, sin point at the position the sequences start from). Rows
// outside every sequence are left as they are. nseq <= 16. The same bits as one call per sequence.
extern "C" int s1_attn_prep_batch(const void* qg, const void* kr, int ld, const void* qw, const void* kw, const void* cos,
                                  const void* sin, void* q, void* gate, void* k, int T, const int* row0, const int* rows,
                                  int nseq, int Hq, int Hk, int Dh, int half, float eps, void* stream) {
    if (nseq <= 0 || nseq > 16 || !row0 || !rows) return cudaErrorInvalidValue;
    PrepSeqs seqs{};
    seqs.n = nseq;
    for (int i = 0; i < nseq; i++) {
        if (row0[i] < 0 || rows[i] <= 0 || row0[i] + rows[i] > T) return cudaErrorInvalidValue;
        seqs.row0[i] = row0[i];
        seqs.rows[i] = rows[i];
    }
    return attn_prep_run(qg, kr, ld, qw, kw, cos, sin, q, gate, k, T, Hq, Hk, Dh, half, eps, seqs, stream);
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
    return s1_attn_tc5(qp, kp, vp, ldv, gp, op, T, Hq, Hk, Dh, scale, prefix_len, kpre, vpre, ldv_prefix, prefix_len,
                       as_stream(stream));
}

// s1_attention_gated_shared_prefix for the sequences of one pack in one launch: sequence i owns
// rows [row0[i], row0[i] + rows[i]) of q, k, v, gate and out and sits at positions
// [prefix_len, prefix_len + rows[i]) behind the shared prefix (prefix_len 0: no prefix, the plain
// packed pass). nseq <= 16, rows[i] > 0. The same bits as one call per sequence.
extern "C" int s1_attention_gated_batch(const void* q, const void* k, const void* v, int ldv, const void* gate, void* out,
                                        const void* k_prefix, const void* v_prefix, int ldv_prefix, int prefix_len,
                                        const int* row0, const int* rows, int nseq, int Hq, int Hk, int Dh, float scale,
                                        void* stream) {
    if ((Dh != 128 && Dh != 256) || Hk <= 0 || Hq <= 0 || Hq % Hk != 0 || ldv % 8 != 0 || ldv < Hk * Dh || prefix_len < 0 ||
        prefix_len % BM || nseq <= 0 || nseq > 16 || !row0 || !rows)
        return cudaErrorInvalidValue;
    if (prefix_len > 0 && (ldv_prefix % 8 != 0 || ldv_prefix < Hk * Dh || !k_prefix || !v_prefix)) return cudaErrorInvalidValue;
    if (!q || !k || !v || !gate || !out) return cudaErrorInvalidValue;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(k_prefix) || !aligned16(v_prefix) ||
        (reinterpret_cast<uintptr_t>(out) & 3) || (reinterpret_cast<uintptr_t>(gate) & 3))
        return cudaErrorInvalidValue;
    int T[16];
    for (int i = 0; i < nseq; i++) {
        if (rows[i] <= 0 || row0[i] < 0) return cudaErrorInvalidValue;
        T[i] = prefix_len + rows[i];
    }
    return s1_attn_tc5_batch(static_cast<const bf16*>(q), static_cast<const bf16*>(k), static_cast<const bf16*>(v), ldv,
                             static_cast<const bf16*>(gate), static_cast<bf16*>(out), row0, T, nseq, Hq, Hk, Dh, scale,
                             prefix_len, static_cast<const bf16*>(k_prefix), static_cast<const bf16*>(v_prefix), ldv_prefix,
                             prefix_len, as_stream(stream));
}

extern "C" int cs1_attention_gated_prefix(const void* q, const void* k, const void* v, int ldv, const void* gate,
                                          void* out, int T, int Hq, int Hk, int Dh, float scale, int q_base,
                                          void* stream) {
    return attention_entry<true>(q, k, v, ldv, gate, out, T, Hq, Hk, Dh, scale, q_base, stream);
}
