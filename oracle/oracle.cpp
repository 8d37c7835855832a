// CPU oracle for the Qwen3.5-style prefill path. TEST INFRASTRUCTURE ONLY.
//
// This file restates, in plain C++ for the host, the arithmetic that the reference
// project (ThinkFlowLab/system1-omni) defines for its prefill hot path. It is the checker
// that the GPU library is compared against and the timed CPU baseline of the benchmark.
// Nothing in the product (the CUDA library, the host executor) links, loads or calls it.
//
// Every function cites the reference file:line (paths relative to the reference
// repository root) whose semantics it follows:
//   tests/qwen3_5/kernels.rs                 float64 oracles and the seeded input generator
//   src/backends/cuda/qwen3_5/*.cu           rounding points of each operator
//   src/models/qwen3_5/native/src/model.rs   order of operators in a layer / decoder
//   src/models/qwen3_5/native/src/inputs.rs  rotary tables
//   src/models/open_jev/native/src/{executor,batching,contract}.rs  head, packing, decision
//   src/models/cua_s1/native/src/executor.rs letter head
//
// Parity pin: the reference keeps no stored tensor golden files for this path. Its pins
// are (1) numeric known-answer tests for the heads and the packing policy
// (tests/open_jev/head.rs, tests/cua_s1/head.rs, tests/open_jev/batching.rs), which
// tests/test_oracle_kat.py replays against this file, and (2) tolerance contracts between
// its kernels and the float64 oracles restated here; on a GPU box the reference's own CUDA
// library (built from its sources into oracle/_ref/) is run beside this oracle on the same
// seeded inputs (tests/test_ref_lib_gpu.py).
//
// bf16 values travel as uint16_t bit patterns.
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

inline float bf2f(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
inline uint32_t fbits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}
// Round to nearest even, as the half crate's bf16::from_f32 and CUDA's __float2bfloat16.
inline uint16_t f2bf(float f) {
    uint32_t u = fbits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
inline float rbf(float f) { return bf2f(f2bf(f)); }
// float64 -> bf16 with a single rounding (bf16::from_f64 in tests/qwen3_5/kernels.rs:190).
inline uint16_t d2bf(double d) {
    const float f = (float)d;
    const uint32_t u = fbits(f);
    if ((u & 0xffffu) == 0x8000u && (double)f != d && isfinite(f)) {
        const bool up = fabs(d) > fabs((double)f);
        return (uint16_t)((u >> 16) + (up ? 1 : 0));
    }
    return f2bf(f);
}
inline float silu_f(float x) { return x / (1.f + expf(-x)); }
inline float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

}  // namespace

extern "C" {

int orc_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

// Uniform values in [-amp, amp) rounded to bf16 from a fixed seed: the xorshift64
// generator of tests/qwen3_5/kernels.rs:25-36.
void orc_random_bf16(uint16_t* out, size_t n, uint64_t seed, float amp) {
    uint64_t x = (seed * 0x9e3779b97f4a7c15ull) | 1ull;
    for (size_t i = 0; i < n; i++) {
        x ^= x << 13;
        x ^= x >> 7;
        x ^= x << 17;
        const float v = ((float)(x >> 40) / (float)(1ull << 24) * 2.0f - 1.0f) * amp;
        out[i] = f2bf(v);
    }
}

void orc_f32_to_bf16(const float* in, uint16_t* out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = f2bf(in[i]);
}
void orc_bf16_to_f32(const uint16_t* in, float* out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = bf2f(in[i]);
}

// out[t] = table[ids[t]] (src/backends/cuda/qwen3_5/elementwise.cu:11-16).
void orc_embed(const int32_t* ids, const uint16_t* table, uint16_t* out, int T, int D) {
    for (int t = 0; t < T; t++) memcpy(out + (size_t)t * D, table + (size_t)ids[t] * D, (size_t)D * 2);
}

// Zero-centred RMSNorm. The value contract is the rounded reference of
// tests/qwen3_5/kernels.rs:126-140: sum of squares in float64, inv = 1/sqrt(f32(mean)+eps)
// in float32, out = bf16(v * inv * (1 + w)); the kernel (norm.cu:11-25) may differ by 1 ULP.
void orc_rms_norm(const uint16_t* x, const uint16_t* w, uint16_t* out, int rows, int D, float eps) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) {
        const uint16_t* xr = x + (size_t)r * D;
        double ss = 0;
        for (int i = 0; i < D; i++) {
            const double v = bf2f(xr[i]);
            ss += v * v;
        }
        const float inv = 1.0f / sqrtf((float)(ss / D) + eps);
        for (int i = 0; i < D; i++) out[(size_t)r * D + i] = f2bf(bf2f(xr[i]) * inv * (1.0f + bf2f(w[i])));
    }
}

// residual = bf16(residual + delta) in place, then RMSNorm of it
// (norm.cu:27-73; tests/qwen3_5/kernels.rs:84-140).
void orc_add_rms_norm(uint16_t* residual, const uint16_t* delta, const uint16_t* w, uint16_t* out, int rows,
                      int D, float eps) {
    const size_t n = (size_t)rows * D;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) residual[i] = f2bf(bf2f(residual[i]) + bf2f(delta[i]));
    orc_rms_norm(residual, w, out, rows, D, eps);
}

// Gated RMSNorm over rows of D (=128): n = bf16(x*inv); s = bf16(w*n); out = bf16(s*silu(z))
// (norm.cu:75-99). z is read with row stride ldz.
void orc_gated_rms_norm(const uint16_t* x, const uint16_t* z, int ldz, const uint16_t* w, uint16_t* out, int T,
                        int H, int D, float eps) {
#pragma omp parallel for schedule(static)
    for (int row = 0; row < T * H; row++) {
        const uint16_t* xr = x + (size_t)row * D;
        const uint16_t* zr = z + (size_t)(row / H) * ldz + (size_t)(row % H) * D;
        double ss = 0;
        for (int i = 0; i < D; i++) {
            const double v = bf2f(xr[i]);
            ss += v * v;
        }
        const float inv = 1.0f / sqrtf((float)(ss / D) + eps);
        for (int i = 0; i < D; i++) {
            const float normed = rbf(bf2f(xr[i]) * inv);
            const float scaled = rbf(bf2f(w[i]) * normed);
            out[(size_t)row * D + i] = f2bf(scaled * silu_f(bf2f(zr[i])));
        }
    }
}

// Depthwise causal conv (kernel 4) + SiLU, split into q, k, v (elementwise.cu:18-40):
// acc = sum_j fma(w[c][j], x[t-3+j][c]) in j order, y = bf16(silu(f32(bf16(acc)))).
void orc_gdn_conv(const uint16_t* qkv, int ld, const uint16_t* w, uint16_t* q, uint16_t* k, uint16_t* v, int T,
                  int key_dim, int value_dim) {
    const int ch = 2 * key_dim + value_dim;
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; t++) {
        for (int c = 0; c < ch; c++) {
            float acc = 0.f;
            for (int j = 0; j < 4; j++) {
                const int s = t - 3 + j;
                if (s >= 0) acc = fmaf(bf2f(w[c * 4 + j]), bf2f(qkv[(size_t)s * ld + c]), acc);
            }
            const uint16_t y = f2bf(silu_f(rbf(acc)));
            if (c < key_dim)
                q[(size_t)t * key_dim + c] = y;
            else if (c < 2 * key_dim)
                k[(size_t)t * key_dim + c - key_dim] = y;
            else
                v[(size_t)t * value_dim + c - 2 * key_dim] = y;
        }
    }
}

// beta = bf16(sigmoid(b)); g = -exp(A_log) * softplus(a + dt_bias), threshold 20, float32
// (elementwise.cu:42-55).
void orc_gdn_gates(const uint16_t* b, const uint16_t* a, int ld, const uint16_t* A_log, const uint16_t* dt_bias,
                   uint16_t* beta, float* g, int T, int H) {
    for (int i = 0; i < T * H; i++) {
        const int h = i % H;
        const size_t src = (size_t)(i / H) * ld + h;
        beta[i] = f2bf(sigmoid_f(bf2f(b[src])));
        const float x = bf2f(a[src]) + bf2f(dt_bias[h]);
        const float sp = x > 20.f ? x : log1pf(expf(x));
        g[i] = -expf(bf2f(A_log[h])) * sp;
    }
}

// out = bf16(bf16(silu(gate)) * up) with silu in float64 as the rounded reference of
// tests/qwen3_5/kernels.rs:184-196 (kernel: elementwise.cu:64-87, float32 silu, <= 1 ULP apart).
void orc_silu_mul(const uint16_t* gate_up, int ld, uint16_t* out, int T, int I) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; t++) {
        const uint16_t* row = gate_up + (size_t)t * ld;
        for (int j = 0; j < I; j++) {
            const double gate = bf2f(row[j]);
            const uint16_t act = d2bf(gate / (1.0 + exp(-gate)));
            out[(size_t)t * I + j] = f2bf(bf2f(act) * bf2f(row[I + j]));
        }
    }
}

// x = bf16(x * bf16(sigmoid(gate))) (elementwise.cu:57-62).
void orc_sigmoid_gate(uint16_t* x, const uint16_t* gate, size_t n) {
    for (size_t i = 0; i < n; i++) x[i] = f2bf(bf2f(x[i]) * rbf(sigmoid_f(bf2f(gate[i]))));
}

// cos/sin tables [T, half] in bf16 for text positions (all three axes equal):
// float32 inverse frequencies and products, float64 trig (inputs.rs:69-95).
void orc_rotary_tables(const int64_t* positions, int T, int half, double theta, uint16_t* cos_t, uint16_t* sin_t) {
    std::vector<float> inv(half);
    for (int i = 0; i < half; i++) inv[i] = 1.0f / powf((float)theta, (float)(2 * i) / (float)(2 * half));
    for (int t = 0; t < T; t++)
        for (int i = 0; i < half; i++) {
            const double angle = (double)(inv[i] * (float)positions[t]);
            cos_t[(size_t)t * half + i] = f2bf((float)cos(angle));
            sin_t[(size_t)t * half + i] = f2bf((float)sin(angle));
        }
}

// q/k RMSNorm(1+w) over Dh rounded to bf16, then rotary on the first 2*half dims with
// every product and the sum rounded to bf16; q_proj rows are [q(Dh) | gate(Dh)] per head
// (attention.cu:19-71).
void orc_attn_prep(const uint16_t* qg, const uint16_t* kr, int ld, const uint16_t* qw, const uint16_t* kw,
                   const uint16_t* cos_t, const uint16_t* sin_t, uint16_t* q, uint16_t* gate, uint16_t* k, int T,
                   int Hq, int Hk, int Dh, int half, float eps) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; t++) {
        std::vector<float> x(Dh);
        for (int hh = 0; hh < Hq + Hk; hh++) {
            const bool is_q = hh < Hq;
            const int h = is_q ? hh : hh - Hq;
            const uint16_t* src = is_q ? qg + (size_t)t * ld + (size_t)h * 2 * Dh : kr + (size_t)t * ld + (size_t)h * Dh;
            const uint16_t* w = is_q ? qw : kw;
            double ss = 0;
            for (int d = 0; d < Dh; d++) {
                const double v = bf2f(src[d]);
                ss += v * v;
            }
            const float inv = 1.0f / sqrtf((float)(ss / Dh) + eps);
            for (int d = 0; d < Dh; d++) x[d] = rbf(bf2f(src[d]) * inv * (1.f + bf2f(w[d])));
            uint16_t* dst = is_q ? q + ((size_t)t * Hq + h) * Dh : k + ((size_t)t * Hk + h) * Dh;
            for (int d = 0; d < Dh; d++) {
                float y = x[d];
                if (d < 2 * half) {
                    const int fi = d % half;
                    const float c = bf2f(cos_t[(size_t)t * half + fi]), s = bf2f(sin_t[(size_t)t * half + fi]);
                    const float r = d < half ? -x[d + half] : x[d - half];
                    y = rbf(rbf(x[d] * c) + rbf(r * s));
                }
                dst[d] = f2bf(y);
            }
            if (is_q) memcpy(gate + ((size_t)t * Hq + h) * Dh, src + Dh, (size_t)Dh * 2);
        }
    }
}

// y[M,N] (rows of ldy) = bf16( x[M,K] . w[N,K]^T ), products exact in float32, partial sums
// in float32 over 16 lanes, combined in float64, one bf16 rounding (gemm.cu:1-9 states
// float32 accumulation with unspecified order; no reference test pins the order).
void orc_gemm(const uint16_t* x, const uint16_t* w, uint16_t* y, int M, int N, int K, int ldy) {
    if (M <= 0 || N <= 0) return;
    const int MB = 4, NB = 4, L = 16;
    const int Kp = (K + L - 1) / L * L;
    std::vector<float> xf((size_t)M * Kp, 0.f);
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++)
        for (int kk = 0; kk < K; kk++) xf[(size_t)m * Kp + kk] = bf2f(x[(size_t)m * K + kk]);
    const int nblocks = (N + NB - 1) / NB;
#pragma omp parallel
    {
        std::vector<float> wf((size_t)NB * Kp, 0.f);
#pragma omp for schedule(dynamic, 8)
        for (int nb = 0; nb < nblocks; nb++) {
            const int n0 = nb * NB, nn = std::min(NB, N - n0);
            for (int j = 0; j < NB; j++)
                for (int kk = 0; kk < K; kk++)
                    wf[(size_t)j * Kp + kk] = j < nn ? bf2f(w[(size_t)(n0 + j) * K + kk]) : 0.f;
            for (int m0 = 0; m0 < M; m0 += MB) {
                const int mm = std::min(MB, M - m0);
                float acc[MB][NB][L];
                memset(acc, 0, sizeof(acc));
                const float* xp[MB];
                for (int i = 0; i < MB; i++) xp[i] = xf.data() + (size_t)(m0 + std::min(i, mm - 1)) * Kp;
                for (int kk = 0; kk < Kp; kk += L) {
                    for (int i = 0; i < MB; i++)
                        for (int j = 0; j < NB; j++) {
                            const float* a = xp[i] + kk;
                            const float* b = wf.data() + (size_t)j * Kp + kk;
#pragma omp simd
                            for (int l = 0; l < L; l++) acc[i][j][l] += a[l] * b[l];
                        }
                }
                for (int i = 0; i < mm; i++)
                    for (int j = 0; j < nn; j++) {
                        double s = 0;
                        for (int l = 0; l < L; l++) s += acc[i][j][l];
                        y[(size_t)(m0 + i) * ldy + n0 + j] = f2bf((float)s);
                    }
            }
        }
    }
}

// Token-by-token gated delta rule in float64 with the L2 norms of q and k inside and q
// scaled by D^-1/2: gated_delta_reference of tests/qwen3_5/kernels.rs:476-525.
// s_in / s_out (nullable) are [H, D, D] float64 states (the reference test starts from zero).
void orc_gdn_recurrent_f64(const uint16_t* q, const uint16_t* k, const uint16_t* v, const float* g,
                           const uint16_t* beta, double* out, int T, int H, int HK, int D, const double* s_in,
                           double* s_out) {
#pragma omp parallel for schedule(dynamic, 1)
    for (int head = 0; head < H; head++) {
        const int kh = head / (H / HK);
        std::vector<double> s((size_t)D * D, 0.0), qv(D), kv(D), vv(D);
        if (s_in) memcpy(s.data(), s_in + (size_t)head * D * D, sizeof(double) * D * D);
        for (int tok = 0; tok < T; tok++) {
            const uint16_t* qr = q + ((size_t)tok * HK + kh) * D;
            const uint16_t* kr = k + ((size_t)tok * HK + kh) * D;
            double qs = 0, ks = 0;
            for (int i = 0; i < D; i++) {
                qv[i] = bf2f(qr[i]);
                kv[i] = bf2f(kr[i]);
                qs += qv[i] * qv[i];
                ks += kv[i] * kv[i];
            }
            const double qi = 1.0 / sqrt(qs + 1e-6), ki = 1.0 / sqrt(ks + 1e-6), rd = sqrt((double)D);
            for (int i = 0; i < D; i++) {
                qv[i] = qv[i] * qi / rd;
                kv[i] = kv[i] * ki;
                vv[i] = bf2f(v[((size_t)tok * H + head) * D + i]);
            }
            const double decay = exp((double)g[(size_t)tok * H + head]);
            const double b = bf2f(beta[(size_t)tok * H + head]);
            for (size_t i = 0; i < (size_t)D * D; i++) s[i] *= decay;
            // mem_j = sum_i k_i S_ij ; delta_j = (v_j - mem_j) * b ; S_ij += k_i delta_j
            std::vector<double> delta(D, 0.0);
            for (int i = 0; i < D; i++) {
                const double ki2 = kv[i];
                const double* srow = s.data() + (size_t)i * D;
                for (int j = 0; j < D; j++) delta[j] += ki2 * srow[j];
            }
            for (int j = 0; j < D; j++) delta[j] = (vv[j] - delta[j]) * b;
            double* o = out + ((size_t)tok * H + head) * D;
            for (int j = 0; j < D; j++) o[j] = 0;
            for (int i = 0; i < D; i++) {
                double* srow = s.data() + (size_t)i * D;
                const double ki2 = kv[i], qi2 = qv[i];
                for (int j = 0; j < D; j++) {
                    srow[j] += ki2 * delta[j];
                    o[j] += qi2 * srow[j];
                }
            }
        }
        if (s_out) memcpy(s_out + (size_t)head * D * D, s.data(), sizeof(double) * D * D);
    }
}

// Chunked (C = 64) WY-form gated delta rule in float32 with the reference kernels' rounding
// points (gdn_prefill.cu:110-544): bf16 qd, kd, P, T*beta, k*exp(cum), u, w, v_new and the
// chunk-entry state; float32 cumsum, norms, pair products, inverse and state.
// q, k [T, HK, 128]; v, o [T, H, 128]; g float [T, H]; beta bf16 [T, H];
// s_in / s_out (nullable) float32 [H, 128, 128] ([K][V]).
void orc_gdn_chunked(const uint16_t* q, const uint16_t* k, const uint16_t* v, const float* g, const uint16_t* beta,
                     uint16_t* o, int T, int H, int HK, float scale, const float* s_in, float* s_out) {
    const int C = 64, D = 128;
    const int NC = (T + C - 1) / C;
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < H; h++) {
        const int hk = h / (H / HK);
        std::vector<float> S((size_t)D * D, 0.f), Sb((size_t)D * D);
        if (s_in) memcpy(S.data(), s_in + (size_t)h * D * D, sizeof(float) * D * D);
        std::vector<float> kn(C * D), qn(C * D), qd(C * D), kd(C * D), ke(C * D), vv(C * D), A(C * C), P(C * C),
            Tm(C * C), Tb(C * C), u(C * D), w(C * D), vn(C * D);
        float cum[C], bt[C];
        for (int c = 0; c < NC; c++) {
            const int r0 = c * C, n = std::min(C, T - r0);
            float run = 0.f;
            for (int i = 0; i < C; i++) {
                const float gi = i < n ? g[(size_t)(r0 + i) * H + h] : 0.f;
                bt[i] = i < n ? bf2f(beta[(size_t)(r0 + i) * H + h]) : 0.f;
                run += gi;
                cum[i] = run;
            }
            const float last = cum[C - 1], decay = expf(last);
            for (int i = 0; i < C; i++) {
                float qs = 0.f, ks = 0.f;
                for (int d = 0; d < D; d++) {
                    const float qx = i < n ? bf2f(q[((size_t)(r0 + i) * HK + hk) * D + d]) : 0.f;
                    const float kx = i < n ? bf2f(k[((size_t)(r0 + i) * HK + hk) * D + d]) : 0.f;
                    qn[i * D + d] = qx;
                    kn[i * D + d] = kx;
                    qs += qx * qx;
                    ks += kx * kx;
                    vv[i * D + d] = i < n ? bf2f(v[((size_t)(r0 + i) * H + h) * D + d]) : 0.f;
                }
                const float qi = 1.0f / sqrtf(qs + 1e-6f) * scale, ki = 1.0f / sqrtf(ks + 1e-6f);
                const float ec = expf(cum[i]), er = expf(last - cum[i]);
                for (int d = 0; d < D; d++) {
                    qn[i * D + d] *= qi;
                    kn[i * D + d] *= ki;
                    qd[i * D + d] = rbf(qn[i * D + d] * ec);
                    kd[i * D + d] = rbf(kn[i * D + d] * er);
                    ke[i * D + d] = rbf(kn[i * D + d] * ec);
                }
            }
            for (int i = 0; i < C; i++)
                for (int j = 0; j < C; j++) {
                    float kk = 0.f, qk = 0.f;
                    if (j <= i) {
                        for (int d = 0; d < D; d++) {
                            kk += kn[i * D + d] * kn[j * D + d];
                            qk += qn[i * D + d] * kn[j * D + d];
                        }
                    }
                    const float e = j <= i ? expf(cum[i] - cum[j]) : 0.f;
                    A[i * C + j] = j < i ? bt[i] * kk * e : 0.f;
                    P[i * C + j] = j <= i ? rbf(qk * e) : 0.f;
                }
            // Tm = (I + A)^-1 by forward substitution, row by row.
            for (int i = 0; i < C; i++) {
                for (int j = 0; j < C; j++) Tm[i * C + j] = i == j ? 1.f : 0.f;
                for (int m = 0; m < i; m++) {
                    const float a = A[i * C + m];
                    if (a != 0.f)
                        for (int j = 0; j <= m; j++) Tm[i * C + j] -= a * Tm[m * C + j];
                }
            }
            for (int i = 0; i < C; i++)
                for (int j = 0; j < C; j++) Tb[i * C + j] = rbf(Tm[i * C + j] * bt[j]);
            for (int i = 0; i < C; i++)
                for (int d = 0; d < D; d++) {
                    float su = 0.f, sw = 0.f;
                    for (int j = 0; j <= i; j++) {
                        su += Tb[i * C + j] * vv[j * D + d];
                        sw += Tb[i * C + j] * ke[j * D + d];
                    }
                    u[i * D + d] = rbf(su);
                    w[i * D + d] = rbf(sw);
                }
            for (size_t i = 0; i < (size_t)D * D; i++) Sb[i] = rbf(S[i]);
            for (int i = 0; i < C; i++)
                for (int d = 0; d < D; d++) {
                    float s = 0.f;
                    for (int kk = 0; kk < D; kk++) s += w[i * D + kk] * Sb[(size_t)kk * D + d];
                    vn[i * D + d] = rbf(u[i * D + d] - s);
                }
            for (int i = 0; i < n; i++)
                for (int d = 0; d < D; d++) {
                    float s = 0.f;
                    for (int kk = 0; kk < D; kk++) s += qd[i * D + kk] * Sb[(size_t)kk * D + d];
                    for (int j = 0; j <= i; j++) s += P[i * C + j] * vn[j * D + d];
                    o[((size_t)(r0 + i) * H + h) * D + d] = f2bf(s);
                }
            for (int kk = 0; kk < D; kk++)
                for (int d = 0; d < D; d++) {
                    float s = 0.f;
                    for (int i = 0; i < C; i++) s += kd[i * D + kk] * vn[i * D + d];
                    S[(size_t)kk * D + d] = decay * S[(size_t)kk * D + d] + s;
                }
        }
        if (s_out) memcpy(s_out + (size_t)h * D * D, S.data(), sizeof(float) * D * D);
    }
}

// Causal attention with grouped KV heads in float64 (tests/qwen3_5/kernels.rs:434-470).
// q, out [T, Hq, Dh] (float64 out); k [T, Hk, Dh]; v rows of ldv. Only rows [q_base, T) of q
// are read and of out are written, as the windowed entry point of attention.cu:84-100; with
// row_step > 1 only every row_step-th of them and the last one (the reference test samples
// about 64 rows per length the same way).
void orc_attention_f64(const uint16_t* q, const uint16_t* k, const uint16_t* v, int ldv, double* out, int T, int Hq,
                       int Hk, int Dh, double scale, int q_base, int row_step) {
    if (row_step < 1) row_step = 1;
    const int nrows = (T - q_base + row_step - 1) / row_step;
#pragma omp parallel for schedule(dynamic, 4) collapse(2)
    for (int ri = 0; ri <= nrows; ri++) {
        for (int h = 0; h < Hq; h++) {
            // every row_step-th row from q_base, and always the last row (kernels.rs:437)
            const int r = ri < nrows ? q_base + ri * row_step : T - 1;
            if (r < q_base || (ri == nrows && (T - 1 - q_base) % row_step == 0)) continue;
            const int i = r;
            const int gidx = h / (Hq / Hk);
            std::vector<double> s(i + 1), qd(Dh);
            for (int d = 0; d < Dh; d++) qd[d] = bf2f(q[((size_t)r * Hq + h) * Dh + d]);
            double m = -INFINITY;
            for (int j = 0; j <= i; j++) {
                const uint16_t* kj = k + ((size_t)j * Hk + gidx) * Dh;
                double acc = 0;
                for (int d = 0; d < Dh; d++) acc += qd[d] * (double)bf2f(kj[d]);
                s[j] = acc * scale;
                m = std::max(m, s[j]);
            }
            double z = 0;
            for (int j = 0; j <= i; j++) {
                s[j] = exp(s[j] - m);
                z += s[j];
            }
            double* orow = out + ((size_t)r * Hq + h) * Dh;
            for (int d = 0; d < Dh; d++) orow[d] = 0;
            for (int j = 0; j <= i; j++) {
                const uint16_t* vj = v + (size_t)j * ldv + (size_t)gidx * Dh;
                const double wj = s[j];
                for (int d = 0; d < Dh; d++) orow[d] += wj * (double)bf2f(vj[d]);
            }
            for (int d = 0; d < Dh; d++) orow[d] /= z;
        }
    }
}

// bf16 attention output with the optional sigmoid gate epilogue: bf16(bf16(o) * bf16(sigmoid(gate)))
// (attention.cu:223-231), o from the float64 attention above.
void orc_attention(const uint16_t* q, const uint16_t* k, const uint16_t* v, int ldv, const uint16_t* gate,
                   uint16_t* out, int T, int Hq, int Hk, int Dh, float scale, int q_base) {
    const size_t n = (size_t)T * Hq * Dh;
    std::vector<double> o(n, 0.0);
    orc_attention_f64(q, k, v, ldv, o.data(), T, Hq, Hk, Dh, (double)scale, q_base, 1);
    for (size_t i = (size_t)q_base * Hq * Dh; i < n; i++) {
        const float a = rbf((float)o[i]);
        out[i] = gate ? f2bf(a * rbf(sigmoid_f(bf2f(gate[i])))) : f2bf(a);
    }
}

// Open-Jev scalar head: float64 accumulation rounded to float32, then the bias added in
// float32 (src/models/open_jev/native/src/executor.rs:56-68). Returns 0, or 1 if non-finite.
int orc_head_score(const float* weights, const float* last, int n, float bias, float* score) {
    double acc = 0;
    for (int i = 0; i < n; i++) acc += (double)weights[i] * (double)last[i];
    *score = (float)acc + bias;
    return isfinite(*score) ? 0 : 1;
}

// Cua-S1 letter head: one float64-accumulated dot product per option row, rounded to
// float32; rows beyond n_options are not read (src/models/cua_s1/native/src/executor.rs:61-78).
int orc_letter_logits(const float* letters, const float* last, int hidden, int n_options, float* logits) {
    int bad = 0;
    for (int o = 0; o < n_options; o++) {
        double acc = 0;
        for (int i = 0; i < hidden; i++) acc += (double)letters[(size_t)o * hidden + i] * (double)last[i];
        logits[o] = (float)acc;
        if (!isfinite(logits[o])) bad = 1;
    }
    return bad;
}

// Order-preserving packing of candidate prompts: at most 16 sequences and 4096 tokens per
// group, a longer prompt alone (src/models/open_jev/native/src/batching.rs:5-25).
// Writes group start indices to `starts` (capacity n) and returns the group count; group i
// is [starts[i], starts[i+1]) with the last one ending at n.
int orc_batch_ranges(const int* lengths, int n, int* starts) {
    const int MAX_SEQUENCES = 16, MAX_TOKENS = 4096;
    int groups = 0, start = 0;
    long tokens = 0;
    for (int index = 0; index < n; index++) {
        if (index > start && (index - start == MAX_SEQUENCES || tokens + lengths[index] > MAX_TOKENS)) {
            starts[groups++] = start;
            start = index;
            tokens = 0;
        }
        tokens += lengths[index];
    }
    if (start < n) starts[groups++] = start;
    return groups;
}

// Calibrated softmax over (x - max) / T in float64 and the decision: the first maximum
// wins ties (src/models/open_jev/native/src/contract.rs:227-247). Returns the argmax.
int orc_decide(const float* logits, int n, double temperature, double* probs) {
    float mx = -INFINITY;
    for (int i = 0; i < n; i++) mx = std::max(mx, logits[i]);
    double total = 0;
    for (int i = 0; i < n; i++) {
        probs[i] = exp(((double)logits[i] - (double)mx) / temperature);
        total += probs[i];
    }
    for (int i = 0; i < n; i++) probs[i] /= total;
    int mode = 0;
    for (int i = 1; i < n; i++)
        if (probs[i] > probs[mode]) mode = i;
    return mode;
}

// ---- decoder composition (src/models/qwen3_5/native/src/model.rs:1119-1338) ----

struct OrcLayer {
    int full_attention;
    const uint16_t *input_norm, *post_norm, *gate_up, *down;
    // linear attention: in_proj = [qkv | z | b | a] stacked rows
    const uint16_t *in_proj, *conv, *a_log, *dt_bias, *norm, *out_proj;
    // full attention: qkv = [q_proj (q|gate per head) | k_proj | v_proj]
    const uint16_t *qkv, *o_proj, *q_norm, *k_norm;
};

struct OrcModel {
    int hidden, intermediate, n_layers, heads, kv_heads, head_dim, rotary_half;
    int lin_k_heads, lin_v_heads, vocab;
    float eps;
    double rope_theta;
    const uint16_t *embed, *final_norm;
    const OrcLayer* layers;
};

// Prefill of a pack of independent sequences (lengths[nseq], ids concatenated):
// pointwise operators and the input / gate-up GEMMs over the whole pack, conv, delta rule,
// attention (positions restart at 0) per sequence. Writes the final-norm hidden state of
// each sequence's last token as float32 [nseq, hidden]; if layer_out is non-null, also the
// bf16 residual stream after every layer [n_layers, T, hidden]; if x_in is non-null it
// replaces the embedding lookup (bf16 [T, hidden]); max_layers < n_layers truncates
// (the final norm weight is then applied after the last layer run).
void orc_forward(const OrcModel* m, const int32_t* ids, const uint16_t* x_in, const int* lengths, int nseq,
                 int max_layers, float* last_hidden, uint16_t* layer_out) {
    int T = 0;
    for (int s = 0; s < nseq; s++) T += lengths[s];
    const int Hd = m->hidden, I = m->intermediate;
    const int kd = m->lin_k_heads * 128, vd = m->lin_v_heads * 128, hv = m->lin_v_heads;
    const int conv = 2 * kd + vd, gdn_in = conv + vd + 2 * hv;
    const int hq = m->heads, hk = m->kv_heads, dh = m->head_dim;
    const int attn_q = hq * dh * 2, attn_in = attn_q + 2 * hk * dh;
    const int L = std::min(m->n_layers, max_layers);
    typedef std::vector<uint16_t> B;
    B res((size_t)T * Hd), x((size_t)T * Hd), delta((size_t)T * Hd);
    if (x_in)
        memcpy(res.data(), x_in, res.size() * 2);
    else
        orc_embed(ids, m->embed, res.data(), T, Hd);
    int maxlen = 0;
    for (int s = 0; s < nseq; s++) maxlen = std::max(maxlen, lengths[s]);
    std::vector<int64_t> pos(maxlen);
    for (int i = 0; i < maxlen; i++) pos[i] = i;
    B cos_t((size_t)maxlen * m->rotary_half), sin_t((size_t)maxlen * m->rotary_half);
    orc_rotary_tables(pos.data(), maxlen, m->rotary_half, m->rope_theta, cos_t.data(), sin_t.data());
    orc_rms_norm(res.data(), m->layers[0].input_norm, x.data(), T, Hd, m->eps);
    for (int li = 0; li < L; li++) {
        const OrcLayer& ly = m->layers[li];
        if (!ly.full_attention) {
            B gin((size_t)T * gdn_in), lq((size_t)T * kd), lk((size_t)T * kd), lv((size_t)T * vd), lo((size_t)T * vd),
                ln((size_t)T * vd), beta((size_t)T * hv);
            std::vector<float> g((size_t)T * hv);
            orc_gemm(x.data(), ly.in_proj, gin.data(), T, gdn_in, Hd, gdn_in);
            const uint16_t* z = gin.data() + conv;
            const uint16_t* b = z + vd;
            const uint16_t* a = b + hv;
            orc_gdn_gates(b, a, gdn_in, ly.a_log, ly.dt_bias, beta.data(), g.data(), T, hv);
            int off = 0;
            for (int s = 0; s < nseq; s++) {
                const int len = lengths[s];
                orc_gdn_conv(gin.data() + (size_t)off * gdn_in, gdn_in, ly.conv, lq.data() + (size_t)off * kd,
                             lk.data() + (size_t)off * kd, lv.data() + (size_t)off * vd, len, kd, vd);
                orc_gdn_chunked(lq.data() + (size_t)off * kd, lk.data() + (size_t)off * kd, lv.data() + (size_t)off * vd,
                                g.data() + (size_t)off * hv, beta.data() + (size_t)off * hv, lo.data() + (size_t)off * vd,
                                len, hv, m->lin_k_heads, 1.0f / sqrtf(128.f), nullptr, nullptr);
                off += len;
            }
            orc_gated_rms_norm(lo.data(), z, gdn_in, ly.norm, ln.data(), T, hv, 128, m->eps);
            orc_gemm(ln.data(), ly.out_proj, delta.data(), T, Hd, vd, Hd);
        } else {
            B ain((size_t)T * attn_in), aq((size_t)T * hq * dh), ag((size_t)T * hq * dh), ak((size_t)T * hk * dh),
                ao((size_t)T * hq * dh);
            orc_gemm(x.data(), ly.qkv, ain.data(), T, attn_in, Hd, attn_in);
            int off = 0;
            for (int s = 0; s < nseq; s++) {
                const int len = lengths[s];
                const uint16_t* base = ain.data() + (size_t)off * attn_in;
                orc_attn_prep(base, base + attn_q, attn_in, ly.q_norm, ly.k_norm, cos_t.data(), sin_t.data(),
                              aq.data() + (size_t)off * hq * dh, ag.data() + (size_t)off * hq * dh,
                              ak.data() + (size_t)off * hk * dh, len, hq, hk, dh, m->rotary_half, m->eps);
                orc_attention(aq.data() + (size_t)off * hq * dh, ak.data() + (size_t)off * hk * dh,
                              base + attn_q + hk * dh, attn_in, ag.data() + (size_t)off * hq * dh,
                              ao.data() + (size_t)off * hq * dh, len, hq, hk, dh, 1.0f / sqrtf((float)dh), 0);
                off += len;
            }
            orc_gemm(ao.data(), ly.o_proj, delta.data(), T, Hd, hq * dh, Hd);
        }
        orc_add_rms_norm(res.data(), delta.data(), ly.post_norm, x.data(), T, Hd, m->eps);
        {
            B gu((size_t)T * 2 * I), act((size_t)T * I);
            orc_gemm(x.data(), ly.gate_up, gu.data(), T, 2 * I, Hd, 2 * I);
            orc_silu_mul(gu.data(), 2 * I, act.data(), T, I);
            orc_gemm(act.data(), ly.down, delta.data(), T, Hd, I, Hd);
        }
        const uint16_t* next = li + 1 < L ? m->layers[li + 1].input_norm : m->final_norm;
        orc_add_rms_norm(res.data(), delta.data(), next, x.data(), T, Hd, m->eps);
        if (layer_out) memcpy(layer_out + (size_t)li * T * Hd, res.data(), (size_t)T * Hd * 2);
    }
    int end = 0;
    for (int s = 0; s < nseq; s++) {
        end += lengths[s];
        for (int i = 0; i < Hd; i++) last_hidden[(size_t)s * Hd + i] = bf2f(x[(size_t)(end - 1) * Hd + i]);
    }
}

}  // extern "C"
