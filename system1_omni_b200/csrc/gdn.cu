// Chunked (C = 64) WY-form gated delta rule, prefill only, head dim 128.
//
// Two kernels per call:
//   gdn_prep  one block per (chunk, value head), fully parallel: cumulative log-decays, L2
//             norms of q and k, the pair products k.k and q.k on TF32 tensor cores, the
//             triangular inverse T = (I + A)^-1 in float32, u = T beta v and
//             w = T beta exp(cum) k on bf16 tensor cores. Leaves u, w, qd = q exp(cum),
//             kd = k exp(cum_last - cum), P = (q.k) decay-masked and exp(cum_last) in the
//             workspace.
//   gdn_scan  one block per (value head, slice of value columns), sequential over chunks:
//             the state S [128 x slice] stays in float32 registers for the whole sequence
//             with a bf16 copy in shared memory as the tensor-core operand; per chunk
//             v_new = u - w S, o = qd S + P v_new (written straight to the output) and
//             S = decay S + kd^T v_new. Neither S nor v_new ever goes to global memory.
//
// Data movement is by the copy engine: gdn_prep takes its v and k rows as two TMA tiles, and
// leaves every workspace tile in the padded row layout its consumer wants in shared memory, so
// gdn_scan fetches a chunk's five tiles with five bulk copies issued by one thread (per-thread
// 16-byte asynchronous copies held up every later shared-memory access of the block).
//
// Arithmetic and rounding points are those of the reference implementation
// (src/backends/cuda/qwen3_5/gdn_prefill.cu:110-544): float32 cumsum, norms, pair products
// (TF32 operands), inverse and state; bf16 qd, kd, P, T*beta, k*exp(cum), u, w, v_new and
// the chunk-entry state. The state is float32 across calls (s_in / s_out), so a window that
// starts on a multiple of 64 tokens continues a previous one bit for bit.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "cs1_ops.h"
#include "mma.cuh"
#include "tc5.cuh"
#include "tmap.h"

namespace s1 {
namespace {

constexpr int C = 64;   // chunk length
constexpr int D = 128;  // key and value head dim
constexpr int LDF = D + 4;   // float row stride of the TF32 operand tiles
constexpr int LDA = C + 4;   // float row stride of A
constexpr int LDH = D + 8;   // bf16 row stride of [64][128] tiles
constexpr int LDT = C + 8;   // bf16 row stride of [64][64] tiles

// Width of the value-column slice one scan block owns: narrow slices when there are few heads,
// so that the scan still covers the SMs.
inline int slice_width(int H) { return H * (D / 32) >= 96 ? 32 : 16; }

// Workspace: per (head, chunk) tiles in the padded row layouts of the scan's shared memory, each
// tile contiguous so that one bulk copy brings it in.
struct Work {
    bf16* u;       // [H, NC, 128 / VS, 64, VS + 8]  one tile per slice of value columns
    bf16* w;       // [H, NC, 64, LDH]
    bf16* qd;      // [H, NC, 64, LDH]
    bf16* kd;      // [H, NC, 64, LDH]
    bf16* p;       // [H, NC, 64, LDT]
    float* decay;  // [H, NC]
    int vs;        // VS
};

struct Layout {
    size_t u, w, qd, kd, p, decay, total;
    Layout(int T, int H) {
        const size_t NC = ((size_t)T + C - 1) / C;
        const size_t vs = (size_t)slice_width(H);
        size_t at = 0;
        auto take = [&](size_t bytes) {
            const size_t off = at;
            at = (at + bytes + 255) / 256 * 256;
            return off;
        };
        u = take((size_t)H * NC * (D / vs) * C * (vs + 8) * 2);
        w = take((size_t)H * NC * C * LDH * 2);
        qd = take((size_t)H * NC * C * LDH * 2);
        kd = take((size_t)H * NC * C * LDH * 2);
        p = take((size_t)H * NC * C * LDT * 2);
        decay = take((size_t)H * NC * 4);
        total = at;
    }
};

Work split(float* workspace, int T, int H) {
    const Layout l(T, H);
    unsigned char* b = reinterpret_cast<unsigned char*>(workspace);
    Work ws;
    ws.u = reinterpret_cast<bf16*>(b + l.u);
    ws.w = reinterpret_cast<bf16*>(b + l.w);
    ws.qd = reinterpret_cast<bf16*>(b + l.qd);
    ws.kd = reinterpret_cast<bf16*>(b + l.kd);
    ws.p = reinterpret_cast<bf16*>(b + l.p);
    ws.decay = reinterpret_cast<float*>(b + l.decay);
    ws.vs = slice_width(H);
    return ws;
}

__device__ int g_gdn_error = 0;  // a bounded wait for a copy gave up (read with s1_gdn_status)

// ---------------------------------------------------------------------------------------
// gdn_prep
// ---------------------------------------------------------------------------------------
constexpr int PREP_THREADS = 256;
// shared memory map (bytes)
constexpr int P_KF = 0;                          // float [64][LDF]  k normalized, TF32 bits
constexpr int P_QF = P_KF + C * LDF * 4;         // float [64][LDF]  q normalized * scale, TF32 bits
constexpr int P_A = P_QF + C * LDF * 4;          // float [64][LDA]  A
constexpr int P_TB = P_A + C * LDA * 4;          // bf16  [64][LDT]  T * beta
constexpr int P_SM = P_TB + C * LDT * 2;         // float [6][64]    g/cum, beta, ecum, erem, kinv, spare
constexpr int LDX = 36;                          // float row stride of the 32 x 32 temporary of the inverse
constexpr int P_X = P_SM + 6 * C * 4;            // float [32][LDX]
constexpr int PREP_SMEM = P_X + 32 * LDX * 4;
// after the pair products the operand tiles are dead: v and k*exp(cum) reuse them
constexpr int P_VS = P_KF;                       // bf16 [64][LDH]
constexpr int P_VR = P_KF + C * LDH * 2;         // bf16 [64][128] raw v rows as the TMA tile leaves them
constexpr int P_KE = P_QF + C * D * 2;           // bf16 [64][LDH], after the unpadded raw k rows
static_assert(C * LDH * 2 + C * D * 2 <= C * LDF * 4, "padded and raw v tiles fit over the k operand tile");
static_assert(P_VR % 128 == 0 && P_QF % 128 == 0, "TMA destinations are 128-byte aligned");
static_assert(C * D * 2 + C * LDH * 2 <= C * LDF * 4, "raw k rows and k*exp(cum) fit over the q tile");

__global__ void __launch_bounds__(PREP_THREADS, 2)
    gdn_prep(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
             const bf16* __restrict__ q, const bf16* __restrict__ k, const float* __restrict__ g,
             const bf16* __restrict__ beta, Work ws, int T, int H, int HK, float scale) {
    extern __shared__ __align__(128) unsigned char smem[];
    float* kf = reinterpret_cast<float*>(smem + P_KF);
    float* qf = reinterpret_cast<float*>(smem + P_QF);
    float* A = reinterpret_cast<float*>(smem + P_A);
    bf16* Tb = reinterpret_cast<bf16*>(smem + P_TB);
    float* cum = reinterpret_cast<float*>(smem + P_SM);
    float* bt = cum + C;
    float* ecum = bt + C;
    float* erem = ecum + C;
    float* kinv = erem + C;
    uint64_t* tile_bar = reinterpret_cast<uint64_t*>(kinv + C);  // the spare row of the scalar block
    bf16* vs = reinterpret_cast<bf16*>(smem + P_VS);
    bf16* ke = reinterpret_cast<bf16*>(smem + P_KE);

    const int c = blockIdx.x, h = blockIdx.y, hk = h / (H / HK);
    const int NC = gridDim.x;
    const int r0 = c * C, n = min(C, T - r0);
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    if (tid == 0) {
        tc5::mbar_init(tile_bar, 1);
        tc5::mbar_init_fence();
    }
    const size_t tile = (size_t)h * NC + c;  // this block's (head, chunk) tile in every workspace array

    // The q and k rows of the norm phase are requested first of all, so that their latency
    // hides behind the decay phase.
    const int sub = tid & 15, rsel = tid >> 4;
    const int d0 = sub * 4;
    uint2 raw[8][2];
#pragma unroll
    for (int pass = 0; pass < 8; pass++) {
        const int i = (pass & 3) * 16 + rsel;
        raw[pass][0] = raw[pass][1] = make_uint2(0, 0);
        if (i < n) {
            const bf16* src = (pass < 4 ? k : q) + ((size_t)(r0 + i) * HK + hk) * D + d0;
            raw[pass][0] = *reinterpret_cast<const uint2*>(src);
            raw[pass][1] = *reinterpret_cast<const uint2*>(src + 64);
        }
    }

    // ---- log-decays: sequential float32 prefix sum, rows past the end have g = beta = 0 ----
    if (tid < C) {
        cum[tid] = tid < n ? g[(size_t)(r0 + tid) * H + h] : 0.f;
        bt[tid] = tid < n ? f32(beta[(size_t)(r0 + tid) * H + h]) : 0.f;
    }
    __syncthreads();
    if (tid == 0) {
        // in registers: 16 wide loads, 64 dependent adds, 16 wide stores
        float4 part[C / 4];
#pragma unroll
        for (int i = 0; i < C / 4; i++) part[i] = reinterpret_cast<const float4*>(cum)[i];
        float run = 0.f;
#pragma unroll
        for (int i = 0; i < C / 4; i++) {
            part[i].x = (run += part[i].x);
            part[i].y = (run += part[i].y);
            part[i].z = (run += part[i].z);
            part[i].w = (run += part[i].w);
        }
#pragma unroll
        for (int i = 0; i < C / 4; i++) reinterpret_cast<float4*>(cum)[i] = part[i];
    }
    __syncthreads();
    if (tid < C) {
        const float last = cum[C - 1];
        ecum[tid] = expf(cum[tid]);
        erem[tid] = expf(last - cum[tid]);
        if (tid == 0) ws.decay[(size_t)h * NC + c] = expf(last);
    }
    __syncthreads();

    // ---- L2 norms; TF32 operand tiles; qd and kd to the workspace ----
    {
        // 16 lanes per row, 16 rows per pass; a lane owns dims [4 sub, 4 sub + 4) and
        // [64 + 4 sub, 64 + 4 sub + 4), so that the float4 stores of a quarter warp fall in one
        // contiguous 128-byte run of shared memory. All 16 loads are requested up front.
        bf16* qd_out = ws.qd + tile * (C * LDH);
        bf16* kd_out = ws.kd + tile * (C * LDH);
#pragma unroll
        for (int pass = 0; pass < 8; pass++) {
            const bool is_k = pass < 4;
            const int i = (pass & 3) * 16 + rsel;
            float x[8];
#pragma unroll
            for (int half = 0; half < 2; half++) {
                x[4 * half + 0] = __uint_as_float(raw[pass][half].x << 16);
                x[4 * half + 1] = __uint_as_float(raw[pass][half].x & 0xffff0000u);
                x[4 * half + 2] = __uint_as_float(raw[pass][half].y << 16);
                x[4 * half + 3] = __uint_as_float(raw[pass][half].y & 0xffff0000u);
            }
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < 8; e++) ss += x[e] * x[e];
            ss = warp_sum<16>(ss);
            float inv = rsqrtf(ss + 1e-6f);
            if (is_k) {
                if (sub == 0) kinv[i] = inv;
            } else {
                inv *= scale;
            }
            const float mult = is_k ? erem[i] : ecum[i];
            float* tile = (is_k ? kf : qf) + i * LDF;
            bf16* dout = (is_k ? kd_out : qd_out) + i * LDH;
#pragma unroll
            for (int half = 0; half < 2; half++) {
                float4 t;
                float nrm[4];
#pragma unroll
                for (int e = 0; e < 4; e++) nrm[e] = x[4 * half + e] * inv;
                t.x = __uint_as_float(to_tf32(nrm[0]));
                t.y = __uint_as_float(to_tf32(nrm[1]));
                t.z = __uint_as_float(to_tf32(nrm[2]));
                t.w = __uint_as_float(to_tf32(nrm[3]));
                *reinterpret_cast<float4*>(tile + 64 * half + d0) = t;
                uint2 o;
                o.x = pack2(nrm[0] * mult, nrm[1] * mult);
                o.y = pack2(nrm[2] * mult, nrm[3] * mult);
                *reinterpret_cast<uint2*>(dout + 64 * half + d0) = o;
            }
        }
    }
    __syncthreads();

    // ---- pair products on TF32 tensor cores: warps 0-3 k.k -> A, warps 4-7 q.k -> P ----
    {
        const int mt = warp & 3;
        const bool is_kk = warp < 4;
        const float* am = is_kk ? kf : qf;
        const int gq = lane / 4, tq = lane % 4;
        const int ntiles = 2 * mt + 2;  // 8-column tiles up to and including the diagonal block
        float acc[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
        for (int k0 = 0; k0 < D; k0 += 8) {
            uint32_t a[4];
            a[0] = __float_as_uint(am[(mt * 16 + gq) * LDF + k0 + tq]);
            a[1] = __float_as_uint(am[(mt * 16 + gq + 8) * LDF + k0 + tq]);
            a[2] = __float_as_uint(am[(mt * 16 + gq) * LDF + k0 + tq + 4]);
            a[3] = __float_as_uint(am[(mt * 16 + gq + 8) * LDF + k0 + tq + 4]);
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                if (nt < ntiles) {
                    const uint32_t b0 = __float_as_uint(kf[(nt * 8 + gq) * LDF + k0 + tq]);
                    const uint32_t b1 = __float_as_uint(kf[(nt * 8 + gq) * LDF + k0 + tq + 4]);
                    mma_tf32(acc[nt], a, b0, b1);
                }
            }
        }
        bf16* p_out = ws.p + tile * (C * LDT);
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const int i = mt * 16 + gq + r * 8;
                const int j = nt * 8 + 2 * tq;
                float v0 = 0.f, v1 = 0.f;
                if (nt < ntiles) {
                    const float ci = cum[i];
                    const float e0 = expf(ci - cum[j]), e1 = expf(ci - cum[j + 1]);
                    if (is_kk) {
                        v0 = j < i ? bt[i] * acc[nt][2 * r] * e0 : 0.f;
                        v1 = j + 1 < i ? bt[i] * acc[nt][2 * r + 1] * e1 : 0.f;
                    } else {
                        v0 = j <= i ? acc[nt][2 * r] * e0 : 0.f;
                        v1 = j + 1 <= i ? acc[nt][2 * r + 1] * e1 : 0.f;
                    }
                }
                if (is_kk) {
                    A[i * LDA + j] = v0;
                    A[i * LDA + j + 1] = v1;
                } else {
                    *reinterpret_cast<uint32_t*>(p_out + i * LDT + j) = pack2(v0, v1);
                }
            }
        }
    }
    __syncthreads();

    // ---- v and the raw k rows come in as two TMA tiles over the dead operand tiles (rows past the
    //      end of the sequence read as zero) ----
    bf16* kraw = reinterpret_cast<bf16*>(smem + P_QF);  // [64][128], no padding
    bf16* vraw = reinterpret_cast<bf16*>(smem + P_VR);  // [64][128], no padding
    if (tid == 0) {
        tc5::mbar_expect_tx(tile_bar, 2 * C * D * 2);
        tc5::tma_load_2d(kraw, &map_k, hk * D, r0, tile_bar);
        tc5::tma_load_2d(vraw, &map_v, h * D, r0, tile_bar);
    }

    // ---- T = (I + A)^-1 (unit lower triangular, float32), in place over A, while the copies land:
    //      the four 16 x 16 diagonal blocks by forward substitution (one column per thread), then the
    //      blocks below them from T21 = -T22 (A21 T11), first 16 -> 32, then 32 -> 64, as plain
    //      float32 products spread over all 256 threads. A is zero on and above its diagonal. ----
    {
        float* X = reinterpret_cast<float*>(smem + P_X);  // [32][LDX]
        float col[16];
        if (tid < 64) {
            const float* blk = A + (16 * (tid >> 4)) * (LDA + 1);
            const int j = tid & 15;
#pragma unroll
            for (int i = 0; i < 16; i++) {
                float acc = i == j ? 1.f : 0.f;
#pragma unroll
                for (int m = 0; m < i; m++) acc -= blk[i * LDA + m] * col[m];  // col[m] is 0 above the diagonal
                col[i] = acc;
            }
        }
        __syncthreads();  // every column of a block is computed before any is written over A
        if (tid < 64) {
            float* blk = A + (16 * (tid >> 4)) * (LDA + 1);
            const int j = tid & 15;
#pragma unroll
            for (int i = 0; i < 16; i++) blk[i * LDA + j] = col[i];
        }
        __syncthreads();
        {   // 16 -> 32: two independent pairs of diagonal blocks; 2 x 256 outputs, two per thread
            const int p = tid >> 7, idx = tid & 127, i = idx >> 3, j0 = (idx & 7) * 2;
            float* t11 = A + (32 * p) * (LDA + 1);
            float* a21 = t11 + 16 * LDA;
            const float* t22 = a21 + 16;
            float x0 = 0.f, x1 = 0.f;
#pragma unroll
            for (int m = 0; m < 16; m++) {
                const float a = a21[i * LDA + m];
                const float2 t = *reinterpret_cast<const float2*>(t11 + m * LDA + j0);
                x0 += a * t.x;
                x1 += a * t.y;
            }
            *reinterpret_cast<float2*>(X + (16 * p + i) * LDX + j0) = make_float2(x0, x1);
            __syncthreads();
            float y0 = 0.f, y1 = 0.f;
#pragma unroll
            for (int m = 0; m < 16; m++) {
                const float a = t22[i * LDA + m];
                const float2 t = *reinterpret_cast<const float2*>(X + (16 * p + m) * LDX + j0);
                y0 -= a * t.x;
                y1 -= a * t.y;
            }
            *reinterpret_cast<float2*>(a21 + i * LDA + j0) = make_float2(y0, y1);
            __syncthreads();
        }
        {   // 32 -> 64: 32 x 32 outputs, four per thread
            const int i = tid >> 3, j0 = (tid & 7) * 4;
            float* a21 = A + 32 * LDA;
            const float* t22 = a21 + 32;
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
            for (int m = 0; m < 32; m++) {
                const float a = a21[i * LDA + m];
                const float4 t = *reinterpret_cast<const float4*>(A + m * LDA + j0);
                x.x += a * t.x, x.y += a * t.y, x.z += a * t.z, x.w += a * t.w;
            }
            *reinterpret_cast<float4*>(X + i * LDX + j0) = x;
            __syncthreads();
            float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
            for (int m = 0; m < 32; m++) {
                const float a = t22[i * LDA + m];
                const float4 t = *reinterpret_cast<const float4*>(X + m * LDX + j0);
                y.x -= a * t.x, y.y -= a * t.y, y.z -= a * t.z, y.w -= a * t.w;
            }
            *reinterpret_cast<float4*>(a21 + i * LDA + j0) = y;
            __syncthreads();
        }
        // T beta as the bf16 operand of the two products below
#pragma unroll
        for (int e = 0; e < C * C / PREP_THREADS; e++) {
            const int idx = tid + e * PREP_THREADS, i = idx >> 6, j = idx & 63;
            Tb[i * LDT + j] = to_bf16(A[i * LDA + j] * bt[j]);
        }
    }
    {
        volatile int never = 0;
        if (!tc5::mbar_wait(tile_bar, 0, &never)) atomicCAS(&g_gdn_error, 0, 41);  // carries on with what is there
    }
#pragma unroll
    for (int piece = 0; piece < 4; piece++) {  // k * exp(cum) in bf16, and v into its padded tile
        const int cidx = tid + piece * PREP_THREADS;
        const int i = cidx / (D / 8), d0 = (cidx % (D / 8)) * 8;
        float x[8], y[8];
        unpack8(ld16(kraw + i * D + d0), x);
        const float inv = kinv[i], ec = ecum[i];
#pragma unroll
        for (int e = 0; e < 8; e++) y[e] = (x[e] * inv) * ec;
        st16(ke + i * LDH + d0, pack8(y));
        st16(vs + i * LDH + d0, ld16(vraw + i * D + d0));
    }
    __syncthreads();

    // ---- u = (T beta) v (warps 0-3), w = (T beta) (k exp(cum)) (warps 4-7), bf16 tensor cores ----
    {
        const int mt = warp & 3;
        const bool is_u = warp < 4;
        const bf16* bm = is_u ? vs : ke;
        float acc[16][4];
#pragma unroll
        for (int nt = 0; nt < 16; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < C / 16; kk++) {
            uint32_t a[4];
            load_a_rm(a, Tb, LDT, mt * 16, kk * 16, lane);
#pragma unroll
            for (int np = 0; np < 8; np++) {
                uint32_t b[4];
                load_b_kn(b, bm, LDH, kk * 16, np * 16, lane);
                mma_bf16(acc[2 * np], a, b[0], b[1]);
                mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
            }
        }
        // w: one [64][LDH] tile; u: one [64][VS + 8] tile per slice of VS value columns
        const int vs_w = ws.vs, ldu = vs_w + 8;
        bf16* dst = is_u ? ws.u + tile * (size_t)(D / vs_w) * (C * ldu) : ws.w + tile * (C * LDH);
        const int gq = lane / 4, tq = lane % 4;
#pragma unroll
        for (int nt = 0; nt < 16; nt++) {
            const int col = nt * 8 + 2 * tq;
            bf16* at = is_u ? dst + (col / vs_w) * (C * ldu) + (col % vs_w) : dst + col;
            const int ld = is_u ? ldu : LDH;
            *reinterpret_cast<uint32_t*>(at + (mt * 16 + gq) * ld) = pack2(acc[nt][0], acc[nt][1]);
            *reinterpret_cast<uint32_t*>(at + (mt * 16 + gq + 8) * ld) = pack2(acc[nt][2], acc[nt][3]);
        }
    }
}

// ---------------------------------------------------------------------------------------
// gdn_scan
// ---------------------------------------------------------------------------------------

template <int VS>
struct ScanSmem {
    static constexpr int LDV = VS + 8;  // bf16 row stride of [*][VS] tiles
    static constexpr int W = 0;                                // [2][64][LDH]
    static constexpr int U = W + 2 * C * LDH * 2;              // [2][64][LDV]
    static constexpr int QD = U + 2 * C * LDV * 2;             // [64][LDH]
    static constexpr int KD = QD + C * LDH * 2;                // [64][LDH]
    static constexpr int P = KD + C * LDH * 2;                 // [64][LDT]
    static constexpr int SB = P + C * LDT * 2;                 // [128][LDV]
    static constexpr int VN = SB + D * LDV * 2;                // [64][LDV]
    static constexpr int BAR = VN + C * LDV * 2;               // three mbarriers and a flag
    static constexpr int BYTES = BAR + 32;
};

// WARPS is 4 or 8. The 64 chunk rows split into four 16-row tiles (rt); with 8 warps the
// slice's columns additionally split into two halves (cb) for the row products, and the 128
// state rows split 16 per warp instead of 32.
template <int VS, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 2)
    gdn_scan(Work ws, bf16* __restrict__ o, int T, int H, int NC, const float* __restrict__ s_in,
             float* __restrict__ s_out) {
    using L = ScanSmem<VS>;
    constexpr int LDV = L::LDV;
    constexpr int NT = VS / 8;               // 8-column tiles across the slice
    constexpr int THREADS = WARPS * 32;
    constexpr int MT = 8 / WARPS;            // 16-row tiles of the state per warp
    constexpr int NTL = NT / (WARPS / 4);    // column tiles per warp in the row products
    static_assert(NTL >= 2 && NTL % 2 == 0, "column tiles are loaded in pairs");
    extern __shared__ __align__(128) unsigned char smem[];
    bf16* Wb = reinterpret_cast<bf16*>(smem + L::W);
    bf16* Ub = reinterpret_cast<bf16*>(smem + L::U);
    bf16* QDb = reinterpret_cast<bf16*>(smem + L::QD);
    bf16* KDb = reinterpret_cast<bf16*>(smem + L::KD);
    bf16* Pb = reinterpret_cast<bf16*>(smem + L::P);
    bf16* Sb = reinterpret_cast<bf16*>(smem + L::SB);
    bf16* VNb = reinterpret_cast<bf16*>(smem + L::VN);
    uint64_t* wu_bar = reinterpret_cast<uint64_t*>(smem + L::BAR);  // [2], one per buffer of w and u
    uint64_t* qpk_bar = wu_bar + 2;
    volatile int* gave_up = reinterpret_cast<volatile int*>(qpk_bar + 1);

    const int h = blockIdx.x, v0 = blockIdx.y * VS;
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int gq = lane / 4, tq = lane % 4;
    const int rt = warp & 3, cb = (warp >> 2) * NTL * 8;

    // this head's tiles; every tile is contiguous and already in the shared-memory row layout
    constexpr uint32_t W_BYTES = C * LDH * 2, U_BYTES = C * LDV * 2, P_BYTES = C * LDT * 2;
    const bf16* w_g = ws.w + (size_t)h * NC * (C * LDH);
    const bf16* u_g = ws.u + ((size_t)h * NC * (D / VS) + blockIdx.y) * (C * LDV);
    const bf16* qd_g = ws.qd + (size_t)h * NC * (C * LDH);
    const bf16* kd_g = ws.kd + (size_t)h * NC * (C * LDH);
    const bf16* p_g = ws.p + (size_t)h * NC * (C * LDT);
    const float* decay_g = ws.decay + (size_t)h * NC;

    if (tid == 0) {
        tc5::mbar_init(&wu_bar[0], 1);
        tc5::mbar_init(&wu_bar[1], 1);
        tc5::mbar_init(qpk_bar, 1);
        *gave_up = 0;
        tc5::mbar_init_fence();
    }
    __syncthreads();
    // Issued by one thread: two bulk copies (w, u) into buffer c & 1, three (qd, kd, P) into the
    // single buffer of the second half of a chunk step.
    auto load_wu = [&](int c) {
        uint64_t* bar = &wu_bar[c & 1];
        tc5::mbar_expect_tx(bar, W_BYTES + U_BYTES);
        tc5::bulk_load(Wb + (c & 1) * C * LDH, w_g + (size_t)c * (C * LDH), W_BYTES, bar);
        tc5::bulk_load(Ub + (c & 1) * C * LDV, u_g + (size_t)c * (D / VS) * (C * LDV), U_BYTES, bar);
    };
    auto load_qpk = [&](int c) {
        tc5::mbar_expect_tx(qpk_bar, 2 * W_BYTES + P_BYTES);
        tc5::bulk_load(QDb, qd_g + (size_t)c * (C * LDH), W_BYTES, qpk_bar);
        tc5::bulk_load(KDb, kd_g + (size_t)c * (C * LDH), W_BYTES, qpk_bar);
        tc5::bulk_load(Pb, p_g + (size_t)c * (C * LDT), P_BYTES, qpk_bar);
    };
    // A wait that runs out records it and lets the block finish its steps (on whatever is there).
    auto wait_for = [&](uint64_t* bar, uint32_t parity) {
        if (!tc5::mbar_wait(bar, parity, gave_up)) {
            atomicCAS(&g_gdn_error, 0, 42);
            *gave_up = 1;
        }
    };

    if (tid == 0) {
        load_wu(0);
        load_qpk(0);
    }

    // state rows [32 warp, 32 warp + 32) x VS columns, float32, in mma accumulator layout
    float S[MT][NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int kr = warp * (MT * 16) + mt * 16 + gq + (e >> 1) * 8;
                const int vc = v0 + nt * 8 + 2 * tq + (e & 1);
                S[mt][nt][e] = s_in ? s_in[((size_t)h * D + kr) * D + vc] : 0.f;
            }

    for (int c = 0; c < NC; c++) {
        // (1) bf16 copy of the chunk-entry state
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int kr = warp * (MT * 16) + mt * 16 + gq, vc = nt * 8 + 2 * tq;
                *reinterpret_cast<uint32_t*>(Sb + kr * LDV + vc) = pack2(S[mt][nt][0], S[mt][nt][1]);
                *reinterpret_cast<uint32_t*>(Sb + (kr + 8) * LDV + vc) = pack2(S[mt][nt][2], S[mt][nt][3]);
            }
        wait_for(&wu_bar[c & 1], (c >> 1) & 1);  // w, u of this chunk have landed
        __syncthreads();                          // and nobody still reads the other buffer
        if (tid == 0 && c + 1 < NC) load_wu(c + 1);

        const bf16* Wc = Wb + (c & 1) * C * LDH;
        const bf16* Uc = Ub + (c & 1) * C * LDV;
        const float decay = decay_g[c];

        // (2) v_new = u - w S
        {
            float acc[NTL][4];
#pragma unroll
            for (int nt = 0; nt < NTL; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < D / 16; kk++) {
                uint32_t a[4];
                load_a_rm(a, Wc, LDH, rt * 16, kk * 16, lane);
#pragma unroll
                for (int np = 0; np < NTL / 2; np++) {
                    uint32_t b[4];
                    load_b_kn(b, Sb, LDV, kk * 16, cb + np * 16, lane);
                    mma_bf16(acc[2 * np], a, b[0], b[1]);
                    mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
                }
            }
#pragma unroll
            for (int nt = 0; nt < NTL; nt++) {
                const int r = rt * 16 + gq, vc = cb + nt * 8 + 2 * tq;
                const uint32_t u0 = *reinterpret_cast<const uint32_t*>(Uc + r * LDV + vc);
                const uint32_t u1 = *reinterpret_cast<const uint32_t*>(Uc + (r + 8) * LDV + vc);
                *reinterpret_cast<uint32_t*>(VNb + r * LDV + vc) =
                    pack2(__uint_as_float(u0 << 16) - acc[nt][0], __uint_as_float(u0 & 0xffff0000u) - acc[nt][1]);
                *reinterpret_cast<uint32_t*>(VNb + (r + 8) * LDV + vc) =
                    pack2(__uint_as_float(u1 << 16) - acc[nt][2], __uint_as_float(u1 & 0xffff0000u) - acc[nt][3]);
            }
        }
        wait_for(qpk_bar, c & 1);  // qd, kd, P of this chunk have landed
        __syncthreads();

        // (3) o = qd S + P v_new
        {
            float acc[NTL][4];
#pragma unroll
            for (int nt = 0; nt < NTL; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < D / 16; kk++) {
                uint32_t a[4];
                load_a_rm(a, QDb, LDH, rt * 16, kk * 16, lane);
#pragma unroll
                for (int np = 0; np < NTL / 2; np++) {
                    uint32_t b[4];
                    load_b_kn(b, Sb, LDV, kk * 16, cb + np * 16, lane);
                    mma_bf16(acc[2 * np], a, b[0], b[1]);
                    mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
                }
            }
#pragma unroll
            for (int kk = 0; kk < C / 16; kk++) {
                uint32_t a[4];
                load_a_rm(a, Pb, LDT, rt * 16, kk * 16, lane);
#pragma unroll
                for (int np = 0; np < NTL / 2; np++) {
                    uint32_t b[4];
                    load_b_kn(b, VNb, LDV, kk * 16, cb + np * 16, lane);
                    mma_bf16(acc[2 * np], a, b[0], b[1]);
                    mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
                }
            }
            const int row = c * C + rt * 16 + gq;
#pragma unroll
            for (int nt = 0; nt < NTL; nt++) {
                const int vc = v0 + cb + nt * 8 + 2 * tq;
                if (row < T)
                    *reinterpret_cast<uint32_t*>(o + ((size_t)row * H + h) * D + vc) = pack2(acc[nt][0], acc[nt][1]);
                if (row + 8 < T)
                    *reinterpret_cast<uint32_t*>(o + ((size_t)(row + 8) * H + h) * D + vc) =
                        pack2(acc[nt][2], acc[nt][3]);
            }
        }

        // (4) S = decay S + kd^T v_new
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) S[mt][nt][e] *= decay;
#pragma unroll
        for (int kk = 0; kk < C / 16; kk++) {
            uint32_t b[NT / 2][4];
#pragma unroll
            for (int np = 0; np < NT / 2; np++) load_b_kn(b[np], VNb, LDV, kk * 16, np * 16, lane);
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                uint32_t a[4];
                load_a_tr(a, KDb, LDH, warp * (MT * 16) + mt * 16, kk * 16, lane);
#pragma unroll
                for (int np = 0; np < NT / 2; np++) {
                    mma_bf16(S[mt][2 * np], a, b[np][0], b[np][1]);
                    mma_bf16(S[mt][2 * np + 1], a, b[np][2], b[np][3]);
                }
            }
        }
        __syncthreads();  // all reads of this chunk's tiles are done
        if (tid == 0 && c + 1 < NC) load_qpk(c + 1);
    }

    if (s_out) {
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int kr = warp * (MT * 16) + mt * 16 + gq + (e >> 1) * 8;
                    const int vc = v0 + nt * 8 + 2 * tq + (e & 1);
                    s_out[((size_t)h * D + kr) * D + vc] = S[mt][nt][e];
                }
    }
}

template <typename F>
cudaError_t set_smem_once(F* kernel, int bytes, bool* done_per_device) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 64) return cudaErrorInvalidDevice;
    if (done_per_device[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) done_per_device[dev] = true;
    return e;
}

int gdn_run(const void* q, const void* k, const void* v, const float* g, const void* beta, void* o,
            float* workspace, int T, int H, int HK, float scale, const void* s_in, void* s_out, void* stream) {
    if (T < 0 || H <= 0 || HK <= 0 || H % HK != 0) return cudaErrorInvalidValue;
    const float* si = static_cast<const float*>(s_in);
    float* so = static_cast<float*>(s_out);
    cudaStream_t st = as_stream(stream);
    if (T == 0) {
        // no tokens: the state passes through unchanged
        if (so == nullptr) return cudaSuccess;
        const size_t bytes = (size_t)H * D * D * sizeof(float);
        return si != nullptr ? cudaMemcpyAsync(so, si, bytes, cudaMemcpyDeviceToDevice, st)
                             : cudaMemsetAsync(so, 0, bytes, st);
    }
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(workspace) ||
        (reinterpret_cast<uintptr_t>(o) & 3))
        return cudaErrorInvalidValue;
    static bool prep_done[64] = {}, scan16_done[64] = {}, scan32_done[64] = {};
    cudaError_t e = set_smem_once(gdn_prep, PREP_SMEM, prep_done);
    if (e != cudaSuccess) return e;
    const int NC = (T + C - 1) / C;
    const Work ws = split(workspace, T, H);
    // v and k rows of a chunk as [64 rows, 128 columns] tiles of the caller's [T, heads, 128] arrays
    CUtensorMap map_k, map_v;
    if (!tensor_map_2d_plain(k, (uint64_t)T, (uint64_t)HK * D, (uint64_t)HK * D, C, D, &map_k) ||
        !tensor_map_2d_plain(v, (uint64_t)T, (uint64_t)H * D, (uint64_t)H * D, C, D, &map_v))
        return CS1_ERR_TENSOR_MAP;
    gdn_prep<<<dim3(NC, H), PREP_THREADS, PREP_SMEM, st>>>(map_k, map_v, static_cast<const bf16*>(q),
                                                          static_cast<const bf16*>(k), g,
                                                          static_cast<const bf16*>(beta), ws, T, H, HK, scale);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (ws.vs == 32) {
        e = set_smem_once(gdn_scan<32, 8>, ScanSmem<32>::BYTES, scan32_done);
        if (e != cudaSuccess) return e;
        gdn_scan<32, 8><<<dim3(H, D / 32), 256, ScanSmem<32>::BYTES, st>>>(ws, static_cast<bf16*>(o), T, H, NC, si, so);
    } else {
        e = set_smem_once(gdn_scan<16, 4>, ScanSmem<16>::BYTES, scan16_done);
        if (e != cudaSuccess) return e;
        gdn_scan<16, 4><<<dim3(H, D / 16), 128, ScanSmem<16>::BYTES, st>>>(ws, static_cast<bf16*>(o), T, H, NC, si, so);
    }
    return cudaGetLastError();
}

}  // namespace
}  // namespace s1

using namespace s1;

// The device error word of the delta-rule kernels on the current device (0 = no bounded wait for
// a copy ever gave up) after waiting for all queued work; cleared by the call.
extern "C" int s1_gdn_status(int* code) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return e;
    int v = 0;
    e = cudaMemcpyFromSymbol(&v, s1::g_gdn_error, sizeof(int));
    if (e != cudaSuccess) return e;
    if (v != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(s1::g_gdn_error, &zero, sizeof(int));
    }
    *code = v;
    return e;
}

extern "C" size_t cs1_gdn_workspace_floats(int T, int H) {
    if (T < 0 || H < 0) return 0;
    return (Layout(T, H).total + 3) / 4;
}

extern "C" int cs1_gdn_prefill(const void* q, const void* k, const void* v, const float* g, const void* beta, void* o,
                               float* workspace, int T, int H, int HK, float scale, void* stream) {
    return gdn_run(q, k, v, g, beta, o, workspace, T, H, HK, scale, nullptr, nullptr, stream);
}

extern "C" int cs1_gdn_prefill_x(const void* q, const void* k, const void* v, const float* g, const void* beta,
                                 void* o, float* workspace, int T, int H, int HK, float scale, const void* s_in,
                                 void* s_out, void* stream) {
    return gdn_run(q, k, v, g, beta, o, workspace, T, H, HK, scale, s_in, s_out, stream);
}

// ---------------------------------------------------------------------------------------
// cs1_gdn_prefill_static: the same delta rule for callers that cannot hand over scratch
// ---------------------------------------------------------------------------------------
// Some hosts of this library have no way to give cs1_gdn_prefill its workspace: a worker
// that received a fixed set of device buffers from another runtime and is not allowed to
// grow it, a plugin slot inside a serving process whose memory pool belongs to the host
// framework, or code on a path where cudaMalloc is off limits because it synchronises the
// whole device. For them this entry point keeps the workspace inside the library, in a
// fixed array in device memory that exists once per GPU for as long as the library is
// loaded. It allocates nothing: no cudaMalloc, no cudaFree, no library call that allocates.
//
// Limits and rules, all consequences of the array being one fixed, shared block:
//   * the window must fit: cs1_gdn_workspace_floats(T, H) * 4 <= CS1_GDN_STATIC_SCRATCH_BYTES
//     (64 MiB: for example 1600 tokens at 32 value heads, 1088 at 48, 3072 at 16); anything
//     larger is refused with CS1_ERR_STATIC_SCRATCH before any launch;
//   * every call on a GPU uses the same bytes, so two calls that may run at the same time
//     on one GPU (different streams, or different threads) race on it; calls on one stream
//     are ordered and safe;
//   * the array still holds what the previous call left there. Nothing in it needs to start
//     at zero: the first kernel of a call writes every byte the second one reads, including
//     the rows that pad the last chunk;
//   * the first call on each GPU looks up the array's device address (the name below is only
//     a host-side handle, not an address a kernel could use) with that GPU current. Make
//     that first call before any stream capture begins.
static __device__ __align__(256) unsigned char g_gdn_static_scratch[CS1_GDN_STATIC_SCRATCH_BYTES];

namespace {

// Device address of the array for the current device, resolved on first use.
int static_scratch_address(float** out) {
    static float* address[64] = {};
    static std::mutex lock;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> hold(lock);
    if (address[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_gdn_static_scratch);
        if (e != cudaSuccess) return e;
        if (p == nullptr) return cudaErrorInvalidSymbol;
        address[dev] = static_cast<float*>(p);
    }
    *out = address[dev];
    return 0;
}

}  // namespace

extern "C" int cs1_gdn_prefill_static(const void* q, const void* k, const void* v, const float* g, const void* beta,
                                      void* o, int T, int H, int HK, float scale, void* stream) {
    if (T < 0 || H <= 0 || HK <= 0 || H % HK != 0) return cudaErrorInvalidValue;
    if (T == 0) return cudaSuccess;
    if (s1::Layout(T, H).total > (size_t)CS1_GDN_STATIC_SCRATCH_BYTES) return CS1_ERR_STATIC_SCRATCH;
    float* scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != 0) return rc;
    return s1::gdn_run(q, k, v, g, beta, o, scratch, T, H, HK, scale, nullptr, nullptr, stream);
}
