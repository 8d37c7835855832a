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
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "cs1_ops.h"
#include "mma.cuh"
#include "status.h"
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
// gdn_prep_tc5: the same work with the dense products on tcgen05, two chunks (128 rows) of one
// value head per block. The pair products k.k and q.k are two 128 x 128 x 128 TF32 MMAs whose
// operands the norm phase writes straight into the swizzled K-major layout (only the two 64 x 64
// diagonal blocks of each result are used); u and w are one 128 x 256 x 128 bf16 MMA of the
// block-diagonal T beta with [v | k exp(cum)], v arriving as a TMA tile and read MN-major. The
// results come back through tensor memory, one row per thread. Everything between - decays,
// norms, masks, the triangular inverse - is the float32 code of gdn_prep on twice the rows.
// ---------------------------------------------------------------------------------------
constexpr int R2 = 2 * C;                        // rows per block
constexpr int BOX = R2 * 128;                    // bytes of one [128 rows x 128 bytes] swizzled box
constexpr int T_KF = 0;                          // float, 4 boxes of 32 columns: k normalised (TF32 bits)
constexpr int T_QF = T_KF + 4 * BOX;             // float, 4 boxes: q normalised * scale (TF32 bits)
constexpr int T_KE = T_QF + 4 * BOX;             // bf16, 2 boxes of 64 columns: k exp(cum)
constexpr int T_A = T_KE + 2 * BOX;              // float [128][LDA]: A, then T, block by chunk
constexpr int T_X = T_A + R2 * LDA * 4;          // float [2][32][LDX]: temporaries of the two inverses
constexpr int T_SM = T_X + 2 * 32 * LDX * 4;     // float [4][128]: cum, beta, exp(cum), exp(cum_last - cum)
constexpr int T_BAR = T_SM + 4 * R2 * 4;         // three mbarriers, the tensor-memory address, a flag
constexpr int PREP2_SMEM = T_BAR + 64 + 1024;    // + slack to align the base to 1024
// once the pair products are done, over their operands:
constexpr int T_TB = T_KF;                       // bf16, 2 boxes of 64 k-columns: T beta (block diagonal)
constexpr int T_VB = T_QF + 2 * BOX;             // bf16, 2 boxes of 64 columns: v, as TMA leaves it; T_KE follows
static_assert(T_VB + 2 * BOX == T_KE, "v and k exp(cum) form one MN-major operand of four boxes");
constexpr int PREP2_THREADS = 512;  // 16 warps: the float32 phases between the MMAs need the threads

__global__ void __launch_bounds__(PREP2_THREADS, 1)
    gdn_prep_tc5(const __grid_constant__ CUtensorMap map_v, const bf16* __restrict__ q, const bf16* __restrict__ k,
                 const float* __restrict__ g, const bf16* __restrict__ beta, Work ws, int T, int H, int HK, int NC,
                 float scale) {
    using namespace tc5;
    grid_dep_trigger();
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    float* A = reinterpret_cast<float*>(smem + T_A);
    float* cum = reinterpret_cast<float*>(smem + T_SM);
    float* bt = cum + R2;
    float* ecum = bt + R2;
    float* erem = ecum + R2;
    uint64_t* bar_s = reinterpret_cast<uint64_t*>(smem + T_BAR);  // pair products done
    uint64_t* bar_v = bar_s + 1;                                  // v has landed
    uint64_t* bar_uw = bar_s + 2;                                 // u, w product done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_s + 3);
    volatile int* gave_up = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int c0 = 2 * blockIdx.x, h = blockIdx.y, hk = h / (H / HK);
    const int r0 = c0 * C;
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const size_t tile0 = (size_t)h * NC + c0;   // (head, chunk) tile of rows [0, 64); rows [64, 128) are tile0 + 1
    const bool second = c0 + 1 < NC;            // the second chunk exists
    if (tid == 0) {
        mbar_init(bar_s, 1);
        mbar_init(bar_v, 1);
        mbar_init(bar_uw, 1);
        *gave_up = 0;
        mbar_init_fence();
        prefetch_tmap(&map_v);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    auto wait_for = [&](uint64_t* bar) {
        if (!mbar_wait(bar, 0, gave_up)) {
            atomicCAS(&g_gdn_error, 0, 43);
            *gave_up = 1;
        }
    };

    grid_dep_sync();
    // ---- log-decays per chunk: sequential float32 prefix sums, rows past the end have g = beta = 0 ----
    if (tid < R2) {
        const int row = r0 + tid;
        cum[tid] = row < T ? g[(size_t)row * H + h] : 0.f;
        bt[tid] = row < T ? f32(beta[(size_t)row * H + h]) : 0.f;
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    if (lane == 0 && warp < 2) {  // one thread per chunk
        float* cc = cum + warp * C;
        float run = 0.f;
#pragma unroll 8
        for (int i = 0; i < C; i++) cc[i] = (run += cc[i]);
    }
    __syncthreads();
    if (tid < R2) {
        const float last = cum[(tid & ~(C - 1)) + C - 1];
        ecum[tid] = expf(cum[tid]);
        erem[tid] = expf(last - cum[tid]);
        if ((tid & (C - 1)) == 0 && (tid == 0 || second)) ws.decay[tile0 + (tid >> 6)] = expf(last);
    }
    __syncthreads();

    // ---- L2 norms; TF32 operand tiles in the swizzled K-major layout; k exp(cum) in the swizzled
    //      MN-major layout; qd and kd to the workspace. 16 lanes per row, 32 rows per pass; a lane
    //      owns dims [4 sub, 4 sub + 4) and [64 + 4 sub, 64 + 4 sub + 4). ----
    {
        const int sub = tid & 15, rsel = tid >> 4, d0 = sub * 4;
        // all rows of k and q are requested before the first is used
        uint2 raws[2][4][2];
#pragma unroll
        for (int which = 0; which < 2; which++) {
            const bf16* src0 = which == 0 ? k : q;
#pragma unroll
            for (int pass = 0; pass < 4; pass++) {
                const int r = pass * 32 + rsel;
                raws[which][pass][0] = raws[which][pass][1] = make_uint2(0, 0);
                if (r0 + r < T) {
                    const bf16* src = src0 + ((size_t)(r0 + r) * HK + hk) * D + d0;
                    raws[which][pass][0] = *reinterpret_cast<const uint2*>(src);
                    raws[which][pass][1] = *reinterpret_cast<const uint2*>(src + 64);
                }
            }
        }
#pragma unroll
        for (int which = 0; which < 2; which++) {  // 0: k, 1: q
            const bool is_k = which == 0;
            const uint2 (&raw)[4][2] = raws[which];
            unsigned char* tile = smem + (is_k ? T_KF : T_QF);
#pragma unroll
            for (int pass = 0; pass < 4; pass++) {
                const int r = pass * 32 + rsel, ch = r >> 6, i = r & (C - 1);
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
                if (!is_k) inv *= scale;
                const float mult = is_k ? erem[r] : ecum[r];
                const float ec = ecum[r];
                bf16* dout = (is_k ? ws.kd : ws.qd) + (tile0 + ch) * (C * LDH) + i * LDH;
                const bool exists = ch == 0 || second;
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    float nrm[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) nrm[e] = x[4 * half + e] * inv;
                    float4 t;
                    t.x = __uint_as_float(to_tf32(nrm[0]));
                    t.y = __uint_as_float(to_tf32(nrm[1]));
                    t.z = __uint_as_float(to_tf32(nrm[2]));
                    t.w = __uint_as_float(to_tf32(nrm[3]));
                    // column 64 half + 4 sub of a float row: box (2 half + sub / 8), 16-byte chunk sub % 8
                    *reinterpret_cast<float4*>(tile + (2 * half + (sub >> 3)) * BOX + r * 128 +
                                               (((sub & 7) ^ (r & 7)) * 16)) = t;
                    if (exists) {
                        uint2 o;
                        o.x = pack2(nrm[0] * mult, nrm[1] * mult);
                        o.y = pack2(nrm[2] * mult, nrm[3] * mult);
                        *reinterpret_cast<uint2*>(dout + 64 * half + d0) = o;
                    }
                    if (is_k) {
                        // k exp(cum), bf16: box `half` of 64 columns, chunk (4 sub) / 8, 8 bytes at (sub & 1) * 8
                        uint2 e2;
                        e2.x = pack2(nrm[0] * ec, nrm[1] * ec);
                        e2.y = pack2(nrm[2] * ec, nrm[3] * ec);
                        *reinterpret_cast<uint2*>(smem + T_KE + half * BOX + r * 128 + (((sub >> 1) ^ (r & 7)) * 16) +
                                                  (sub & 1) * 8) = e2;
                    }
                }
            }
        }
    }
    fence_proxy_async();  // the operand tiles were written by threads, the MMAs read them
    __syncthreads();

    // ---- pair products: S_kk = k k^T into tensor-memory columns [0, 128), S_qk = q k^T into [128, 256) ----
    if (tid == 0) {
        fence_after_sync();
        constexpr uint32_t idesc = instr_desc(2, R2, R2);
        const uint32_t kf = smem_addr(smem + T_KF), qf = smem_addr(smem + T_QF);
#pragma unroll
        for (int ks = 0; ks < D / 8; ks++) {  // 8 float columns per step; four steps per 32-column box
            const uint64_t bk = smem_desc_sw128(kf + (ks / 4) * BOX + (ks % 4) * 32);
            mma_tf32_ss(tmem_base, bk, bk, idesc, ks > 0 ? 1u : 0u);
            mma_tf32_ss(tmem_base + R2, smem_desc_sw128(qf + (ks / 4) * BOX + (ks % 4) * 32), bk, idesc,
                        ks > 0 ? 1u : 0u);
        }
        mma_commit(bar_s);
    }
    wait_for(bar_s);
    fence_after_sync();
    // the q operand is dead: v comes in over its second half, four [64 rows, 64 columns] boxes
    if (tid == 0) {
        mbar_expect_tx(bar_v, 2 * BOX);
        for (int cb = 0; cb < 2; cb++)
            for (int rh = 0; rh < 2; rh++)
                tma_load_2d(smem + T_VB + cb * BOX + rh * (C * 128), &map_v, h * D + cb * 64, r0 + rh * C, bar_v);
    }

    // ---- decay masks: warps 0-7 read S_kk -> A (float32, shared), warps 8-15 S_qk -> P (bf16, workspace);
    //      a thread takes one row, and of its chunk's 64 columns the 32 of its warp group ----
    {
        const int quarter = warp & 3, r = quarter * 32 + lane, ch = r >> 6, i = r & (C - 1);
        const bool is_kk = warp < 8;
        const int cc = (warp >> 2) & 1;
        const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (is_kk ? 0 : R2) + ch * C;
        const float ci = cum[r], bi = bt[r];
        const float* cj = cum + ch * C;
        float* a_row = A + r * LDA;
        bf16* p_row = ws.p + (tile0 + ch) * (C * LDT) + i * LDT;
        const bool exists = ch == 0 || second;
        {
            uint32_t v[32];
            tmem_ld_32x32(t_row + cc * 32, v);
            tmem_ld_wait();
            float y[32];
#pragma unroll
            for (int e = 0; e < 32; e++) {
                const int j = cc * 32 + e;
                const float w = __uint_as_float(v[e]) * expf(ci - cj[j]);
                y[e] = is_kk ? (j < i ? bi * w : 0.f) : (j <= i ? w : 0.f);
            }
            if (is_kk) {
#pragma unroll
                for (int e = 0; e < 8; e++)
                    *reinterpret_cast<float4*>(a_row + cc * 32 + 4 * e) =
                        make_float4(y[4 * e], y[4 * e + 1], y[4 * e + 2], y[4 * e + 3]);
            } else if (exists) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    uint4 o;
                    o.x = pack2(y[8 * e + 0], y[8 * e + 1]);
                    o.y = pack2(y[8 * e + 2], y[8 * e + 3]);
                    o.z = pack2(y[8 * e + 4], y[8 * e + 5]);
                    o.w = pack2(y[8 * e + 6], y[8 * e + 7]);
                    *reinterpret_cast<uint4*>(p_row + cc * 32 + 8 * e) = o;
                }
            }
        }
    }
    fence_before_sync();
    __syncthreads();

    // ---- T = (I + A)^-1 for both chunks at once: threads [0, 256) the first, [256, 512) the second ----
    {
        const int g2 = tid >> 8, t = tid & 255;
        float* Ab = A + g2 * C * LDA;
        float* X = reinterpret_cast<float*>(smem + T_X) + g2 * 32 * LDX;
        float col[16];
        if (t < 64) {
            const float* blk = Ab + (16 * (t >> 4)) * (LDA + 1);
            const int j = t & 15;
#pragma unroll
            for (int i = 0; i < 16; i++) {
                float acc = i == j ? 1.f : 0.f;
#pragma unroll
                for (int m = 0; m < i; m++) acc -= blk[i * LDA + m] * col[m];
                col[i] = acc;
            }
        }
        __syncthreads();
        if (t < 64) {
            float* blk = Ab + (16 * (t >> 4)) * (LDA + 1);
            const int j = t & 15;
#pragma unroll
            for (int i = 0; i < 16; i++) blk[i * LDA + j] = col[i];
        }
        __syncthreads();
        {   // 16 -> 32: two pairs of diagonal blocks, 2 x 256 outputs, two per thread
            const int p = t >> 7, idx = t & 127, i = idx >> 3, j0 = (idx & 7) * 2;
            float* t11 = Ab + (32 * p) * (LDA + 1);
            float* a21 = t11 + 16 * LDA;
            const float* t22 = a21 + 16;
            float x0 = 0.f, x1 = 0.f;
#pragma unroll
            for (int m = 0; m < 16; m++) {
                const float a = a21[i * LDA + m];
                const float2 tt = *reinterpret_cast<const float2*>(t11 + m * LDA + j0);
                x0 += a * tt.x;
                x1 += a * tt.y;
            }
            *reinterpret_cast<float2*>(X + (16 * p + i) * LDX + j0) = make_float2(x0, x1);
            __syncthreads();
            float y0 = 0.f, y1 = 0.f;
#pragma unroll
            for (int m = 0; m < 16; m++) {
                const float a = t22[i * LDA + m];
                const float2 tt = *reinterpret_cast<const float2*>(X + (16 * p + m) * LDX + j0);
                y0 -= a * tt.x;
                y1 -= a * tt.y;
            }
            *reinterpret_cast<float2*>(a21 + i * LDA + j0) = make_float2(y0, y1);
            __syncthreads();
        }
        {   // 32 -> 64: 32 x 32 outputs as 4 x 4 register tiles on 64 threads (a quarter of the
            // shared-memory traffic of one row per thread, which bounded this step)
            const int ib = (t >> 3) * 4, j0 = (t & 7) * 4;
            float* a21 = Ab + 32 * LDA;
            const float* t22 = a21 + 32;
            float acc[4][4];
            if (t < 64) {
#pragma unroll
                for (int rr = 0; rr < 4; rr++) acc[rr][0] = acc[rr][1] = acc[rr][2] = acc[rr][3] = 0.f;
#pragma unroll 4
                for (int m = 0; m < 32; m++) {
                    const float4 tt = *reinterpret_cast<const float4*>(Ab + m * LDA + j0);
#pragma unroll
                    for (int rr = 0; rr < 4; rr++) {
                        const float a = a21[(ib + rr) * LDA + m];
                        acc[rr][0] += a * tt.x, acc[rr][1] += a * tt.y, acc[rr][2] += a * tt.z, acc[rr][3] += a * tt.w;
                    }
                }
#pragma unroll
                for (int rr = 0; rr < 4; rr++)
                    *reinterpret_cast<float4*>(X + (ib + rr) * LDX + j0) =
                        make_float4(acc[rr][0], acc[rr][1], acc[rr][2], acc[rr][3]);
            }
            __syncthreads();
            if (t < 64) {
#pragma unroll
                for (int rr = 0; rr < 4; rr++) acc[rr][0] = acc[rr][1] = acc[rr][2] = acc[rr][3] = 0.f;
#pragma unroll 4
                for (int m = 0; m < 32; m++) {
                    const float4 tt = *reinterpret_cast<const float4*>(X + m * LDX + j0);
#pragma unroll
                    for (int rr = 0; rr < 4; rr++) {
                        const float a = t22[(ib + rr) * LDA + m];
                        acc[rr][0] -= a * tt.x, acc[rr][1] -= a * tt.y, acc[rr][2] -= a * tt.z, acc[rr][3] -= a * tt.w;
                    }
                }
#pragma unroll
                for (int rr = 0; rr < 4; rr++)
                    *reinterpret_cast<float4*>(a21 + (ib + rr) * LDA + j0) =
                        make_float4(acc[rr][0], acc[rr][1], acc[rr][2], acc[rr][3]);
            }
            __syncthreads();
        }
    }
    // ---- T beta as the bf16 K-major operand [128 rows][128 k], block diagonal: a thread writes 32
    //      k-columns of one box of one row - its chunk's values, or zeros off the diagonal ----
    {
        const int r = tid >> 2, box = (tid >> 1) & 1, part = tid & 1, ch = r >> 6;
        unsigned char* dst = smem + T_TB + box * BOX + r * 128;
        const float* t_row = A + r * LDA;
        const float* bj = bt + ch * C;
#pragma unroll
        for (int c4 = 0; c4 < 4; c4++) {
            const int cj = 4 * part + c4;
            uint4 o = make_uint4(0, 0, 0, 0);
            if (box == ch) {
                const float4 a0 = *reinterpret_cast<const float4*>(t_row + 8 * cj);
                const float4 a1 = *reinterpret_cast<const float4*>(t_row + 8 * cj + 4);
                o.x = pack2(a0.x * bj[8 * cj + 0], a0.y * bj[8 * cj + 1]);
                o.y = pack2(a0.z * bj[8 * cj + 2], a0.w * bj[8 * cj + 3]);
                o.z = pack2(a1.x * bj[8 * cj + 4], a1.y * bj[8 * cj + 5]);
                o.w = pack2(a1.z * bj[8 * cj + 6], a1.w * bj[8 * cj + 7]);
            }
            *reinterpret_cast<uint4*>(dst + ((cj ^ (r & 7)) * 16)) = o;
        }
    }
    fence_proxy_async();
    wait_for(bar_v);
    __syncthreads();

    // ---- [u | w] = (T beta) [v | k exp(cum)]: one 128 x 256 x 128 product into columns [256, 512) ----
    if (tid == 0) {
        fence_after_sync();
        constexpr uint32_t idesc = instr_desc_b_mn(1, R2, 2 * D);
        const uint32_t tb = smem_addr(smem + T_TB), vb = smem_addr(smem + T_VB);
#pragma unroll
        for (int kk = 0; kk < R2 / 16; kk++)
            mma_bf16_ss(tmem_base + 2 * R2, smem_desc_sw128(tb + (kk / 4) * BOX + (kk % 4) * 32),
                        smem_desc_mn_sw128(vb + kk * 2048, BOX, 1024), idesc, kk > 0 ? 1u : 0u);
        mma_commit(bar_uw);
    }
    wait_for(bar_uw);
    fence_after_sync();
    {   // warps 0-7 store u, warps 8-15 w; a thread takes one row and the 64 columns of its warp group
        const int quarter = warp & 3, r = quarter * 32 + lane, ch = r >> 6, i = r & (C - 1);
        const bool is_u = warp < 8;
        const int cc0 = ((warp >> 2) & 1) * 2;
        const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + 2 * R2 + (is_u ? 0 : D);
        const int vs_w = ws.vs, ldu = vs_w + 8;
        bf16* u_tile = ws.u + (tile0 + ch) * (size_t)(D / vs_w) * (C * ldu);
        bf16* w_row = ws.w + (tile0 + ch) * (C * LDH) + i * LDH;
        const bool exists = ch == 0 || second;
#pragma unroll 1
        for (int cc = cc0; cc < cc0 + 2; cc++) {
            uint32_t v[32];
            tmem_ld_32x32(t_row + cc * 32, v);
            tmem_ld_wait();
            if (!exists) continue;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                uint4 o;
                o.x = pack2(__uint_as_float(v[8 * e + 0]), __uint_as_float(v[8 * e + 1]));
                o.y = pack2(__uint_as_float(v[8 * e + 2]), __uint_as_float(v[8 * e + 3]));
                o.z = pack2(__uint_as_float(v[8 * e + 4]), __uint_as_float(v[8 * e + 5]));
                o.w = pack2(__uint_as_float(v[8 * e + 6]), __uint_as_float(v[8 * e + 7]));
                const int col = cc * 32 + 8 * e;
                bf16* at = is_u ? u_tile + (col / vs_w) * (C * ldu) + i * ldu + (col % vs_w) : w_row + col;
                *reinterpret_cast<uint4*>(at) = o;
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
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
    grid_dep_trigger();
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
    grid_dep_sync();
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
    static const bool prep_on_tc5 = [] {
        const char* v = getenv("S1_GDN_PREP");
        return !(v && strcmp(v, "mma") == 0);  // S1_GDN_PREP=mma keeps the mma.sync kernel, for A/B runs
    }();
    if (prep_on_tc5) {
        static bool prep2_done[64] = {};
        e = set_smem_once(gdn_prep_tc5, PREP2_SMEM, prep2_done);
        if (e != cudaSuccess) return e;
        CUtensorMap map_v;  // [64 rows, 64 columns] boxes, 128-byte swizzle
        if (!tensor_map_2d(v, (uint64_t)T, (uint64_t)H * D, (uint64_t)H * D, C, &map_v)) return CS1_ERR_TENSOR_MAP;
        launch_dep_family(DEP_GDN, gdn_prep_tc5, dim3((NC + 1) / 2, H), PREP2_THREADS, PREP2_SMEM, st, map_v, static_cast<const bf16*>(q), static_cast<const bf16*>(k), g, static_cast<const bf16*>(beta), ws, T, H, HK, NC, scale);
    } else {
        // v and k rows of a chunk as [64 rows, 128 columns] tiles of the caller's [T, heads, 128] arrays
        CUtensorMap map_k, map_v;
        if (!tensor_map_2d_plain(k, (uint64_t)T, (uint64_t)HK * D, (uint64_t)HK * D, C, D, &map_k) ||
            !tensor_map_2d_plain(v, (uint64_t)T, (uint64_t)H * D, (uint64_t)H * D, C, D, &map_v))
            return CS1_ERR_TENSOR_MAP;
        gdn_prep<<<dim3(NC, H), PREP_THREADS, PREP_SMEM, st>>>(map_k, map_v, static_cast<const bf16*>(q),
                                                              static_cast<const bf16*>(k), g,
                                                              static_cast<const bf16*>(beta), ws, T, H, HK, scale);
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (ws.vs == 32) {
        e = set_smem_once(gdn_scan<32, 8>, ScanSmem<32>::BYTES, scan32_done);
        if (e != cudaSuccess) return e;
        launch_dep_family(DEP_GDN, gdn_scan<32, 8>, dim3(H, D / 32), 256, ScanSmem<32>::BYTES, st, ws, static_cast<bf16*>(o), T, H, NC, si, so);
    } else {
        e = set_smem_once(gdn_scan<16, 4>, ScanSmem<16>::BYTES, scan16_done);
        if (e != cudaSuccess) return e;
        launch_dep_family(DEP_GDN, gdn_scan<16, 4>, dim3(H, D / 16), 128, ScanSmem<16>::BYTES, st, ws, static_cast<bf16*>(o), T, H, NC, si, so);
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

// Device address of this device's error word, for the executor's status copy.
int s1::gdn_error_address(int** p) {
    void* a = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&a, s1::g_gdn_error);
    *p = static_cast<int*>(a);
    return e;
}
