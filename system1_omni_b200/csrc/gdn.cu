// Chunked (C = 64) WY-form gated delta rule, prefill only, head dim 128.
//
// Two kernels per call, both on tcgen05 tensor cores with accumulators in tensor memory, each
// over all the sequences of a pack (a table of up to 16 sequences is a kernel parameter):
//   gdn_prep_tc5  one block per (chunk = 64 rows, value head, sequence), fully parallel: cumulative
//             log-decays, L2 norms of q and k, the pair products k.k and q.k (TF32), the
//             triangular inverse T = (I + A)^-1 in float32, [u | w] = T beta [v | k exp(cum)]
//             (bf16). Leaves u, w, qd = q exp(cum), kd = k exp(cum_last - cum), P = (q.k)
//             decay-masked and exp(cum_last) in the workspace.
//   gdn_scan_tc5  one block per (value head, 64 value columns, sequence), sequential over chunks: the
//             state S [128 x 64] stays on the chip for the whole sequence - the float32 master
//             in tensor memory, its bf16 copy in shared memory as the operand of the next
//             chunk's products. Per chunk v_new = u - w S, o = qd S + P v_new (written straight
//             to the output) and S = decay S + kd^T v_new. Neither S nor v_new ever goes to
//             global memory.
//
// Every workspace tile is stored in the 128-byte-swizzled layout the tensor core reads from
// shared memory, so the scan brings a chunk's tiles in with four bulk copies and issues its
// products on them as they land.
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
#include "status.h"
#include "tc5.cuh"
#include "tmap.h"

namespace s1 {
namespace {

constexpr int C = 64;   // chunk length
constexpr int D = 128;  // key and value head dim
constexpr int LDA = C + 4;   // float row stride of A
constexpr int LDX = 36;      // float row stride of the 32 x 32 temporary of the inverse
constexpr int VS = 64;       // value columns per scan block: one 128-byte swizzle row of bf16

// Workspace tiles of one (head, chunk), each a sequence of "boxes" of 128-byte rows whose eight
// 16-byte pieces are permuted by the row number (the 128-byte swizzle of TMA and tcgen05), rows
// in groups of eight:
//   wq  two boxes of [128 rows x 64 k-dims]: rows 0-63 w, rows 64-127 qd (one K-major A operand)
//   kd  two boxes of [64 tokens x 64 k-dims] (an MN-major A operand: kd^T)
//   p   one box of [64 rows x 64 tokens]
//   u   two boxes of [64 rows x 64 value columns], one per scan block of the head
constexpr int WQ_BYTES = 2 * 128 * 128;
constexpr int KD_BYTES = 2 * C * 128;
constexpr int P_BYTES = C * 128;
constexpr int U_BYTES = C * 128;

// Byte offset of 16-byte piece `piece` (0..7) of row `row` inside a box.
__host__ __device__ constexpr int swz(int row, int piece) { return row * 128 + ((piece ^ (row & 7)) << 4); }

struct Work {
    unsigned char *wq, *kd, *p, *u;
    float* decay;  // [H, NC]
};

struct Layout {
    size_t wq, kd, p, u, decay, total;
    Layout(int T, int H) {
        const size_t tiles = (size_t)H * (((size_t)T + C - 1) / C);
        size_t at = 0;
        auto take = [&](size_t bytes) {
            const size_t off = at;
            at = (at + bytes + 1023) / 1024 * 1024;
            return off;
        };
        wq = take(tiles * WQ_BYTES);
        kd = take(tiles * KD_BYTES);
        p = take(tiles * P_BYTES);
        u = take(tiles * 2 * U_BYTES);
        decay = take(tiles * 4);
        total = at;
    }
};

Work split(float* workspace, int T, int H) {
    const Layout l(T, H);
    unsigned char* b = reinterpret_cast<unsigned char*>(workspace);
    return Work{b + l.wq, b + l.kd, b + l.p, b + l.u, reinterpret_cast<float*>(b + l.decay)};
}

// The sequences of one launch: a pack holds at most 16 (s1_batch_ranges). A sequence is rows
// [row0, row0 + len) of the packed operands and chunks [chunk0, chunk0 + ceil(len / 64)) of every
// head's run of workspace tiles (chunks chunks per head in all).
constexpr int MAX_SEQS = 16;
struct Seqs {
    int n, chunks;
    int row0[MAX_SEQS], len[MAX_SEQS], chunk0[MAX_SEQS];
};

__device__ int g_gdn_error = 0;  // a bounded wait gave up (read with s1_gdn_status / s1_device_status)

__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}

// ---------------------------------------------------------------------------------------
// gdn_prep_tc5: one chunk (64 rows) of one value head per block, two blocks to an SM so that one
// block's float32 phases run under the other's waits. The pair products k.k and q.k are one
// 128 x 64 x 128 TF32 MMA: its A operand stacks the normalised k rows on the normalised q rows
// (written by the norm phase straight into the swizzled K-major layout), its B operand is the k
// half of the same tile, so rows 0-63 of the result are k k^T and rows 64-127 q k^T. u and w are
// one 128 x 256 x 64 bf16 MMA of T beta (its 64 rows stored twice, so that all eight warps can
// read results out of their quarter of tensor memory) with [v | k exp(cum)], v arriving as a
// TMA tile and read MN-major. Everything between - decays, norms, masks, the triangular
// inverse - is float32 code on the CUDA cores.
// ---------------------------------------------------------------------------------------
constexpr int KQ_BOX = 128 * 128;                // bytes of one [128 rows x 128 bytes] swizzled box
constexpr int T_KQ = 0;                          // float, 4 boxes of 32 columns: rows 0-63 k, 64-127 q, normalised (TF32 bits)
constexpr int T_KE = T_KQ + 4 * KQ_BOX;          // bf16, 2 boxes of [64 tokens x 64 columns]: k exp(cum)
constexpr int T_A = T_KE + 2 * U_BYTES;          // float [64][LDA]: A, then T
constexpr int T_X = T_A + C * LDA * 4;           // float [32][LDX]: temporary of the inverse
constexpr int T_SM = T_X + 32 * LDX * 4;         // float [4][64]: cum, beta, exp(cum), exp(cum_last - cum)
constexpr int T_BAR = T_SM + 4 * C * 4;          // three mbarriers, the tensor-memory address, a flag
constexpr int PREP_SMEM = T_BAR + 64 + 1024;     // + slack to align the base to 1024
// once the pair products are done, over their operand:
constexpr int T_TB = T_KQ;                       // bf16, one box of [128 rows x 64 k]: T beta, twice
constexpr int T_VB = T_KE - 2 * U_BYTES;         // bf16, 2 boxes of [64 tokens x 64 columns]: v, as TMA leaves it; T_KE follows
static_assert(T_VB >= T_TB + KQ_BOX, "v lands behind T beta");
static_assert(2 * PREP_SMEM + 2048 <= 227 * 1024, "two blocks share an SM");
constexpr int PREP_THREADS = 256;
constexpr int PREP_TMEM_COLS = 256;              // pair products in columns [0, 64), then [u | w] in [0, 256)

__global__ void __launch_bounds__(PREP_THREADS, 2)
    gdn_prep_tc5(const __grid_constant__ CUtensorMap map_v, const bf16* __restrict__ q, const bf16* __restrict__ k,
                 const float* __restrict__ g, const bf16* __restrict__ beta, Work ws, const __grid_constant__ Seqs seqs,
                 int H, int HK, float scale) {
    using namespace tc5;
    grid_dep_trigger();
    // blockIdx.z: the sequence; its rows start at row0 of the packed operands. Chunks past its end
    // have nothing to do (the grid is as wide as the longest sequence).
    const int T = seqs.len[blockIdx.z], row0 = seqs.row0[blockIdx.z], NC = seqs.chunks;
    if ((int)blockIdx.x * C >= T) return;
    q += (size_t)row0 * HK * D;
    k += (size_t)row0 * HK * D;
    g += (size_t)row0 * H;
    beta += (size_t)row0 * H;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    float* A = reinterpret_cast<float*>(smem + T_A);
    float* X = reinterpret_cast<float*>(smem + T_X);
    float* cum = reinterpret_cast<float*>(smem + T_SM);
    float* bt = cum + C;
    float* ecum = bt + C;
    float* erem = ecum + C;
    uint64_t* bar_s = reinterpret_cast<uint64_t*>(smem + T_BAR);  // pair products done
    uint64_t* bar_v = bar_s + 1;                                  // v has landed
    uint64_t* bar_uw = bar_s + 2;                                 // u, w product done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_s + 3);
    volatile int* gave_up = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int c = blockIdx.x, h = blockIdx.y, hk = h / (H / HK);
    const int r0 = c * C;
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int quarter = warp & 3;               // the 32 tensor-memory lanes this warp may touch
    const size_t tile = (size_t)h * NC + seqs.chunk0[blockIdx.z] + c;  // this block's (head, chunk) tile in every workspace array
    if (tid == 0) {
        mbar_init(bar_s, 1);
        mbar_init(bar_v, 1);
        mbar_init(bar_uw, 1);
        *gave_up = 0;
        mbar_init_fence();
        prefetch_tmap(&map_v);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, PREP_TMEM_COLS);
        tmem_relinquish();
    }
    auto wait_for = [&](uint64_t* bar) {
        if (!mbar_wait(bar, 0, gave_up)) {
            atomicCAS(&g_gdn_error, 0, 43);
            *gave_up = 1;
        }
    };

    grid_dep_sync();
    // ---- q and k rows are requested first of all: 16 lanes per row, 16 rows per pass; a lane owns
    //      the 8 dims [8 sub, 8 sub + 8), one 16-byte piece of the row ----
    const int sub = tid & 15, rsel = tid >> 4;
    uint4 raws[2][4];
#pragma unroll
    for (int which = 0; which < 2; which++) {
        const bf16* src0 = which == 0 ? k : q;
#pragma unroll
        for (int pass = 0; pass < 4; pass++) {
            const int r = pass * 16 + rsel;
            raws[which][pass] = make_uint4(0, 0, 0, 0);
            if (r0 + r < T) raws[which][pass] = ld16(src0 + ((size_t)(r0 + r) * HK + hk) * D + sub * 8);
        }
    }
    // ---- log-decays: float32 prefix sums over the chunk (a shuffle scan in each of the two warps,
    //      the second adding the first one's total), rows past the end have g = beta = 0 ----
    if (tid < C) {
        const int row = r0 + tid;
        float x = row < T ? g[(size_t)row * H + h] : 0.f;
        bt[tid] = row < T ? f32(beta[(size_t)row * H + h]) : 0.f;
#pragma unroll
        for (int o2 = 1; o2 < 32; o2 <<= 1) {
            const float y = __shfl_up_sync(0xffffffffu, x, o2);
            if (lane >= o2) x += y;
        }
        cum[tid] = x;
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t t_lanes = tmem_base + ((uint32_t)(quarter * 32) << 16);
    if (tid >= 32 && tid < C) cum[tid] += cum[31];
    __syncthreads();
    if (tid < C) {
        const float last = cum[C - 1];
        ecum[tid] = expf(cum[tid]);
        erem[tid] = expf(last - cum[tid]);
        if (tid == 0) ws.decay[tile] = expf(last);
    }
    __syncthreads();

    // ---- L2 norms; the TF32 operand tile in the swizzled K-major layout (k rows, then q rows);
    //      k exp(cum) in the swizzled MN-major layout; qd and kd to the workspace ----
#pragma unroll
    for (int which = 0; which < 2; which++) {  // 0: k, 1: q
        const bool is_k = which == 0;
#pragma unroll
        for (int pass = 0; pass < 4; pass++) {
            const int i = pass * 16 + rsel, r = is_k ? i : C + i;
            float x[8];
            unpack8(raws[which][pass], x);
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < 8; e++) ss += x[e] * x[e];
            ss = warp_sum<16>(ss);
            float inv = rsqrtf(ss + 1e-6f);
            if (!is_k) inv *= scale;
            const float mult = is_k ? erem[i] : ecum[i];
            const float ec = ecum[i];
            float nrm[8];
#pragma unroll
            for (int e = 0; e < 8; e++) nrm[e] = x[e] * inv;
            // float columns [8 sub, 8 sub + 8): box sub / 4, 16-byte pieces 2 (sub % 4) and the next
            unsigned char* tf = smem + T_KQ + (sub >> 2) * KQ_BOX;
            *reinterpret_cast<float4*>(tf + swz(r, 2 * (sub & 3))) =
                make_float4(__uint_as_float(to_tf32(nrm[0])), __uint_as_float(to_tf32(nrm[1])), __uint_as_float(to_tf32(nrm[2])),
                            __uint_as_float(to_tf32(nrm[3])));
            *reinterpret_cast<float4*>(tf + swz(r, 2 * (sub & 3) + 1)) =
                make_float4(__uint_as_float(to_tf32(nrm[4])), __uint_as_float(to_tf32(nrm[5])), __uint_as_float(to_tf32(nrm[6])),
                            __uint_as_float(to_tf32(nrm[7])));
            // kd: token row i of the two [64 tokens x 64 dims] boxes; qd: row 64 + i of the two
            // [128 rows x 64 dims] boxes it shares with w. bf16 columns [8 sub, +8): box sub / 8, piece sub % 8
            float scaled[8];
#pragma unroll
            for (int e = 0; e < 8; e++) scaled[e] = nrm[e] * mult;
            unsigned char* dout = is_k ? ws.kd + tile * KD_BYTES + (sub >> 3) * (KD_BYTES / 2) + swz(i, sub & 7)
                                       : ws.wq + tile * WQ_BYTES + (sub >> 3) * (WQ_BYTES / 2) + swz(C + i, sub & 7);
            st16(dout, pack8(scaled));
            if (is_k) {  // k exp(cum), the MN-major operand half of [v | k exp(cum)]
#pragma unroll
                for (int e = 0; e < 8; e++) scaled[e] = nrm[e] * ec;
                st16(smem + T_KE + (sub >> 3) * U_BYTES + swz(i, sub & 7), pack8(scaled));
            }
        }
    }
    fence_proxy_async();  // the operand tiles were written by threads, the MMAs read them
    __syncthreads();

    // ---- pair products: rows 0-63 k k^T, rows 64-127 q k^T, tensor-memory columns [0, 64) ----
    if (tid == 0) {
        fence_after_sync();
        constexpr uint32_t idesc = instr_desc(2, 2 * C, C);
        const uint32_t kq = smem_addr(smem + T_KQ);
#pragma unroll
        for (int ks = 0; ks < D / 8; ks++) {  // 8 float columns per step; four steps per 32-column box
            const uint64_t tile_k = smem_desc_sw128(kq + (ks / 4) * KQ_BOX + (ks % 4) * 32);
            mma_tf32_ss(tmem_base, tile_k, tile_k, idesc, ks > 0 ? 1u : 0u);  // B: the first 64 rows of the same boxes
        }
        mma_commit(bar_s);
    }
    wait_for(bar_s);
    fence_after_sync();
    // the operand tile is dead: v comes in over its end, two [64 rows, 64 columns] boxes
    if (tid == 0) {
        mbar_expect_tx(bar_v, 2 * U_BYTES);
        // rows past the sequence's end hold the next sequence's values (or zeros past the end of the
        // buffer): beta is zero there, so T beta has zero columns for them
        for (int cb = 0; cb < 2; cb++) tma_load_2d(smem + T_VB + cb * U_BYTES, &map_v, h * D + cb * 64, row0 + r0, bar_v);
    }

    // ---- decay masks: the warps of quarters 0-1 read k k^T -> A (float32, shared), those of
    //      quarters 2-3 q k^T -> P (bf16, workspace); a thread takes one row and 32 of its 64 columns ----
    {
        const int i = (quarter & 1) * 32 + lane, cc = warp >> 2;
        const bool is_kk = quarter < 2;
        const float ci = cum[i], bi = bt[i];
        float* a_row = A + i * LDA;
        unsigned char* p_tile = ws.p + tile * P_BYTES;
        uint32_t v[32];
        tmem_ld_32x32(t_lanes + cc * 32, v);
        tmem_ld_wait();
        float y[32];
#pragma unroll
        for (int e = 0; e < 32; e++) {
            const int j = cc * 32 + e;
            const float w = __uint_as_float(v[e]) * __expf(ci - cum[j]);
            y[e] = is_kk ? (j < i ? bi * w : 0.f) : (j <= i ? w : 0.f);
        }
        if (is_kk) {
#pragma unroll
            for (int e = 0; e < 8; e++)
                *reinterpret_cast<float4*>(a_row + cc * 32 + 4 * e) = make_float4(y[4 * e], y[4 * e + 1], y[4 * e + 2], y[4 * e + 3]);
        } else {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                uint4 o;
                o.x = pack2(y[8 * e + 0], y[8 * e + 1]);
                o.y = pack2(y[8 * e + 2], y[8 * e + 3]);
                o.z = pack2(y[8 * e + 4], y[8 * e + 5]);
                o.w = pack2(y[8 * e + 6], y[8 * e + 7]);
                *reinterpret_cast<uint4*>(p_tile + swz(i, cc * 4 + e)) = o;
            }
        }
    }
    fence_before_sync();
    __syncthreads();

    // ---- T = (I + A)^-1 in float32: 16 x 16 diagonal blocks by substitution, then
    //      T21 = -T22 (A21 T11) for 16 -> 32 and 32 -> 64 ----
    {
        const int t = tid;
        float col[16];
        if (t < 64) {
            const float* blk = A + (16 * (t >> 4)) * (LDA + 1);
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
            float* blk = A + (16 * (t >> 4)) * (LDA + 1);
            const int j = t & 15;
#pragma unroll
            for (int i = 0; i < 16; i++) blk[i * LDA + j] = col[i];
        }
        __syncthreads();
        {   // 16 -> 32: two pairs of diagonal blocks, 2 x 256 outputs, two per thread
            const int p = t >> 7, idx = t & 127, i = idx >> 3, j0 = (idx & 7) * 2;
            float* t11 = A + (32 * p) * (LDA + 1);
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
        {   // 32 -> 64: 32 x 32 outputs as 4 x 2 register tiles on 128 threads, four steps of the sum
            // per pass so that the left factor's rows come in as float4
            const int ib = (t >> 4) * 4, j0 = (t & 15) * 2;
            float* a21 = A + 32 * LDA;
            const float* t22 = a21 + 32;
            float acc[4][2];
            if (t < 128) {
#pragma unroll
                for (int rr = 0; rr < 4; rr++) acc[rr][0] = acc[rr][1] = 0.f;
#pragma unroll 2
                for (int m = 0; m < 32; m += 4) {
                    float2 tt[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) tt[e] = *reinterpret_cast<const float2*>(A + (m + e) * LDA + j0);
#pragma unroll
                    for (int rr = 0; rr < 4; rr++) {
                        const float4 a = *reinterpret_cast<const float4*>(a21 + (ib + rr) * LDA + m);
                        acc[rr][0] += a.x * tt[0].x, acc[rr][1] += a.x * tt[0].y;
                        acc[rr][0] += a.y * tt[1].x, acc[rr][1] += a.y * tt[1].y;
                        acc[rr][0] += a.z * tt[2].x, acc[rr][1] += a.z * tt[2].y;
                        acc[rr][0] += a.w * tt[3].x, acc[rr][1] += a.w * tt[3].y;
                    }
                }
#pragma unroll
                for (int rr = 0; rr < 4; rr++) *reinterpret_cast<float2*>(X + (ib + rr) * LDX + j0) = make_float2(acc[rr][0], acc[rr][1]);
            }
            __syncthreads();
            if (t < 128) {
#pragma unroll
                for (int rr = 0; rr < 4; rr++) acc[rr][0] = acc[rr][1] = 0.f;
#pragma unroll 2
                for (int m = 0; m < 32; m += 4) {
                    float2 tt[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) tt[e] = *reinterpret_cast<const float2*>(X + (m + e) * LDX + j0);
#pragma unroll
                    for (int rr = 0; rr < 4; rr++) {
                        const float4 a = *reinterpret_cast<const float4*>(t22 + (ib + rr) * LDA + m);
                        acc[rr][0] -= a.x * tt[0].x, acc[rr][1] -= a.x * tt[0].y;
                        acc[rr][0] -= a.y * tt[1].x, acc[rr][1] -= a.y * tt[1].y;
                        acc[rr][0] -= a.z * tt[2].x, acc[rr][1] -= a.z * tt[2].y;
                        acc[rr][0] -= a.w * tt[3].x, acc[rr][1] -= a.w * tt[3].y;
                    }
                }
#pragma unroll
                for (int rr = 0; rr < 4; rr++) *reinterpret_cast<float2*>(a21 + (ib + rr) * LDA + j0) = make_float2(acc[rr][0], acc[rr][1]);
            }
            __syncthreads();
        }
    }
    // ---- T beta as the bf16 K-major operand [128 rows][64 k]: rows 0-63 and, again, rows 64-127.
    //      A thread writes 16 k-columns of one row, into both copies ----
    {
        const int r = tid >> 2, part = tid & 3;
        const float* t_row = A + r * LDA;
#pragma unroll
        for (int c2 = 0; c2 < 2; c2++) {
            const int cj = 2 * part + c2;
            const float4 a0 = *reinterpret_cast<const float4*>(t_row + 8 * cj);
            const float4 a1 = *reinterpret_cast<const float4*>(t_row + 8 * cj + 4);
            uint4 o;
            o.x = pack2(a0.x * bt[8 * cj + 0], a0.y * bt[8 * cj + 1]);
            o.y = pack2(a0.z * bt[8 * cj + 2], a0.w * bt[8 * cj + 3]);
            o.z = pack2(a1.x * bt[8 * cj + 4], a1.y * bt[8 * cj + 5]);
            o.w = pack2(a1.z * bt[8 * cj + 6], a1.w * bt[8 * cj + 7]);
            *reinterpret_cast<uint4*>(smem + T_TB + swz(r, cj)) = o;
            *reinterpret_cast<uint4*>(smem + T_TB + swz(C + r, cj)) = o;
        }
    }
    fence_proxy_async();
    wait_for(bar_v);
    __syncthreads();

    // ---- [u | w] = (T beta) [v | k exp(cum)]: one 128 x 256 x 64 product into columns [0, 256) ----
    if (tid == 0) {
        fence_after_sync();
        constexpr uint32_t idesc = instr_desc_b_mn(1, 2 * C, 2 * D);
        const uint32_t tb = smem_addr(smem + T_TB), vb = smem_addr(smem + T_VB);
#pragma unroll
        for (int kk = 0; kk < C / 16; kk++)
            mma_bf16_ss(tmem_base, smem_desc_sw128(tb + kk * 32), smem_desc_mn_sw128(vb + kk * 2048, U_BYTES, 1024), idesc,
                        kk > 0 ? 1u : 0u);
        mma_commit(bar_uw);
    }
    wait_for(bar_uw);
    fence_after_sync();
    {   // a thread takes one row (from either copy of the result) and 64 of the 256 columns: u for the
        // warps of the first four, w for the others
        const int i = (quarter & 1) * 32 + lane;
        const int group = (warp >> 2) * 2 + (quarter >> 1);  // 0, 1: u columns [64 group, +64); 2, 3: w columns
        unsigned char* dst = group < 2 ? ws.u + tile * (2 * U_BYTES) + group * U_BYTES
                                       : ws.wq + tile * WQ_BYTES + (group - 2) * (WQ_BYTES / 2);
#pragma unroll 1
        for (int cc = 0; cc < 2; cc++) {
            uint32_t v[32];
            tmem_ld_32x32(t_lanes + group * 64 + cc * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 4; e++) {
                uint4 o;
                o.x = pack2(__uint_as_float(v[8 * e + 0]), __uint_as_float(v[8 * e + 1]));
                o.y = pack2(__uint_as_float(v[8 * e + 2]), __uint_as_float(v[8 * e + 3]));
                o.z = pack2(__uint_as_float(v[8 * e + 4]), __uint_as_float(v[8 * e + 5]));
                o.w = pack2(__uint_as_float(v[8 * e + 6]), __uint_as_float(v[8 * e + 7]));
                *reinterpret_cast<uint4*>(dst + swz(i, cc * 4 + e)) = o;
            }
        }
    }
    if (*gave_up) __nanosleep(1000000);
    fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, PREP_TMEM_COLS);
}

// ---------------------------------------------------------------------------------------
// gdn_scan_tc5: the serial half. One block per (value head, 64 value columns); per chunk
//   D [128 x 64]  = [w ; qd] Sb            one M = 128 product: rows 0-63 w Sb, rows 64-127 qd Sb
//   v_new         = bf16(u - D[0:64])      by threads, straight into the next products' operand
//   D            += [. ; P] v_new          rows 64-127 become o = qd Sb + P v_new (rows 0-63 are dead by then)
//   S             = decay S + kd^T v_new   accumulated onto the float32 state in tensor memory,
//                                          which its threads scaled by decay beforehand
// Sb is the bf16 copy of the chunk-entry state, written by the state's threads into the swizzled
// MN-major operand layout. The chain S -> Sb -> D -> v_new -> S is what bounds a step, so every
// leg of it is spread over as many threads as tensor memory allows (a warp reaches only the 32
// lanes of its quarter): warps 0-7 own the state (a row of S and half of its columns per
// thread), warps 8-9 and 12-13 make v_new, warps 10-11 and 14-15 read o out of the accumulator
// (two of them, used in turn, so that a chunk's output is stored while the next chunk's first
// product runs) and store it, warp 16 feeds the copy engine (three stages of tiles) and issues
// the MMAs. The scaling of S is off the chain: the first product needs only Sb. Every wait is
// on an mbarrier and bounded.
// ---------------------------------------------------------------------------------------
constexpr int SCAN_THREADS = 17 * 32;
constexpr int STAGES = 3;                             // a chunk's tiles are requested two chunks ahead
constexpr int S_WQ = 0;                               // per stage: [w ; qd], two boxes of 128 rows
constexpr int S_KD = S_WQ + WQ_BYTES;                 // kd, two boxes of 64 token rows
constexpr int S_P = S_KD + KD_BYTES;                  // P, one box of 64 rows
// The product [.. ; P] v_new has M = 128: its A operand is the box of 128 rows that ends with P,
// i.e. it begins with the second box of kd. What those 64 rows contribute lands in rows 0-63 of
// D, which nobody reads after v_new has been taken from them.
constexpr int S_PA = S_P - P_BYTES;
constexpr int S_U = S_P + P_BYTES;                    // this block's box of u
constexpr int S_STAGE = S_U + U_BYTES;
constexpr int S_SB = STAGES * S_STAGE;                // bf16 state, one box of [128 k rows x 64 columns]
constexpr int S_VN = S_SB + D * 128;                  // v_new, one box of [64 tokens x 64 columns]
constexpr int S_BAR = S_VN + C * 128;                 // barriers, the tensor-memory address, a flag
constexpr int SCAN_SMEM = S_BAR + 128 + 1024;         // + slack to align the base to 1024
constexpr uint32_t STAGE_TX = WQ_BYTES + KD_BYTES + P_BYTES + U_BYTES;
constexpr int SCAN_TMEM_COLS = 256;                   // S in columns [0, 64), the two D in [64, 128) and [128, 192)
static_assert(S_STAGE % 1024 == 0 && S_KD % 1024 == 0 && S_PA % 1024 == 0 && S_U % 1024 == 0, "boxes are 1024-byte aligned");
static_assert(SCAN_SMEM <= 227 * 1024, "the stages fit an SM");

__global__ void __launch_bounds__(SCAN_THREADS, 1)
    gdn_scan_tc5(Work ws, bf16* __restrict__ o, const __grid_constant__ Seqs seqs, int H, const float* __restrict__ s_in,
                 float* __restrict__ s_out) {
    using namespace tc5;
    grid_dep_trigger();
    // blockIdx.z: the sequence. Every sequence starts from the same s_in (the candidates of one
    // prefix) and leaves its state in its own slot of s_out.
    const int T = seqs.len[blockIdx.z], NC = (T + C - 1) / C;
    o += (size_t)seqs.row0[blockIdx.z] * H * D;
    if (s_out) s_out += (size_t)blockIdx.z * H * D * D;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + S_BAR);  // [STAGES] a stage's tiles have landed
    uint64_t* sb_ready = full + 3;   // 256 arrivals: Sb written
    uint64_t* s_scaled = full + 4;   // 256 arrivals: decay S is back in tensor memory
    uint64_t* d1_done = full + 5;    // the first product is complete
    uint64_t* vn_ready = full + 6;   // 128 arrivals: v_new written
    uint64_t* s_done = full + 7;     // the state's product (the third) is complete
    uint64_t* d2_done = full + 8;    // [2], by chunk parity: every product of the chunk is complete
    uint64_t* d_free = full + 10;    // [2] 128 arrivals: that D has been read out
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(full + 12);
    volatile int* gave_up = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int h = blockIdx.x, slice = blockIdx.y, v0 = slice * VS;
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int quarter = warp & 3;  // the 32 tensor-memory lanes this warp may touch
    const size_t tile0 = (size_t)h * seqs.chunks + seqs.chunk0[blockIdx.z];

    if (tid == 0) {
        for (int i = 0; i < STAGES; i++) mbar_init(&full[i], 1);
        mbar_init(sb_ready, 256);
        mbar_init(s_scaled, 256);
        mbar_init(d1_done, 1);
        mbar_init(vn_ready, 128);
        mbar_init(s_done, 1);
        mbar_init(&d2_done[0], 1);
        mbar_init(&d2_done[1], 1);
        mbar_init(&d_free[0], 128);
        mbar_init(&d_free[1], 128);
        *gave_up = 0;
        mbar_init_fence();
    }
    if (warp == 16) {
        tmem_alloc(tmem_slot, SCAN_TMEM_COLS);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t t_lanes = tmem_base + ((uint32_t)(quarter * 32) << 16);
    auto fail = [&](int code) {
        atomicCAS(&g_gdn_error, 0, code);
        *gave_up = 1;
    };
    grid_dep_sync();

    if (warp < 8) {
        // ---- state: thread (k, hh) owns S[k][v0 + 32 hh .. + 32) ----
        const int hh = warp >> 2, k = quarter * 32 + lane;
        const uint32_t t_row = t_lanes + hh * 32;
        uint32_t s[32];
        if (s_in) {
            const float4* src = reinterpret_cast<const float4*>(s_in + ((size_t)h * D + k) * D + v0 + hh * 32);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float4 x = src[j];
                s[4 * j] = __float_as_uint(x.x), s[4 * j + 1] = __float_as_uint(x.y);
                s[4 * j + 2] = __float_as_uint(x.z), s[4 * j + 3] = __float_as_uint(x.w);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++) s[j] = 0u;
        }
        float decay = ws.decay[tile0];
        bool ok = true;
        for (int c = 0; c < NC; c++) {
            // bf16 copy of the chunk-entry state as the MN-major operand (row k, this thread's 32 columns)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint4 piece;
                piece.x = pack2(__uint_as_float(s[8 * j + 0]), __uint_as_float(s[8 * j + 1]));
                piece.y = pack2(__uint_as_float(s[8 * j + 2]), __uint_as_float(s[8 * j + 3]));
                piece.z = pack2(__uint_as_float(s[8 * j + 4]), __uint_as_float(s[8 * j + 5]));
                piece.w = pack2(__uint_as_float(s[8 * j + 6]), __uint_as_float(s[8 * j + 7]));
                *reinterpret_cast<uint4*>(smem + S_SB + swz(k, hh * 4 + j)) = piece;
            }
            fence_proxy_async();
            mbar_arrive(sb_ready);
            // decay S back into tensor memory: the third product accumulates onto it
#pragma unroll
            for (int j = 0; j < 32; j++) s[j] = __float_as_uint(__uint_as_float(s[j]) * decay);
            tmem_st_32x32(t_row, s);
            tmem_st_wait();
            fence_before_sync();
            mbar_arrive(s_scaled);
            if (c + 1 < NC) decay = ws.decay[tile0 + c + 1];
            if (!mbar_wait(s_done, c & 1, gave_up)) {
                fail(44);
                ok = false;
                break;
            }
            fence_after_sync();
            tmem_ld_32x32(t_row, s);
            tmem_ld_wait();
        }
        if (s_out && ok) {
            float4* dst = reinterpret_cast<float4*>(s_out + ((size_t)h * D + k) * D + v0 + hh * 32);
#pragma unroll
            for (int j = 0; j < 8; j++)
                dst[j] = make_float4(__uint_as_float(s[4 * j]), __uint_as_float(s[4 * j + 1]), __uint_as_float(s[4 * j + 2]),
                                     __uint_as_float(s[4 * j + 3]));
        }
    } else if (warp < 16 && quarter < 2) {
        // ---- v_new: thread (i, hh) owns v_new[i][32 hh .. + 32) of the chunk ----
        const int hh = (warp - 8) >> 2, i = quarter * 32 + lane;
        for (int c = 0; c < NC; c++) {
            // this thread's 32 values of u wait in registers for the product they are subtracted from
            if (!mbar_wait(&full[c % STAGES], (c / STAGES) & 1, gave_up)) {
                fail(53);
                break;
            }
            const unsigned char* u_box = smem + (c % STAGES) * S_STAGE + S_U;
            uint4 u_pieces[4];
#pragma unroll
            for (int j = 0; j < 4; j++) u_pieces[j] = *reinterpret_cast<const uint4*>(u_box + swz(i, hh * 4 + j));
            if (!mbar_wait(d1_done, c & 1, gave_up)) {
                fail(45);
                break;
            }
            fence_after_sync();
            uint32_t acc[32];
            tmem_ld_32x32(t_lanes + VS + (c & 1) * VS + hh * 32, acc);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float uf[8];
                unpack8(u_pieces[j], uf);
                uint4 piece;
                piece.x = pack2(uf[0] - __uint_as_float(acc[8 * j + 0]), uf[1] - __uint_as_float(acc[8 * j + 1]));
                piece.y = pack2(uf[2] - __uint_as_float(acc[8 * j + 2]), uf[3] - __uint_as_float(acc[8 * j + 3]));
                piece.z = pack2(uf[4] - __uint_as_float(acc[8 * j + 4]), uf[5] - __uint_as_float(acc[8 * j + 5]));
                piece.w = pack2(uf[6] - __uint_as_float(acc[8 * j + 6]), uf[7] - __uint_as_float(acc[8 * j + 7]));
                *reinterpret_cast<uint4*>(smem + S_VN + swz(i, hh * 4 + j)) = piece;
            }
            fence_proxy_async();
            fence_before_sync();
            mbar_arrive(vn_ready);
        }
    } else if (warp < 16) {
        // ---- output: thread (i, hh) reads o[row i][32 hh .. + 32) out of tensor-memory lane 64 + i ----
        const int hh = (warp - 8) >> 2, i = (quarter - 2) * 32 + lane;
        for (int c = 0; c < NC; c++) {
            if (!mbar_wait(&d2_done[c & 1], (c >> 1) & 1, gave_up)) {
                fail(46);
                break;
            }
            fence_after_sync();
            uint32_t acc[32];
            tmem_ld_32x32(t_lanes + VS + (c & 1) * VS + hh * 32, acc);
            tmem_ld_wait();
            fence_before_sync();
            mbar_arrive(&d_free[c & 1]);  // the first product of chunk c + 2 may overwrite it
            const int row = c * C + i;
            if (row < T) {
                uint4* dst = reinterpret_cast<uint4*>(o + ((size_t)row * H + h) * D + v0 + hh * 32);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    uint4 piece;
                    piece.x = pack2(__uint_as_float(acc[8 * j + 0]), __uint_as_float(acc[8 * j + 1]));
                    piece.y = pack2(__uint_as_float(acc[8 * j + 2]), __uint_as_float(acc[8 * j + 3]));
                    piece.z = pack2(__uint_as_float(acc[8 * j + 4]), __uint_as_float(acc[8 * j + 5]));
                    piece.w = pack2(__uint_as_float(acc[8 * j + 6]), __uint_as_float(acc[8 * j + 7]));
                    dst[j] = piece;
                }
            }
        }
    } else {
        // ---- copies and MMA issue: the whole warp runs the loop, one elected lane issues ----
        const bool issuer = elect_one();
        const unsigned char* wq_g = ws.wq + tile0 * WQ_BYTES;
        const unsigned char* kd_g = ws.kd + tile0 * KD_BYTES;
        const unsigned char* p_g = ws.p + tile0 * P_BYTES;
        const unsigned char* u_g = ws.u + tile0 * (2 * U_BYTES) + slice * U_BYTES;
        auto load = [&](int c) {
            if (!issuer) return;
            unsigned char* st = smem + (c % STAGES) * S_STAGE;
            uint64_t* bar = &full[c % STAGES];
            mbar_expect_tx(bar, STAGE_TX);
            bulk_load(st + S_WQ, wq_g + (size_t)c * WQ_BYTES, WQ_BYTES, bar);
            bulk_load(st + S_KD, kd_g + (size_t)c * KD_BYTES, KD_BYTES, bar);
            bulk_load(st + S_P, p_g + (size_t)c * P_BYTES, P_BYTES, bar);
            bulk_load(st + S_U, u_g + (size_t)c * (2 * U_BYTES), U_BYTES, bar);
        };
        for (int c = 0; c < STAGES - 1 && c < NC; c++) load(c);
        // The tiles of chunk c + 2 are requested during chunk c, into the stage chunk c - 1 has left
        // (its last product, the one that reads P, must have completed). When in the chunk matters: a
        // proxy fence issued by a thread while a bulk copy is still writing this block's shared
        // memory was measured to wait for the copy (500 cycles and more), and both the state's and
        // the v_new threads fence once per chunk - behind the first product's issue the copy has the
        // longest stretch without one of those fences to land in (10 % faster than behind the
        // v_new threads' fence).
        auto next_tiles = [&](int c) {
            if (c + STAGES - 1 >= NC) return true;
            if (c >= 1 && !mbar_wait(&d2_done[(c - 1) & 1], ((c - 1) >> 1) & 1, gave_up)) {
                fail(50);
                return false;
            }
            load(c + STAGES - 1);
            return true;
        };
        constexpr uint32_t idesc_b = instr_desc_b_mn(1, 128, VS);                // A K-major, B MN-major
        constexpr uint32_t idesc_ab = instr_desc_b_mn(1, 128, VS) | (1u << 15);  // both MN-major
        const uint32_t sb = smem_addr(smem + S_SB), vn = smem_addr(smem + S_VN);
        for (int c = 0; c < NC; c++) {
            const uint32_t st = smem_addr(smem + (c % STAGES) * S_STAGE);
            const uint32_t d = tmem_base + VS + (c & 1) * VS;
            if (!mbar_wait(&full[c % STAGES], (c / STAGES) & 1, gave_up)) {
                fail(47);
                break;
            }
            if (c >= 2 && !mbar_wait(&d_free[c & 1], ((c >> 1) - 1) & 1, gave_up)) {
                fail(51);
                break;
            }
            if (!mbar_wait(sb_ready, c & 1, gave_up)) {
                fail(48);
                break;
            }
            fence_after_sync();
            if (issuer) {
#pragma unroll
                for (int ks = 0; ks < D / 16; ks++)
                    mma_bf16_ss(d, smem_desc_sw128(st + S_WQ + (ks / 4) * (WQ_BYTES / 2) + (ks % 4) * 32),
                                smem_desc_mn_sw128(sb + ks * 2048, D * 128, 1024), idesc_b, ks > 0 ? 1u : 0u);
                mma_commit(d1_done);
            }
            __syncwarp();
            if (!next_tiles(c)) break;
            if (!mbar_wait(vn_ready, c & 1, gave_up)) {
                fail(49);
                break;
            }
            if (!mbar_wait(s_scaled, c & 1, gave_up)) {
                fail(52);
                break;
            }
            fence_after_sync();
            if (issuer) {
#pragma unroll
                for (int ks = 0; ks < C / 16; ks++)  // the state first: the next chunk waits for it alone
                    mma_bf16_ss(tmem_base, smem_desc_mn_sw128(st + S_KD + ks * 2048, KD_BYTES / 2, 1024),
                                smem_desc_mn_sw128(vn + ks * 2048, C * 128, 1024), idesc_ab, 1u);
                mma_commit(s_done);
#pragma unroll
                for (int ks = 0; ks < C / 16; ks++)
                    mma_bf16_ss(d, smem_desc_sw128(st + S_PA + ks * 32), smem_desc_mn_sw128(vn + ks * 2048, C * 128, 1024), idesc_b, 1u);
                mma_commit(&d2_done[c & 1]);
            }
            __syncwarp();
        }
        __syncwarp();
    }

    // wind down: after an abort give copies and MMAs in flight time to land before the
    // shared memory and tensor memory are released
    if (*gave_up) __nanosleep(1000000);
    fence_before_sync();
    __syncthreads();
    if (warp == 16) tmem_dealloc(tmem_base, SCAN_TMEM_COLS);
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

// The sequences row0[i], len[i] (i < nseq <= 16) of the packed operands in one pair of launches.
// workspace_bytes: what the caller has (0 = not checked: the single-sequence entry points size
// it by their documented rule).
int gdn_run_batch(const void* q, const void* k, const void* v, const float* g, const void* beta, void* o,
                  float* workspace, size_t workspace_bytes, const int* row0, const int* len, int nseq, int H, int HK,
                  float scale, const void* s_in, void* s_out, void* stream) {
    if (nseq <= 0 || nseq > MAX_SEQS || !row0 || !len || H <= 0 || HK <= 0 || H % HK != 0) return cudaErrorInvalidValue;
    const float* si = static_cast<const float*>(s_in);
    float* so = static_cast<float*>(s_out);
    cudaStream_t st = as_stream(stream);
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(workspace) || !aligned16(o) ||
        (si && !aligned16(si)) || (so && !aligned16(so)))
        return cudaErrorInvalidValue;
    Seqs seqs{};
    seqs.n = nseq;
    int longest = 0;
    long rows = 0;
    for (int i = 0; i < nseq; i++) {
        if (len[i] <= 0 || row0[i] < 0) return cudaErrorInvalidValue;
        seqs.row0[i] = row0[i];
        seqs.len[i] = len[i];
        seqs.chunk0[i] = seqs.chunks;
        seqs.chunks += (len[i] + C - 1) / C;
        longest = std::max(longest, len[i]);
        rows = std::max<long>(rows, (long)row0[i] + len[i]);
    }
    const Layout layout(seqs.chunks * C, H);
    if (workspace_bytes != 0 && layout.total > workspace_bytes) return cudaErrorInvalidValue;
    static bool prep_done[64] = {}, scan_done[64] = {};
    cudaError_t e = set_smem_once(gdn_prep_tc5, PREP_SMEM, prep_done);
    if (e != cudaSuccess) return e;
    e = set_smem_once(gdn_scan_tc5, SCAN_SMEM, scan_done);
    if (e != cudaSuccess) return e;
    const Work ws = split(workspace, seqs.chunks * C, H);
    CUtensorMap map_v;  // [64 rows, 64 columns] boxes over all the packed rows, 128-byte swizzle
    if (!tensor_map_2d(v, (uint64_t)rows, (uint64_t)H * D, (uint64_t)H * D, C, &map_v)) return CS1_ERR_TENSOR_MAP;
    e = launch_dep_family(DEP_GDN, gdn_prep_tc5, dim3((longest + C - 1) / C, H, nseq), PREP_THREADS, PREP_SMEM, st, map_v,
                          static_cast<const bf16*>(q), static_cast<const bf16*>(k), g, static_cast<const bf16*>(beta), ws, seqs,
                          H, HK, scale);
    if (e != cudaSuccess) return e;
    e = launch_dep_family(DEP_GDN, gdn_scan_tc5, dim3(H, D / VS, nseq), SCAN_THREADS, SCAN_SMEM, st, ws, static_cast<bf16*>(o),
                          seqs, H, si, so);
    return e != cudaSuccess ? e : cudaGetLastError();
}

int gdn_run(const void* q, const void* k, const void* v, const float* g, const void* beta, void* o,
            float* workspace, int T, int H, int HK, float scale, const void* s_in, void* s_out, void* stream) {
    if (T < 0 || H <= 0 || HK <= 0 || H % HK != 0) return cudaErrorInvalidValue;
    if (T == 0) {
        // no tokens: the state passes through unchanged
        if (s_out == nullptr) return cudaSuccess;
        const size_t bytes = (size_t)H * D * D * sizeof(float);
        return s_in != nullptr ? cudaMemcpyAsync(s_out, s_in, bytes, cudaMemcpyDeviceToDevice, as_stream(stream))
                               : cudaMemsetAsync(s_out, 0, bytes, as_stream(stream));
    }
    const int zero = 0;
    return gdn_run_batch(q, k, v, g, beta, o, workspace, 0, &zero, &T, 1, H, HK, scale, s_in, s_out, stream);
}

}  // namespace
}  // namespace s1

using namespace s1;

// The device error word of the delta-rule kernels on the current device (0 = no bounded wait
// ever gave up) after waiting for all queued work; cleared by the call.
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

// Several sequences of one pack in one pair of launches: sequence i is rows [row0[i], row0[i] +
// len[i]) of the packed q, k, v, g, beta and o (nseq <= 16, the pack limit); all start from the
// same state s_in (nullable: zero) - the candidates of one captured prefix - and sequence i
// leaves its state in s_out + i H 128 128 (nullable). Bit for bit what nseq calls of
// cs1_gdn_prefill_x compute. The workspace must hold cs1_gdn_workspace_floats(64 * chunks, H)
// floats, chunks = sum of ceil(len[i] / 64); workspace_floats is what the caller has.
extern "C" int s1_gdn_prefill_batch(const void* q, const void* k, const void* v, const float* g, const void* beta,
                                    void* o, float* workspace, size_t workspace_floats, const int* row0, const int* len,
                                    int nseq, int H, int HK, float scale, const void* s_in, void* s_out, void* stream) {
    if (workspace_floats == 0) return cudaErrorInvalidValue;
    return gdn_run_batch(q, k, v, g, beta, o, workspace, workspace_floats * sizeof(float), row0, len, nseq, H, HK, scale, s_in,
                         s_out, stream);
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
//     (64 MiB: for example 1792 tokens at 32 value heads, 1152 at 48, 3584 at 16); anything
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
