// Causal GQA flash attention for sm_100a on tcgen05: one block per (128 query rows, query head,
// sequence); a launch covers the sequences of a pack (a table of up to 16 is a kernel parameter).
//
//   warp 0    TMA producer: the Q tile once, then K and V tiles of BN keys through two stages
//             each ([64 rows, 64 columns] boxes, 128-byte swizzle)
//   warp 1    one thread issues the MMAs: S = Q K^T (128 x BN, K-major operands from shared
//             memory) into one of two score buffers in tensor memory, and O += P V (128 x Dh) with
//             P read from tensor memory (where the softmax threads left it, over the scores) and V
//             MN-major from shared memory, as it lies in global memory; O stays in tensor memory
//   warps 2-9 two threads per query row (warps w and w + 4 share the rows of one quarter of
//             tensor memory, each takes half of the columns): tcgen05.ld the scores, scale,
//             causal mask, online softmax in base 2 (the two halves exchange only their row
//             maximum, through shared memory; the exponent offset of a row moves only when its
//             maximum has grown by 2^8, so O is rescaled on few tiles; every fourth exponential
//             is a cubic on the FMA pipe), tcgen05.st P (bf16) back into tensor memory, and at the
//             end normalise, gate and store.
//
// Head dim 128 runs key tiles of 64 and two blocks per SM, so that one block's MMAs and copies
// run under the other's softmax; head dim 256 key tiles of 128 and one block per SM. The score
// MMA of tile j + 1 is issued before the P V MMA of tile j, so it runs under tile j's softmax.
// Arithmetic contract as in the reference's kernel (attention.cu:110-233 there): P rounded to
// bf16 before P V, the row sum taken from the unrounded p, output divided by the sum, then the
// gate. A row's result does not depend on where its 128-row block starts, only on the key tiling
// (tiles of BN from position 0), so windows that start at a multiple of 64 repeat the one-shot
// arithmetic. Every barrier wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "attention_tc5.h"
#include "common.cuh"
#include "cs1_ops.h"
#include "status.h"
#include "tc5.cuh"
#include "tmap.h"

namespace s1 {
namespace {

constexpr int ABM = 128;       // query rows per block
constexpr int ATHREADS = 320;  // producer warp, MMA warp, eight softmax warps

#ifndef ATTN_TWO_PER_SM
#define ATTN_TWO_PER_SM 1  // head dim 128: key tiles of 64 and two blocks to an SM
#endif

template <int DH>
struct ACfg {
    // Head dim 128 runs with key tiles of 64 so that two blocks fit an SM (99 KB of shared memory
    // and 256 tensor-memory columns each): one block's MMAs and copies then run under the other's
    // softmax, which is what bounds a block.
    static constexpr bool TWO = DH == 128 && ATTN_TWO_PER_SM;
    static constexpr int BN = DH == 256 || TWO ? 64 : 128;   // keys per tile
    static constexpr int Q_BYTES = ABM * DH * 2;       // DH / 64 boxes of [128 rows, 64 columns]
    static constexpr int KV_BYTES = BN * DH * 2;       // one K or V tile: DH / 64 column boxes of [BN rows, 64]
    static constexpr int OFF_K = Q_BYTES;
    static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;
    static constexpr int OFF_BAR = OFF_V + 2 * KV_BYTES;   // P has no tile here: it goes back into tensor memory
    static constexpr int OFF_X = OFF_BAR + 256;        // float [2][2][128]: row maxima (and sums) of the two halves
    // 99 KB (Dh 128), 195 KB (Dh 256); Dh 64 needs 83 KB and asks for 120 so that two blocks never share
    // an SM (each allocates all 512 tensor-memory columns)
    static constexpr int SMEM = TWO ? OFF_X + 2048 + 1024 : (OFF_X + 2048 + 1024) > 120 * 1024 ? (OFF_X + 2048 + 1024) : 120 * 1024;
    static constexpr int O_COL = 2 * BN;               // tensor memory: two score buffers, then the output
    static constexpr int TMEM_COLS = TWO ? 256 : 512;
    static constexpr int BLOCKS_PER_SM = TWO ? 2 : 1;
    static_assert(!TWO || (2 * (SMEM + 1024) <= 227 * 1024 && O_COL + DH <= TMEM_COLS), "two blocks share an SM");
};

__device__ int g_attn_error = 0;

struct AttnMaps {
    CUtensorMap q, k, v, kpre, vpre;
};

// ex2.approx: the exponentials of the softmax (2 ulp; the row sum and P carry the same value).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 2^x for x <= 0 (and a little above) without the special-function unit, which the softmax
// otherwise saturates (16 results per clock and SM against 128 FMAs): the integer below x taken
// from the low mantissa bits of x + 1.5 * 2^23 rounded down, a cubic for 2^fraction (relative
// error 8.6e-5, far below the bf16 step P is rounded to), the exponent put in by an integer add.
// Arguments below -127, -inf included, give exactly 0.
__device__ __forceinline__ float poly_exp2(float x) {
    x = fmaxf(x, -127.f);
    const float t = __fadd_rd(x, 12582912.f);
    const float f = x - (t - 12582912.f);
    float p = fmaf(0.07706612f, f, 0.22764599f);
    p = fmaf(p, f, 0.69511658f);
    p = fmaf(p, f, 1.f);
    return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}
#ifndef ATTN_POLY_EVERY
#define ATTN_POLY_EVERY 4  // every n-th exponential of a row goes to the FMA pipe; 0 = none
#endif

// The eight softmax warps. Warp 2 + i and warp 6 + i (i = 0..3) own the 32 query rows of tensor
// memory lanes [32 ((2 + i) & 3), +32); the first takes the lower half of the score and output
// columns, the second the upper half.
template <int DH, bool GATED, bool CAUSAL>
__device__ __forceinline__ void softmax_rows(unsigned char* smem, uint64_t* bars, uint32_t tmem_base,
                                             volatile int* abort_flag, const bf16* __restrict__ gate,
                                             bf16* __restrict__ out, int T, int Hq, int h, int q0, int own_base, int ntiles,
                                             float scale_log2, int vec_ok, int warp, int lane) {
    using namespace tc5;
    using G = ACfg<DH>;
    constexpr int BN = G::BN;
    constexpr int HN = BN / 2;   // score columns per thread
    constexpr int HD = DH / 2;   // output columns per thread
    uint64_t *s_full = bars + 9, *s_empty = bars + 11, *p_full = bars + 13, *o_done = bars + 14;
    float* xchg = reinterpret_cast<float*>(smem + G::OFF_X);  // [2][2][128]
    const int quarter = warp & 3, hf = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const int row = q0 + r;
    const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16);
    auto fail = [&](int code) {
        atomicCAS(&g_attn_error, 0, code);
        *abort_flag = 1;
    };
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    // Every one of the 256 threads runs every iteration and meets the others at the named
    // barrier, also after a wait has given up (ok = false): nobody is left waiting there.
#pragma unroll 1
    for (int j = 0; j < ntiles; j++) {
        const int b = j & 1;
        if (ok && !mbar_wait(&s_full[b], (j >> 1) & 1, abort_flag)) {
            fail(31);
            ok = false;
        }
        uint32_t sv[HN];
        float mx = -INFINITY;
        if (ok) {
            fence_after_sync();
#pragma unroll
            for (int cc = 0; cc < HN / 32; cc++)
                tmem_ld_32x32(t_row + b * BN + hf * HN + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[cc * 32]));
            tmem_ld_wait();
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[b]);
            const int k0 = j * BN + hf * HN;
            if (CAUSAL ? k0 + HN - 1 > row : k0 + HN > T) {  // causal: keys after the row; else: keys past the end
#pragma unroll
                for (int i = 0; i < HN; i++)
                    if (CAUSAL ? k0 + i > row : k0 + i >= T) sv[i] = 0xff800000u;  // -inf
            }
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four short chains instead of one long one
#pragma unroll
            for (int i = 0; i < HN; i++) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(sv[i]));
            mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        }
        // the row maximum over both halves; the buffers alternate, so one barrier per tile is enough
        xchg[(b * 2 + hf) * ABM + r] = mx;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (!ok) continue;
        mx = fmaxf(mx, xchg[(b * 2 + (hf ^ 1)) * ABM + r]);
        // m is the offset the exponentials are taken against, not necessarily the running maximum: it
        // moves only when the maximum has grown by more than 8 (in log2 units) past it. Until then the
        // exponentials stay below 2^8 - nothing for float32 sums or bf16 P - and the accumulator and the
        // row sum need no rescaling, which saves a round trip of O through the registers on most tiles
        // (with the exact maximum nearly every tile of the first few thousand keys moves some row's).
        // Both threads of a row see the same m and mx, so they decide alike.
        const float top = fmaxf(m, mx * scale_log2);
        const bool move = top > m + 8.f;
        const float mn = move ? top : m;
        const float alpha = move ? fast_exp2(m - mn) : 1.f;
        m = mn;
        float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < HN; i++) {
            const float arg = __uint_as_float(sv[i]) * scale_log2 - mn;
            const float p = ATTN_POLY_EVERY > 0 && i % ATTN_POLY_EVERY == ATTN_POLY_EVERY - 1 ? poly_exp2(arg) : fast_exp2(arg);
            sv[i] = __float_as_uint(p);
            s4[i & 3] += p;
        }
        l = l * alpha + ((s4[0] + s4[1]) + (s4[2] + s4[3]));

        if (j > 0) {
            // P V of the previous tile is complete: the accumulator may be rescaled and P overwritten
            if (!mbar_wait(o_done, (j - 1) & 1, abort_flag)) {
                fail(32);
                ok = false;
                continue;
            }
            fence_after_sync();
            if (__any_sync(__activemask(), alpha != 1.f)) {
#pragma unroll 1
                for (int cc = 0; cc < HD / 32; cc++) {
                    uint32_t o[32];
                    tmem_ld_32x32(t_row + G::O_COL + hf * HD + cc * 32, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st_32x32(t_row + G::O_COL + hf * HD + cc * 32, o);
                }
                tmem_st_wait();
            }
        }
        // P goes back into tensor memory as bf16, two keys to a column, over the first half of the
        // score buffer it came from (every thread of the block has taken its scores out of it: the
        // exchange of the row maxima lies in between); the P V product reads it from there as its A
        // operand. The next scores for this buffer are issued behind that product.
        {
            uint32_t pk[HN / 2];
#pragma unroll
            for (int i = 0; i < HN / 2; i++) pk[i] = pack2(__uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1]));
            if constexpr (HN == 64)
                tmem_st_32x32(t_row + b * BN + hf * (HN / 2), pk);
            else
                tmem_st_32x16(t_row + b * BN + hf * (HN / 2), pk);
            tmem_st_wait();
        }
        fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full);
    }
    // The row sum is the lower half's plus the upper half's, in that order for both threads. Every
    // thread comes here, also after a failed wait (the barrier counts all 256).
    xchg[hf * ABM + r] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (!ok || ntiles == 0) return;
    if (!mbar_wait(o_done, (ntiles - 1) & 1, abort_flag)) {
        fail(33);
        return;
    }
    fence_after_sync();
    const float inv = 1.f / (xchg[r] + xchg[ABM + r]);
    const size_t base = ((size_t)(row - own_base) * Hq + h) * DH + hf * HD;
#pragma unroll 1
    for (int cc = 0; cc < HD / 32; cc++) {
        uint32_t o[32];
        tmem_ld_32x32(t_row + G::O_COL + hf * HD + cc * 32, o);
        tmem_ld_wait();
        if (row >= T) continue;
        float y[32];
#pragma unroll
        for (int i = 0; i < 32; i++) y[i] = __uint_as_float(o[i]) * inv;
        if constexpr (GATED) {
            // attention -> bf16 store -> bf16 sigmoid -> multiply, without the store
            const uint32_t* gp = reinterpret_cast<const uint32_t*>(gate + base + cc * 32);
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const uint32_t gw = gp[i];
                y[2 * i] = rbf(y[2 * i]) * rbf(sigmoid(__uint_as_float(gw << 16)));
                y[2 * i + 1] = rbf(y[2 * i + 1]) * rbf(sigmoid(__uint_as_float(gw & 0xffff0000u)));
            }
        }
        bf16* dst = out + base + cc * 32;
        if (vec_ok) {
#pragma unroll
            for (int q = 0; q < 4; q++) {
                uint4 w;
                w.x = pack2(y[8 * q + 0], y[8 * q + 1]);
                w.y = pack2(y[8 * q + 2], y[8 * q + 3]);
                w.z = pack2(y[8 * q + 4], y[8 * q + 5]);
                w.w = pack2(y[8 * q + 6], y[8 * q + 7]);
                *reinterpret_cast<uint4*>(dst + 8 * q) = w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; i++) *reinterpret_cast<uint32_t*>(dst + 2 * i) = pack2(y[2 * i], y[2 * i + 1]);
        }
    }
}

// The sequences of one launch (a pack holds at most 16): sequence i has positions [0, T[i]) and its
// own rows - positions from own_base on - start at row row0[i] of q, k, v, gate and out.
constexpr int ATTN_MAX_SEQS = 16;
struct AttnSeqs {
    int n;
    int row0[ATTN_MAX_SEQS], T[ATTN_MAX_SEQS];
};

template <int DH, bool GATED, bool CAUSAL>
__global__ void __launch_bounds__(ATHREADS, ACfg<DH>::BLOCKS_PER_SM)
    attn_tc5_kernel(const __grid_constant__ AttnMaps maps, const bf16* __restrict__ gate, bf16* __restrict__ out,
                    const __grid_constant__ AttnSeqs seqs, int Hq, int Hk, float scale_log2, int q_base, int own_base,
                    int vec_ok) {
    using namespace tc5;
    using G = ACfg<DH>;
    constexpr int BN = G::BN;
    grid_dep_trigger();
    // Block index -> (query block, sequence, head), the heads and sequences of one query block next
    // to each other and the last query block first: under a causal mask a block's work grows with
    // its position, so the blocks are handed out longest first over the whole launch and its ragged
    // end is made of the shortest blocks (the heads of a query block also share their keys in L2).
    // The grid is as deep as the longest sequence: a block past its sequence's end has nothing to do.
    const int per_q = seqs.n * Hq;
    const int rest = blockIdx.x % per_q, sq = rest / Hq;
    const int h = rest % Hq, hk = h / (Hq / Hk);
    const int T = seqs.T[sq], row0 = seqs.row0[sq] - own_base;  // row of position p: row0 + p
    const int q0 = q_base + (gridDim.x / per_q - 1 - blockIdx.x / per_q) * ABM;
    if (q0 >= T) return;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + G::OFF_BAR);
    uint64_t* q_full = bars;          // 1
    uint64_t* k_full = bars + 1;      // 2
    uint64_t* v_full = bars + 3;      // 2
    uint64_t* k_empty = bars + 5;     // 2
    uint64_t* v_empty = bars + 7;     // 2
    uint64_t* s_full = bars + 9;      // 2
    uint64_t* s_empty = bars + 11;    // 2
    uint64_t* p_full = bars + 13;     // 1
    uint64_t* o_done = bars + 14;     // 1
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int kv_end = CAUSAL ? min(T, q0 + ABM) : T;
    const int ntiles = (kv_end + BN - 1) / BN;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; i++) {
            mbar_init(&k_full[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&s_empty[i], 8);
        }
        mbar_init(p_full, 8);
        mbar_init(o_done, 1);
        *abort_flag = 0;
        mbar_init_fence();
        prefetch_tmap(&maps.q);
        prefetch_tmap(&maps.k);
        prefetch_tmap(&maps.v);
    }
    if (warp == 2) {
        tmem_alloc(tmem_slot, G::TMEM_COLS);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    grid_dep_sync();
    auto fail = [&](int code) {
        atomicCAS(&g_attn_error, 0, code);
        *abort_flag = 1;
    };

    if (warp == 0) {
        {  // the whole warp runs the loop, one lane issues (addresses and counters stay warp-uniform)
            const bool issuer = elect_one();
            if (issuer) {
                mbar_expect_tx(q_full, G::Q_BYTES);
                for (int c = 0; c < DH / 64; c++)
                    tma_load_2d(smem + c * (ABM * 128), &maps.q, h * DH + c * 64, row0 + q0, q_full);
            }
            for (int j = 0; j < ntiles; j++) {
                const int stage = j & 1;
                const uint32_t parity = ((j >> 1) & 1) ^ 1;
                // a tile is BN / 64 groups of 64 keys; a group lies wholly in the prefix or in the window
                if (!mbar_wait(&k_empty[stage], parity, abort_flag)) {
                    fail(21);
                    break;
                }
                if (issuer) mbar_expect_tx(&k_full[stage], G::KV_BYTES);
                for (int c = 0; c < DH / 64 && issuer; c++)
                    for (int g = 0; g < BN / 64; g++) {
                        const int r0 = j * BN + g * 64;
                        unsigned char* dst = smem + G::OFF_K + stage * G::KV_BYTES + c * (BN * 128) + g * (64 * 128);
                        if (r0 < own_base)
                            tma_load_2d(dst, &maps.kpre, hk * DH + c * 64, r0, &k_full[stage]);
                        else
                            tma_load_2d(dst, &maps.k, hk * DH + c * 64, row0 + r0, &k_full[stage]);
                    }
                if (!mbar_wait(&v_empty[stage], parity, abort_flag)) {
                    fail(22);
                    break;
                }
                if (issuer) mbar_expect_tx(&v_full[stage], G::KV_BYTES);
                for (int c = 0; c < DH / 64 && issuer; c++)
                    for (int g = 0; g < BN / 64; g++) {
                        const int r0 = j * BN + g * 64;
                        unsigned char* dst = smem + G::OFF_V + stage * G::KV_BYTES + c * (BN * 128) + g * (64 * 128);
                        if (r0 < own_base)
                            tma_load_2d(dst, &maps.vpre, hk * DH + c * 64, r0, &v_full[stage]);
                        else
                            tma_load_2d(dst, &maps.v, hk * DH + c * 64, row0 + r0, &v_full[stage]);
                    }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        {
            const bool issuer = elect_one();
            constexpr uint32_t idesc_s = instr_desc(1, ABM, BN);
            constexpr uint32_t idesc_o = instr_desc_b_mn(1, ABM, DH);
            const uint32_t q_addr = smem_addr(smem);
            bool ok = mbar_wait(q_full, 0, abort_flag);
            if (!ok) fail(23);
            // P V of tile t: A = P in tensor memory (K-major over keys, where the scores were), B = V tile read MN-major
            auto issue_pv = [&](int t) {
                const int stage = t & 1;
                if (!mbar_wait(p_full, t & 1, abort_flag)) {
                    fail(26);
                    return false;
                }
                if (!mbar_wait(&v_full[stage], (t >> 1) & 1, abort_flag)) {
                    fail(27);
                    return false;
                }
                fence_after_sync();
                const uint32_t v_addr = smem_addr(smem + G::OFF_V + stage * G::KV_BYTES);
                if (issuer) {
#pragma unroll
                    for (int kk = 0; kk < BN / 16; kk++) {
                        const uint64_t b = smem_desc_mn_sw128(v_addr + kk * 2048, BN * 128, 1024);
                        mma_bf16_ts(tmem_base + G::O_COL, tmem_base + stage * BN + kk * 8, b, idesc_o, (t > 0 || kk > 0) ? 1u : 0u);
                    }
                    mma_commit(&v_empty[stage]);
                    mma_commit(o_done);
                }
                return true;
            };
            for (int j = 0; ok && j < ntiles; j++) {
                const int stage = j & 1;
                const uint32_t use = (j >> 1) & 1;
                if (!mbar_wait(&k_full[stage], use, abort_flag)) {
                    fail(24);
                    ok = false;
                    break;
                }
                if (!mbar_wait(&s_empty[stage], use ^ 1, abort_flag)) {
                    fail(25);
                    ok = false;
                    break;
                }
                fence_after_sync();
                const uint32_t k_addr = smem_addr(smem + G::OFF_K + stage * G::KV_BYTES);
                if (issuer) {
#pragma unroll
                    for (int kk = 0; kk < DH / 16; kk++) {
                        const uint64_t a = smem_desc_sw128(q_addr + (kk / 4) * (ABM * 128) + (kk % 4) * 32);
                        const uint64_t b = smem_desc_sw128(k_addr + (kk / 4) * (BN * 128) + (kk % 4) * 32);
                        mma_bf16_ss(tmem_base + stage * BN, a, b, idesc_s, kk > 0 ? 1u : 0u);
                    }
                    mma_commit(&k_empty[stage]);
                    mma_commit(&s_full[stage]);
                }
                if (j > 0) ok = issue_pv(j - 1);
            }
            if (ok && ntiles > 0) issue_pv(ntiles - 1);
        }
        __syncwarp();
    } else {
        softmax_rows<DH, GATED, CAUSAL>(smem, bars, tmem_base, abort_flag, gate, out, T, Hq, h, q0, -row0, ntiles, scale_log2,
                                vec_ok, warp, lane);
    }

    // wind down: after an abort give copies and MMAs in flight time to land before the
    // shared memory and tensor memory are released
    if (*abort_flag) __nanosleep(1000000);
    fence_before_sync();
    __syncthreads();
    if (warp == 2) tmem_dealloc(tmem_base, G::TMEM_COLS);
}

template <int DH, bool GATED, bool CAUSAL = true>
int launch_attn(const AttnMaps& maps, const bf16* gate, bf16* out, const AttnSeqs& seqs, int Hq, int Hk, float scale,
                int q_base, int own_base, cudaStream_t st) {
    using G = ACfg<DH>;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 64) return cudaErrorInvalidDevice;
    if (!configured[dev]) {
        e = cudaFuncSetAttribute(attn_tc5_kernel<DH, GATED, CAUSAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    constexpr float LOG2E = 1.4426950408889634f;
    int longest = 0;
    for (int i = 0; i < seqs.n; i++) longest = max(longest, seqs.T[i]);
    const dim3 grid(((longest - q_base + ABM - 1) / ABM) * seqs.n * Hq);
    const int vec_ok = aligned16(out) && (!GATED || aligned16(gate));
    return launch_dep_family(DEP_ATTENTION, attn_tc5_kernel<DH, GATED, CAUSAL>, grid, ATHREADS, G::SMEM, st, maps, gate, out, seqs, Hq, Hk, scale * LOG2E,
                      q_base, own_base, vec_ok);
}

}  // namespace
}  // namespace s1

using namespace s1;

int s1_attn_tc5_batch(const bf16* q, const bf16* k, const bf16* v, int ldv, const bf16* gate, bf16* out, const int* row0,
                      const int* T, int nseq, int Hq, int Hk, int Dh, float scale, int q_base, const bf16* kpre,
                      const bf16* vpre, int ldvpre, int own_base, cudaStream_t st) {
    if (nseq <= 0 || nseq > ATTN_MAX_SEQS) return cudaErrorInvalidValue;
    AttnSeqs seqs{};
    seqs.n = nseq;
    uint64_t own_rows = 0;  // rows of q, k, v that the launch may address
    for (int i = 0; i < nseq; i++) {
        if (row0[i] < 0 || T[i] <= q_base) return cudaErrorInvalidValue;
        seqs.row0[i] = row0[i];
        seqs.T[i] = T[i];
        own_rows = std::max<uint64_t>(own_rows, (uint64_t)row0[i] + (uint64_t)(T[i] - own_base));
    }
    AttnMaps maps;
    if (!tensor_map_2d(q, own_rows, (uint64_t)Hq * Dh, (uint64_t)Hq * Dh, ABM, &maps.q) ||
        !tensor_map_2d(k, own_rows, (uint64_t)Hk * Dh, (uint64_t)Hk * Dh, 64, &maps.k) ||
        !tensor_map_2d(v, own_rows, (uint64_t)Hk * Dh, (uint64_t)ldv, 64, &maps.v))
        return CS1_ERR_TENSOR_MAP;
    if (own_base > 0) {
        if (!tensor_map_2d(kpre, (uint64_t)own_base, (uint64_t)Hk * Dh, (uint64_t)Hk * Dh, 64, &maps.kpre) ||
            !tensor_map_2d(vpre, (uint64_t)own_base, (uint64_t)Hk * Dh, (uint64_t)ldvpre, 64, &maps.vpre))
            return CS1_ERR_TENSOR_MAP;
    } else {
        maps.kpre = maps.k;
        maps.vpre = maps.v;
    }
    if (Dh == 256)
        return gate ? launch_attn<256, true>(maps, gate, out, seqs, Hq, Hk, scale, q_base, own_base, st)
                    : launch_attn<256, false>(maps, gate, out, seqs, Hq, Hk, scale, q_base, own_base, st);
    return gate ? launch_attn<128, true>(maps, gate, out, seqs, Hq, Hk, scale, q_base, own_base, st)
                : launch_attn<128, false>(maps, gate, out, seqs, Hq, Hk, scale, q_base, own_base, st);
}

int s1_attn_tc5(const bf16* q, const bf16* k, const bf16* v, int ldv, const bf16* gate, bf16* out, int T, int Hq, int Hk,
                int Dh, float scale, int q_base, const bf16* kpre, const bf16* vpre, int ldvpre, int own_base,
                cudaStream_t st) {
    const int zero = 0;
    return s1_attn_tc5_batch(q, k, v, ldv, gate, out, &zero, &T, 1, Hq, Hk, Dh, scale, q_base, kpre, vpre, ldvpre, own_base, st);
}

// Non-causal attention over all n positions, head dim 64, as many key-value heads as query heads
// (the vision tower's: 16 heads, cs1_vision_attention). v rows are ldv elements apart.
int s1_attn_tc5_full64(const bf16* q, const bf16* k, const bf16* v, int ldv, bf16* out, int n, int heads, float scale,
                       cudaStream_t st) {
    AttnMaps maps;
    if (!tensor_map_2d(q, (uint64_t)n, (uint64_t)heads * 64, (uint64_t)heads * 64, ABM, &maps.q) ||
        !tensor_map_2d(k, (uint64_t)n, (uint64_t)heads * 64, (uint64_t)heads * 64, 64, &maps.k) ||
        !tensor_map_2d(v, (uint64_t)n, (uint64_t)heads * 64, (uint64_t)ldv, 64, &maps.v))
        return CS1_ERR_TENSOR_MAP;
    maps.kpre = maps.k;
    maps.vpre = maps.v;
    AttnSeqs seqs{};
    seqs.n = 1;
    seqs.T[0] = n;
    return launch_attn<64, false, false>(maps, nullptr, out, seqs, heads, heads, scale, 0, 0, st);
}

// The device error word of the attention kernel on the current device (0 = no bounded wait ever
// gave up) after waiting for all queued work; cleared by the call.
extern "C" int s1_attn_tc5_status(int* code) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return e;
    int v = 0;
    e = cudaMemcpyFromSymbol(&v, g_attn_error, sizeof(int));
    if (e != cudaSuccess) return e;
    if (v != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_attn_error, &zero, sizeof(int));
    }
    *code = v;
    return e;
}

// Device address of this device's error word, for the executor's status copy.
int s1::attn_error_address(int** p) {
    void* a = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&a, s1::g_attn_error);
    *p = static_cast<int*>(a);
    return e;
}
