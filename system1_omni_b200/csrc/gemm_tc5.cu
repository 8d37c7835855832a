// bf16 GEMM y = x w^T for sm_100a on tcgen05: a persistent, warp-specialised kernel.
//
//   warp 0    TMA producer: streams 128 x 64 tiles of x and BN x 64 tiles of w (both K-major,
//             128-byte swizzled) through a ring of shared-memory stages
//   warp 1    one thread issues tcgen05.mma (128 x BN x 16 per instruction) into one of two
//             float32 accumulators in tensor memory and commits stage / accumulator barriers
//   warps 2-5 epilogue: tcgen05.ld the finished accumulator (one row per thread), round to
//             bf16 and store, while the MMA warp already fills the other accumulator
//
// Tiles are assigned round-robin to the resident blocks with all row-blocks of one column
// block adjacent, so a w tile is fetched from HBM once and then served from L2. Rows past M,
// columns past N and a K tail are zero-filled by TMA and masked in the epilogue. Every block
// fetches its own tiles (no load is shared across blocks by the copy engine). Every barrier
// wait is bounded; a wait that runs out records a code in a device error word (read with
// s1_gemm_tc5_status) and the block winds down.
//
// Two kernels: gemm_tc5_kernel, one block per 128 x BN tile, for up to 128 rows; and
// gemm_tc5_pair_kernel for more rows, where the two blocks of a cluster work as a pair on a
// 256 x BN tile (tcgen05 cta_group::2): each block loads its 128 rows of x and only half of
// the w tile, the pair leader issues one MMA that reads both halves, and each block keeps and
// stores its own 128 rows of the result. That cuts the shared-memory fill per flop by a third
// and lets BN be any multiple of 32, chosen per problem so that the tile count fills whole
// waves of the 74 pairs.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <math.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "cs1_ops.h"
#include "gemm_tc5.h"
#include "status.h"
#include "tc5.cuh"

namespace s1 {
namespace {

constexpr int BM = 128, BK = 64;
constexpr int GEMM_THREADS = 192;

template <int BN>
struct Cfg {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE = A_BYTES + B_BYTES;
    static constexpr int STAGES = (192 * 1024) / STAGE;
    static constexpr int TMEM_COLS = 2 * BN;  // two accumulators; 128, 256 or 512 columns
    static constexpr int BAR_BYTES = 256;
    static constexpr int SMEM = STAGES * STAGE + BAR_BYTES + 1024;  // + slack to align to 1024
};

__device__ int g_gemm_error = 0;

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_tc5_kernel(const __grid_constant__ CUtensorMap tma_x, const __grid_constant__ CUtensorMap tma_w,
                    bf16* __restrict__ y, int M, int N, int K, int ldy, int vec_ok, int splits,
                    const bf16* __restrict__ bias) {
    using namespace tc5;
    using G = Cfg<BN>;
    grid_dep_trigger();
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + G::STAGES * G::STAGE);
    uint64_t* empty = full + G::STAGES;
    uint64_t* tfull = empty + G::STAGES;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (threadIdx.x == 0) {
        for (int s = 0; s < G::STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&tfull[a], 1);
            mbar_init(&tempty[a], 4);
        }
        *abort_flag = 0;
        mbar_init_fence();
        prefetch_tmap(&tma_x);
        prefetch_tmap(&tma_w);
    }
    if (warp == 2) {
        tmem_alloc(tmem_slot, G::TMEM_COLS);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int num_m = (M + BM - 1) / BM, num_n = (N + BN - 1) / BN;
    const int tiles = num_m * num_n, kblocks = (K + BK - 1) / BK;
    // splits > 1: the launch is made of clusters of `splits` blocks, one cluster per tile, and
    // the block of cluster rank r accumulates the r-th share of the k-blocks
    const uint32_t crank = splits > 1 ? cluster_ctarank() : 0u;
    const int kb_per = (kblocks + splits - 1) / splits;
    const int kb0 = (int)crank * kb_per, kb1 = min(kblocks, kb0 + kb_per);
    const int first = splits > 1 ? (int)blockIdx.x / splits : (int)blockIdx.x;
    const int step = splits > 1 ? tiles : (int)gridDim.x;
    constexpr int LDS = BN + 4;  // row pitch (floats) of the float32 tile staged for the cluster sum
    float* staged = reinterpret_cast<float*>(smem);
    auto fail = [&](int code) {
        atomicCAS(&g_gemm_error, 0, code);
        *abort_flag = 1;
    };

    if (warp == 0) {
        {  // the whole warp runs the loop, one lane issues (addresses and counters stay warp-uniform)
            const bool issuer = elect_one();
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            // The first ring-full of w tiles goes out before this kernel waits for the one ahead of
            // it on the stream: weights are written by no kernel of a forward pass, x may still be
            // in the making. (The stages are fresh, so there is nothing to wait for on `empty`.)
            int ahead = 0;
            if (first < tiles) {
                ahead = min(kb1 - kb0, G::STAGES);
                for (int i = 0; i < ahead && issuer; i++) {
                    mbar_expect_tx(&full[i], G::STAGE);
                    tma_load_2d(smem + i * G::STAGE + G::A_BYTES, &tma_w, (kb0 + i) * BK, (first / num_m) * BN, &full[i]);
                }
            }
            grid_dep_sync();
            for (int tile = first; ok && tile < tiles; tile += step) {
                const int m_idx = tile % num_m, n_idx = tile / num_m;
                for (int kb = kb0; kb < kb1; kb++) {
                    unsigned char* dst = smem + stage * G::STAGE;
                    if (tile != first || kb - kb0 >= ahead) {
                        if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
                            fail(1);
                            ok = false;
                            break;
                        }
                        if (issuer) {
                            mbar_expect_tx(&full[stage], G::STAGE);
                            tma_load_2d(dst + G::A_BYTES, &tma_w, kb * BK, n_idx * BN, &full[stage]);
                        }
                    }
                    if (issuer) tma_load_2d(dst, &tma_x, kb * BK, m_idx * BM, &full[stage]);
                    if (++stage == G::STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        {
            const bool issuer = elect_one();
            constexpr uint32_t idesc = instr_desc(1, BM, BN);
            uint32_t stage = 0, phase = 0, it = 0;
            bool ok = true;
            for (int tile = first; ok && tile < tiles; tile += step, it++) {
                const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
                if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) {
                    fail(3);
                    break;
                }
                fence_after_sync();
                const uint32_t d = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!mbar_wait(&full[stage], phase, abort_flag)) {
                        fail(2);
                        ok = false;
                        break;
                    }
                    fence_after_sync();
                    const uint32_t a_addr = smem_addr(smem + stage * G::STAGE);
                    const uint32_t b_addr = a_addr + G::A_BYTES;
                    if (issuer) {
#pragma unroll
                        for (int k = 0; k < BK / 16; k++) {
                            mma_bf16_ss(d, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), idesc,
                                        ((kb - kb0) | k) != 0);
                        }
                        mma_commit(&empty[stage]);
                    }
                    if (++stage == G::STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok && issuer) mma_commit(&tfull[acc]);
            }
        }
        __syncwarp();
    } else {
        grid_dep_sync();  // these warps store y, which the kernel ahead may still read
        const int quarter = warp & 3;  // tensor-memory lanes [32 quarter, 32 quarter + 32) belong to this warp
        uint32_t it = 0;
        for (int tile = first; tile < tiles; tile += step, it++) {
            const int m_idx = tile % num_m, n_idx = tile / num_m;
            const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
            if (!mbar_wait_idle(&tfull[acc], acc_phase, abort_flag)) {
                fail(4);
                break;
            }
            fence_after_sync();
            const int row = m_idx * BM + quarter * 32 + lane;
#pragma unroll 1
            for (int cc = 0; cc < BN / 32; cc++) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + cc * 32, v);
                tmem_ld_wait();
                const int col0 = n_idx * BN + cc * 32;
                if (splits > 1) {
                    // this block's share of the sum over k, float32, into the stage ring (all of its
                    // loads have been consumed: the accumulator barrier follows the last MMA)
                    if (row < M) {
                        float4* dst = reinterpret_cast<float4*>(staged + (quarter * 32 + lane) * LDS + cc * 32);
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            dst[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                 __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                    }
                } else if (row < M && col0 < N) {
                    bf16* dst = y + (size_t)row * ldy + col0;
                    if (bias) {  // joins the float32 sum before the one rounding (whole tiles only: splits == 1)
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (col0 + j < N) v[j] = __float_as_uint(__uint_as_float(v[j]) + f32(bias[col0 + j]));
                    }
                    if (vec_ok && col0 + 32 <= N) {
                        uint4 o[4];
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            o[j].x = pack2(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]));
                            o[j].y = pack2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
                            o[j].z = pack2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
                            o[j].w = pack2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
                        }
                        if (vec_ok == 2) {  // whole 32-byte sectors per store
                            st32(dst, o[0], o[1]);
                            st32(dst + 16, o[2], o[3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; j++) st16(dst + 8 * j, o[j]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (col0 + j < N) dst[j] = to_bf16(__uint_as_float(v[j]));
                    }
                }
            }
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[acc]);
        }
    }

    if (splits > 1) {
        // Sum over the cluster in rank order (the same order whatever the timing): every block reads
        // its share of the tile's elements from all the blocks' staged tiles through distributed
        // shared memory, rounds once and stores. Both cluster barriers are reached by every thread
        // of every block, also after a wait gave up, so no block is left waiting at one.
        __syncwarp();
        cluster_sync();
        if (!*abort_flag && first < tiles) {
            const int m_idx = first % num_m, n_idx = first / num_m;
            const int rows = min(BM, M - m_idx * BM);
            constexpr int Q = BN / 4;
            const int total = rows * Q;
            const int lo = (int)((long)total * crank / splits), hi = (int)((long)total * (crank + 1) / splits);
            uint32_t peer[8];
#pragma unroll
            for (int p = 0; p < 8; p++) peer[p] = p < splits ? map_to_rank(smem_addr(staged), p) : 0u;
            for (int idx = lo + (int)threadIdx.x; idx < hi; idx += GEMM_THREADS) {
                const int r = idx / Q, c4 = idx % Q;
                const uint32_t off = (uint32_t)(r * LDS + c4 * 4) * 4u;
                float4 part[8];
#pragma unroll
                for (int p = 0; p < 8; p++)
                    if (p < splits) part[p] = ld_cluster_f4(peer[p] + off);
                float4 sum = part[0];
#pragma unroll
                for (int p = 1; p < 8; p++)
                    if (p < splits) {
                        sum.x += part[p].x;
                        sum.y += part[p].y;
                        sum.z += part[p].z;
                        sum.w += part[p].w;
                    }
                const int col = n_idx * BN + c4 * 4;
                if (col < N) {
                    bf16* dst = y + (size_t)(m_idx * BM + r) * ldy + col;
                    if (vec_ok && col + 4 <= N) {
                        uint2 o;
                        o.x = pack2(sum.x, sum.y);
                        o.y = pack2(sum.z, sum.w);
                        *reinterpret_cast<uint2*>(dst) = o;
                    } else {
                        const float e[4] = {sum.x, sum.y, sum.z, sum.w};
                        for (int j = 0; j < 4; j++)
                            if (col + j < N) dst[j] = to_bf16(e[j]);
                    }
                }
            }
        }
        cluster_sync();  // no block leaves while another still reads its staged tile
    }

    // wind down: after an abort give copies and MMAs in flight time to land before the
    // shared memory and tensor memory are released
    if (*abort_flag) __nanosleep(1000000);
    fence_before_sync();
    __syncthreads();
    if (warp == 2) tmem_dealloc(tmem_base, G::TMEM_COLS);
}

// ---- CTA-pair kernel: 256 x BN tiles on two blocks of a cluster ----
constexpr int PAIR_MAX_STAGES = 12;
constexpr int PAIR_DATA_BYTES = 7 * 32768;         // the stage ring: as many stages as fit (7 at BN = 256, 11 at 64)
constexpr int PAIR_A_BYTES = BM * BK * 2;          // this block's 128 rows of x
constexpr int PAIR_SMEM = PAIR_DATA_BYTES + 256 + 1024;
constexpr int PAIR_TMEM_COLS = 512;                // two accumulators 256 columns apart
constexpr int PAIR_ACC_STRIDE = 256;

// Tile index -> (row block, column block) for the pair kernel. Blocks that run at the same time
// take consecutive indices and fetch the same k-block at the same time; requests for one
// x or w tile then coincide in L2. Walking GM = 8 row blocks per column block (instead of all of
// them) makes the 74 tiles in flight an 8 x 9 patch: 17 distinct operand tiles per k-block
// rather than num_m + 74 / num_m. The host widens the walk to 16 row blocks where their rows of x
// stay in L2 from one column block to the next (pair_walk): w then streams from HBM once per 16
// row blocks instead of once per 8.
__device__ __forceinline__ void pair_tile_coords(int tile, int num_m, int num_n, int GM, int& m, int& n) {
    const int per_group = GM * num_n;
    const int group = tile / per_group, in = tile - group * per_group;
    const int first = group * GM;
    const int gm = min(GM, num_m - first);
    m = first + in % gm;
    n = in / gm;
}

// One piece of work of a block pair: k-blocks [kb0, kb1) of one output tile. When the tile's
// K range is shared (nparts > 1) the piece is contributor `part` of `nparts` and leaves a
// float32 partial tile in slot slot_of(part); whichever contributor finishes last adds the
// slots in part order, so the sum does not depend on the arrival order.
struct Piece {
    int tile, kb0, kb1, part, nparts;
    int mode, first, splits;
    __device__ __forceinline__ size_t slot_of(int j) const {
        return mode == 0 ? (size_t)tile * splits + j : (size_t)(first + j) * 2 + (j == 0 ? 1 : 0);
    }
};

// Two ways of handing pieces to the pairs, identical in the three roles of a block.
//   mode 0: a tile's k-blocks are cut into `splits` equal parts (1 = whole tiles); the parts
//           go round-robin over the pairs.
//   mode 1: the k-blocks of all tiles, laid end to end, are cut into one contiguous run per
//           pair (lengths differ by at most one), and a run is cut at tile boundaries. A
//           pair has at most two pieces that share their tile: its first (a tile entered
//           part-way, slot 2*pair) and its last (a tile left before its end, slot 2*pair+1).
struct PieceIter {
    int mode, tiles, kblocks, splits, kb_per, npairs, pair;
    int unit;
    long long g, g1, per, extra;
    __device__ __forceinline__ void init(int mode_, int tiles_, int kblocks_, int splits_, int pair_, int npairs_) {
        mode = mode_, tiles = tiles_, kblocks = kblocks_, splits = splits_, pair = pair_, npairs = npairs_;
        kb_per = (kblocks + splits - 1) / splits;
        unit = pair;
        const long long total = (long long)tiles * kblocks;
        per = total / npairs, extra = total % npairs;
        g = (long long)pair * per + (pair < extra ? pair : extra);
        g1 = g + per + (pair < extra ? 1 : 0);
    }
    __device__ __forceinline__ int owner(long long at) const {
        const long long cut = extra * (per + 1);
        return (int)(at < cut ? at / (per + 1) : extra + (at - cut) / per);
    }
    __device__ __forceinline__ bool next(Piece& p) {
        p.mode = mode, p.splits = splits;
        if (mode == 0) {
            if (unit >= tiles * splits) return false;
            p.tile = unit / splits, p.part = unit % splits, p.nparts = splits, p.first = 0;
            p.kb0 = p.part * kb_per;
            p.kb1 = min(kblocks, (p.part + 1) * kb_per);
            unit += npairs;
            return true;
        }
        if (g >= g1) return false;
        p.tile = (int)(g / kblocks);
        p.kb0 = (int)(g - (long long)p.tile * kblocks);
        p.kb1 = (int)min((long long)kblocks, p.kb0 + (g1 - g));
        if (p.kb0 == 0 && p.kb1 == kblocks) {
            p.part = 0, p.nparts = 1, p.first = pair;
        } else {
            p.first = owner((long long)p.tile * kblocks);
            p.nparts = owner((long long)(p.tile + 1) * kblocks - 1) - p.first + 1;
            p.part = pair - p.first;
        }
        g += p.kb1 - p.kb0;
        return true;
    }
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
    gemm_tc5_pair_kernel(const __grid_constant__ CUtensorMap tma_x, const __grid_constant__ CUtensorMap tma_w,
                         bf16* __restrict__ y, int M, int N, int K, int ldy, int vec_ok, int BN, int splits, int mode,
                         float* __restrict__ partials, int* __restrict__ counters, int swiglu, int walk) {
    using namespace tc5;
    grid_dep_trigger();
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + PAIR_DATA_BYTES);  // used in the leader only
    uint64_t* empty = full + PAIR_MAX_STAGES;                              // one copy per block
    uint64_t* tfull = empty + PAIR_MAX_STAGES;                             // one copy per block
    uint64_t* tempty = tfull + 2;                                                   // used in the leader only
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_MAX_STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&tfull[a], 1);
            mbar_init(&tempty[a], 8);  // four epilogue warps in each block of the pair
        }
        *abort_flag = 0;
        mbar_init_fence();
        prefetch_tmap(&tma_x);
        prefetch_tmap(&tma_w);
    }
    if (warp == 2) {
        tmem_alloc_pair(tmem_slot, PAIR_TMEM_COLS);
        tmem_relinquish_pair();
    }
    fence_before_sync();
    __syncthreads();
    cluster_sync();  // both blocks' barriers exist before anything arrives on them
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // swiglu: w is [gate (N rows) | up (N rows)]; a tile pairs BN / 2 gate columns (loaded by the
    // pair's first block) with the same BN / 2 up columns (second block), so both land in one
    // accumulator and the epilogue writes BN / 2 columns of silu(gate) * up.
    const int num_m = (M + 2 * BM - 1) / (2 * BM), num_n = swiglu ? (N + BN / 2 - 1) / (BN / 2) : (N + BN - 1) / BN;
    const int tiles = num_m * num_n, kblocks = (K + BK - 1) / BK;
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    PieceIter pieces;
    pieces.init(mode, tiles, kblocks, splits, pair, npairs);
    Piece pc;
    const int half_n = BN / 2;
    // a stage holds this block's 128 rows of x and its half of the w tile; 1024-byte multiples
    // (BN is a multiple of 32), as the 128-byte swizzle needs
    const uint32_t stage_bytes = PAIR_A_BYTES + half_n * BK * 2;
    const uint32_t nstages = min((uint32_t)PAIR_MAX_STAGES, (uint32_t)PAIR_DATA_BYTES / stage_bytes);
    auto fail = [&](int code) {
        atomicCAS(&g_gemm_error, 0, code);
        *abort_flag = 1;
    };

    if (warp == 0) {
        {  // the whole warp runs the loop, one lane issues
            const bool issuer = elect_one();
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            // As in the single-block kernel: this block's w tiles of the first ring-full of stages go
            // out before the wait for the kernel ahead on the stream; x follows after it.
            bool more = pieces.next(pc);
            int ahead = 0;
            if (more) {
                int m_idx, n_idx;
                pair_tile_coords(pc.tile, num_m, num_n, walk, m_idx, n_idx);
                const int n0 = swiglu ? n_idx * half_n + (int)rank * N : n_idx * BN + (int)rank * half_n;
                ahead = min(pc.kb1 - pc.kb0, (int)nstages);
                for (int i = 0; i < ahead && issuer; i++) {
                    if (leader) mbar_expect_tx(&full[i], 2 * stage_bytes);  // both blocks' bytes land on it
                    tma_load_2d_pair(smem + i * stage_bytes + PAIR_A_BYTES, &tma_w, (pc.kb0 + i) * BK, n0, &full[i]);
                }
            }
            grid_dep_sync();
            for (bool first_piece = true; ok && more; first_piece = false, more = pieces.next(pc)) {
                int m_idx, n_idx;
                pair_tile_coords(pc.tile, num_m, num_n, walk, m_idx, n_idx);
                const int m0 = m_idx * 2 * BM + (int)rank * BM;
                const int n0 = swiglu ? n_idx * half_n + (int)rank * N : n_idx * BN + (int)rank * half_n;
                for (int kb = pc.kb0; kb < pc.kb1; kb++) {
                    unsigned char* dst = smem + stage * stage_bytes;
                    if (!first_piece || kb - pc.kb0 >= ahead) {
                        if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
                            fail(11);
                            ok = false;
                            break;
                        }
                        if (issuer) {
                            if (leader) mbar_expect_tx(&full[stage], 2 * stage_bytes);
                            tma_load_2d_pair(dst + PAIR_A_BYTES, &tma_w, kb * BK, n0, &full[stage]);
                        }
                    }
                    if (issuer) tma_load_2d_pair(dst, &tma_x, kb * BK, m0, &full[stage]);
                    if (++stage == nstages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (leader) {  // the whole warp runs the loop, one lane issues
            const bool issuer = elect_one();
            const uint32_t idesc = instr_desc(1, 2 * BM, BN);
            uint32_t stage = 0, phase = 0, it = 0;
            bool ok = true;
            for (; ok && pieces.next(pc); it++) {
                const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
                if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) {
                    fail(13);
                    break;
                }
                fence_after_sync();
                const uint32_t d = tmem_base + acc * PAIR_ACC_STRIDE;
                const int kb0 = pc.kb0, kb1 = pc.kb1;
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!mbar_wait(&full[stage], phase, abort_flag)) {
                        fail(12);
                        ok = false;
                        break;
                    }
                    fence_after_sync();
                    const uint32_t a_addr = smem_addr(smem + stage * stage_bytes);
                    const uint32_t b_addr = a_addr + PAIR_A_BYTES;
                    if (issuer) {
#pragma unroll
                        for (int k = 0; k < BK / 16; k++) {
                            mma_bf16_ss_pair(d, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), idesc,
                                             (kb > kb0 || k > 0) ? 1u : 0u);
                        }
                        mma_commit_pair(&empty[stage], 3);  // frees the stage in both blocks
                    }
                    if (++stage == nstages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok && issuer) mma_commit_pair(&tfull[acc], 3);  // wakes both blocks' epilogues
            }
        }
        __syncwarp();
    } else {
        grid_dep_sync();  // these warps store y and use the scratch of shared tiles, which the kernel ahead may still use
        const int quarter = warp & 3;
        uint32_t it = 0;
        int* last_flag = const_cast<int*>(abort_flag) + 1;  // shared word next to the abort flag
        for (; pieces.next(pc); it++) {
            const int tile = pc.tile;
            const bool shared_tile = pc.nparts > 1;
            int m_idx, n_idx;
            pair_tile_coords(tile, num_m, num_n, walk, m_idx, n_idx);
            const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
            if (!mbar_wait_idle(&tfull[acc], acc_phase, abort_flag)) {
                fail(14);
                break;
            }
            fence_after_sync();
            const int row_local = quarter * 32 + lane;
            const int row = m_idx * 2 * BM + (int)rank * BM + row_local;
            // this block's 128 x BN float32 partial of (tile, part), stored as [BN / 4][128][4] so
            // that the 32 rows a warp holds make one contiguous 512-byte access per column group
            float* mine = partials + (pc.slot_of(pc.part) * 2 + rank) * (size_t)(BM * BN) + (size_t)row_local * 4;
            if (swiglu) {
                const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * PAIR_ACC_STRIDE;
#pragma unroll 1
                for (int cc = 0; cc < half_n / 32; cc++) {
                    const int col0 = n_idx * half_n + cc * 32;
                    if (col0 >= N) break;
                    uint32_t g[32], u[32];
                    tmem_ld_32x32(t_row + cc * 32, g);
                    tmem_ld_32x32(t_row + half_n + cc * 32, u);
                    tmem_ld_wait();
                    if (row < M) {
                        // the unfused sequence rounds both projections to bf16 first, then
                        // bf16(bf16(silu(gate)) * up)
                        float o32[32];
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            o32[j] = rbf(silu_fast(rbf(__uint_as_float(g[j])))) * rbf(__uint_as_float(u[j]));
                        bf16* dst = y + (size_t)row * ldy + col0;
                        if (vec_ok && col0 + 32 <= N) {
                            uint4 o[4];
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                o[j].x = pack2(o32[8 * j + 0], o32[8 * j + 1]);
                                o[j].y = pack2(o32[8 * j + 2], o32[8 * j + 3]);
                                o[j].z = pack2(o32[8 * j + 4], o32[8 * j + 5]);
                                o[j].w = pack2(o32[8 * j + 6], o32[8 * j + 7]);
                            }
                            if (vec_ok == 2) {
                                st32(dst, o[0], o[1]);
                                st32(dst + 16, o[2], o[3]);
                            } else {
#pragma unroll
                                for (int j = 0; j < 4; j++) st16(dst + 8 * j, o[j]);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (col0 + j < N) dst[j] = to_bf16(o32[j]);
                        }
                    }
                }
                fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if (leader)
                        mbar_arrive(&tempty[acc]);
                    else
                        mbar_arrive_remote(&tempty[acc], 0);
                }
                continue;
            }
            bool others_done = false;
            if (shared_tile) {
                // When every other contributor has already left its partial tile, this piece adds
                // them to its accumulator, in the same part order, and writes the rows at once:
                // no partial tile of its own, no second pass.
                if (warp == 2 && lane == 0) {
                    int seen;
                    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];"
                                 : "=r"(seen)
                                 : "l"(counters + tile * 2 + (int)rank)
                                 : "memory");
                    *last_flag = seen == pc.nparts - 1;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                others_done = *last_flag != 0;
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            if (others_done) {
                __threadfence();
                const float* base = partials + (size_t)rank * (BM * BN) + (size_t)row_local * 4;
                const size_t slot_stride = (size_t)2 * BM * BN;
#pragma unroll 1
                for (int cc = 0; cc < BN / 32; cc++) {
                    const int col0 = n_idx * BN + cc * 32;
                    if (col0 >= N) break;
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * PAIR_ACC_STRIDE + cc * 32, v);
                    float sum[32];
                    for (int s = 0; s < pc.nparts; s++) {
                        if (s == pc.part) {
                            tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 32; j++) sum[j] = s == 0 ? __uint_as_float(v[j]) : sum[j] + __uint_as_float(v[j]);
                        } else {
                            const float* other = base + pc.slot_of(s) * slot_stride;
                            float4 p[8];
#pragma unroll
                            for (int j = 0; j < 8; j++)
                                p[j] = __ldcg(reinterpret_cast<const float4*>(other + (size_t)(cc * 8 + j) * (BM * 4)));
#pragma unroll
                            for (int j = 0; j < 8; j++) {
                                sum[4 * j] = s == 0 ? p[j].x : sum[4 * j] + p[j].x;
                                sum[4 * j + 1] = s == 0 ? p[j].y : sum[4 * j + 1] + p[j].y;
                                sum[4 * j + 2] = s == 0 ? p[j].z : sum[4 * j + 2] + p[j].z;
                                sum[4 * j + 3] = s == 0 ? p[j].w : sum[4 * j + 3] + p[j].w;
                            }
                        }
                    }
                    if (row < M) {
                        bf16* dst = y + (size_t)row * ldy + col0;
                        if (vec_ok && col0 + 32 <= N) {
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                uint4 o;
                                o.x = pack2(sum[8 * j + 0], sum[8 * j + 1]);
                                o.y = pack2(sum[8 * j + 2], sum[8 * j + 3]);
                                o.z = pack2(sum[8 * j + 4], sum[8 * j + 5]);
                                o.w = pack2(sum[8 * j + 6], sum[8 * j + 7]);
                                st16(dst + 8 * j, o);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (col0 + j < N) dst[j] = to_bf16(sum[j]);
                        }
                    }
                }
                fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if (leader)
                        mbar_arrive(&tempty[acc]);
                    else
                        mbar_arrive_remote(&tempty[acc], 0);
                }
                if (warp == 2 && lane == 0) counters[tile * 2 + (int)rank] = 0;  // ready for the next launch
                continue;
            }
#pragma unroll 1
            for (int cc = 0; cc < BN / 32; cc++) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * PAIR_ACC_STRIDE + cc * 32, v);
                tmem_ld_wait();
                const int col0 = n_idx * BN + cc * 32;
                if (shared_tile) {
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        *reinterpret_cast<uint4*>(mine + (size_t)(cc * 8 + j) * (BM * 4)) =
                            make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                } else if (row < M && col0 < N) {
                    bf16* dst = y + (size_t)row * ldy + col0;
                    if (vec_ok && col0 + 32 <= N) {
                        uint4 o[4];
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            o[j].x = pack2(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]));
                            o[j].y = pack2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
                            o[j].z = pack2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
                            o[j].w = pack2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
                        }
                        if (vec_ok == 2) {  // whole 32-byte sectors per store
                            st32(dst, o[0], o[1]);
                            st32(dst + 16, o[2], o[3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; j++) st16(dst + 8 * j, o[j]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (col0 + j < N) dst[j] = to_bf16(__uint_as_float(v[j]));
                    }
                }
            }
            fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (leader)
                    mbar_arrive(&tempty[acc]);
                else
                    mbar_arrive_remote(&tempty[acc], 0);
            }
            if (shared_tile) {
                // The piece that finishes last adds the tile's partial sums in part order (so the
                // result does not depend on which piece that is) and writes the bf16 rows.
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps of this block
                if (warp == 2 && lane == 0) {
                    const int done = atomicAdd(&counters[tile * 2 + (int)rank], 1);
                    *last_flag = done == pc.nparts - 1;
                    if (done == pc.nparts - 1) counters[tile * 2 + (int)rank] = 0;  // ready for the next launch
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const bool last = *last_flag != 0;
                asm volatile("bar.sync 1, 128;" ::: "memory");  // everyone has read the flag before it is reused
                if (last && row < M) {
                    __threadfence();
                    const float* mine_base = partials + (size_t)rank * (BM * BN) + (size_t)row_local * 4;
                    const size_t slot_stride = (size_t)2 * BM * BN;
                    const float* first = mine_base + pc.slot_of(0) * slot_stride;
#pragma unroll 1
                    for (int cc = 0; cc < BN / 32; cc++) {
                        const int col0 = n_idx * BN + cc * 32;
                        if (col0 >= N) break;
                        float sum[32];
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const float4 p =
                                __ldcg(reinterpret_cast<const float4*>(first + (size_t)(cc * 8 + j) * (BM * 4)));
                            sum[4 * j] = p.x, sum[4 * j + 1] = p.y, sum[4 * j + 2] = p.z, sum[4 * j + 3] = p.w;
                        }
                        for (int s = 1; s < pc.nparts; s++) {
                            const float* other = mine_base + pc.slot_of(s) * slot_stride;
#pragma unroll
                            for (int j = 0; j < 8; j++) {
                                const float4 p =
                                    __ldcg(reinterpret_cast<const float4*>(other + (size_t)(cc * 8 + j) * (BM * 4)));
                                sum[4 * j] += p.x, sum[4 * j + 1] += p.y, sum[4 * j + 2] += p.z, sum[4 * j + 3] += p.w;
                            }
                        }
                        bf16* dst = y + (size_t)row * ldy + col0;
                        if (vec_ok && col0 + 32 <= N) {
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                uint4 o;
                                o.x = pack2(sum[8 * j + 0], sum[8 * j + 1]);
                                o.y = pack2(sum[8 * j + 2], sum[8 * j + 3]);
                                o.z = pack2(sum[8 * j + 4], sum[8 * j + 5]);
                                o.w = pack2(sum[8 * j + 6], sum[8 * j + 7]);
                                st16(dst + 8 * j, o);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (col0 + j < N) dst[j] = to_bf16(sum[j]);
                        }
                    }
                }
            }
        }
    }

    if (*abort_flag) __nanosleep(1000000);
    fence_before_sync();
    __syncthreads();
    cluster_sync();  // the leader's MMAs read the peer's shared memory until here
    if (warp == 2) tmem_dealloc_pair(tmem_base, PAIR_TMEM_COLS);
}

// ---- host side ----

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
    static EncodeTiled fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiled>(p);
    }();
    return fn;
}

struct MapKey {
    const void* ptr;
    int rows, K, box_rows;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && K == o.K && box_rows == o.box_rows;
    }
};
struct MapHash {
    size_t operator()(const MapKey& k) const {
        size_t h = reinterpret_cast<size_t>(k.ptr);
        h = h * 1000003u ^ (size_t)k.rows;
        h = h * 1000003u ^ (size_t)k.K;
        h = h * 1000003u ^ (size_t)k.box_rows;
        return h;
    }
};

// Tensor map of a row-major [rows, K] bf16 matrix with a [box_rows, 64] box, 128-byte swizzle.
bool tensor_map(const void* ptr, int rows, int K, int box_rows, CUtensorMap* out) {
    static std::mutex lock;
    static std::unordered_map<MapKey, CUtensorMap, MapHash> cache;
    const MapKey key{ptr, rows, K, box_rows};
    std::lock_guard<std::mutex> hold(lock);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeTiled fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap map;
    const CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, map);
    *out = map;
    return true;
}

struct DeviceInfo {
    int sms = 0;
    bool smem_set[3] = {false, false, false};
    bool pair_smem_set = false;
    int cluster_room[3][9] = {};  // clusters of c blocks of the single-block kernel that fit the GPU at once; 0 = not asked yet, -1 = none
};

DeviceInfo* device_info(cudaError_t* err) {
    static DeviceInfo info[64];
    int dev = 0;
    *err = cudaGetDevice(&dev);
    if (*err != cudaSuccess) return nullptr;
    if (dev >= 64) {
        *err = cudaErrorInvalidDevice;
        return nullptr;
    }
    if (info[dev].sms == 0) {
        *err = cudaDeviceGetAttribute(&info[dev].sms, cudaDevAttrMultiProcessorCount, dev);
        if (*err != cudaSuccess) return nullptr;
    }
    return &info[dev];
}

// How the epilogue may store a row's 32-column chunk: 2 = 32-byte stores (whole sectors), 1 = 16-byte, 0 = by element.
int store_width(const void* y, int ldy) {
    if (ldy % 16 == 0 && (reinterpret_cast<uintptr_t>(y) & 31) == 0) return 2;
    return ldy % 8 == 0 && aligned16(y) ? 1 : 0;
}

template <int BN>
cudaError_t prepare(DeviceInfo* info, int slot) {
    if (info->smem_set[slot]) return cudaSuccess;
    using G = Cfg<BN>;
    cudaError_t e = cudaFuncSetAttribute(gemm_tc5_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM);
    if (e != cudaSuccess) return e;
    info->smem_set[slot] = true;
    return cudaSuccess;
}

// How many clusters of c blocks of gemm_tc5_kernel<BN> the GPU holds at once (its blocks take a
// whole SM each, and a cluster must fit one GPC).
template <int BN>
int cluster_room(DeviceInfo* info, int slot, int c) {
    if (c < 2 || c > 8) return 0;
    if (info->cluster_room[slot][c] == 0) {
        int n = 0;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(c * info->sms);
        cfg.blockDim = dim3(GEMM_THREADS);
        cfg.dynamicSmemBytes = Cfg<BN>::SMEM;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = c;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (prepare<BN>(info, slot) != cudaSuccess ||
            cudaOccupancyMaxActiveClusters(&n, gemm_tc5_kernel<BN>, &cfg) != cudaSuccess) {
            cudaGetLastError();
            n = 0;
        }
        info->cluster_room[slot][c] = n > 0 ? n : -1;
    }
    return info->cluster_room[slot][c] > 0 ? info->cluster_room[slot][c] : 0;
}

template <int BN>
int launch(const void* x, const void* w, void* y, int M, int N, int K, int ldy, DeviceInfo* info, int slot, int splits,
           cudaStream_t st, const bf16* bias = nullptr) {
    using G = Cfg<BN>;
    const cudaError_t e = prepare<BN>(info, slot);
    if (e != cudaSuccess) return e;
    CUtensorMap mx, mw;
    if (!tensor_map(x, M, K, BM, &mx) || !tensor_map(w, N, K, BN, &mw)) return CS1_ERR_TENSOR_MAP;
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int vec_ok = store_width(y, ldy);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits > 1 ? tiles * splits : (tiles < info->sms ? tiles : info->sms));
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = G::SMEM;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (splits > 1) {  // one cluster per tile, its blocks share the k-blocks
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = splits;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        n++;
    }
    if (dep_launch_gemm()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, gemm_tc5_kernel<BN>, mx, mw, static_cast<bf16*>(y), M, N, K, ldy, vec_ok, splits, bias);
}

// Plan for at most 128 rows: the column-block width and over how many blocks of a cluster a
// tile's k-blocks are shared. With so few rows the product streams w once, and the time is set
// by how many SMs pull on it and for how long. Measured on B200 (microseconds): a block takes a
// k-block every 0.30 to 0.38 whatever else runs (SMALL_KB_US, by width), all blocks together
// take w in at about 4.5 MB per microsecond at best, a launch costs about 4 from its first
// block's set-up to its last store, a launch of clusters 6.5 + 0.2 c (cluster placement, the
// staged float32 tiles, two cluster barriers and the sum through distributed shared memory),
// and every further wave of clusters about 6, of a persistent block's next tile about 1.
struct SmallPlan {
    int bn, splits;
    double us;  // the estimate it was chosen by
};
// Planner overrides for the schedule tests and for tuning runs (s1_gemm_plan_override); 0 = the
// planners decide. Process-wide, plain reads on the launch path.
struct PlanOverride {
    int bn = 0, splits = 0;
    int runs = 2;        // contiguous runs in the pair kernel: 0 never, 1 always, 2 by the estimate
    int small_rows = 0;  // up to this many rows the single-block kernel, above it the pair kernel
};
PlanOverride g_override;
constexpr double SMALL_KB_US[3] = {0.38, 0.31, 0.30};  // widths 256, 128, 64
constexpr double SMALL_W_BYTES_PER_US = 4.5e6;

// Whole tiles only (no K split: the executor's default, where a row's bits must not depend on the
// row count): the width alone is chosen, by what the blocks have to pull in. Every block reads its
// rows of w once from HBM and all of x from L2, and what a launch of n busy SMs takes in per
// microsecond was measured to saturate as 9.8 (1 - exp(-n / 62)) MB (27B-shaped projections at 81
// rows, widths 64 to 256: 2.5 MB/us on 20 SMs, 4.6-5.0 on 40, 6.9-7.2 on 80, 8.9 on 112-129), with
// w itself bounded by 6.3 MB/us of HBM; a launch costs 4 us beside that. Narrow tiles put more SMs
// to work but fetch x more often; the estimate below weighs the two.
SmallPlan small_plan_whole(int M, int N, int K, DeviceInfo* info) {
    const int rows = M < BM ? M : BM;
    const double w_mb = (double)N * K * 2.0 / 1e6, x_mb = (double)rows * K * 2.0 / 1e6;
    const int widths[3] = {256, 128, 64};
    SmallPlan best{64, 1, 1e30};
    auto intake = [](double busy) { return 9.8 * (1.0 - exp(-busy / 62.0)); };
    for (int i = 0; i < 3; i++) {
        const int bn = widths[i];
        if (g_override.bn && bn != g_override.bn) continue;
        const long tiles = (long)((M + BM - 1) / BM) * ((N + bn - 1) / bn);
        // a block has one tile: tiles beyond the SM count run as a further wave, which lasts as long
        // as its blocks need for their bytes (an SM takes in 0.125 MB/us at most)
        const double block_mb = (double)bn * K * 2.0 / 1e6 + x_mb;
        const long full = tiles / info->sms, rest = tiles % info->sms;
        auto wave = [&](double blocks) {
            const double all = blocks * block_mb / intake(blocks), one = block_mb / 0.125;
            return all > one ? all : one;
        };
        double pull = (double)full * wave((double)info->sms);
        if (rest) pull += wave((double)rest);
        const double hbm = w_mb / 6.3;
        const double cost = 4.0 + (pull > hbm ? pull : hbm);
        if (cost < best.us - 1e-9) best = SmallPlan{bn, 1, cost};
    }
    return best;
}

SmallPlan small_plan(int M, int N, int K, DeviceInfo* info, bool may_split) {
    if (!may_split && !g_override.splits && M <= BM) return small_plan_whole(M, N, K, info);  // measured at one row block only
    const int kblocks = (K + BK - 1) / BK;
    const int rows = M < BM ? M : BM;
    const int force_bn = g_override.bn, force_s = g_override.splits;
    const int widths[3] = {256, 128, 64};
    SmallPlan best{64, 1, 1e30};
    double best_cost = 1e30;
    for (int i = 0; i < 3; i++) {
        const int bn = widths[i];
        if (force_bn && bn != force_bn) continue;
        const long tiles = (long)((M + BM - 1) / BM) * ((N + bn - 1) / bn);
        const double kb_us = SMALL_KB_US[i] + 0.015 * rows / BM;
        const double stream_us = (double)N * K * 2.0 / SMALL_W_BYTES_PER_US;
        for (int c = 1; c <= (may_split ? 8 : 1); c++) {
            if (force_s && c != force_s) continue;
            const int kb_per = (kblocks + c - 1) / c;
            long room = info->sms;
            if (c > 1) {
                if ((c - 1) * kb_per >= kblocks || kb_per < 4) continue;
                room = i == 0 ? cluster_room<256>(info, 0, c) : i == 1 ? cluster_room<128>(info, 1, c) : cluster_room<64>(info, 2, c);
                if (room <= 0) continue;
            }
            const long waves = (tiles + room - 1) / room;
            const double busy = (double)waves * kb_per * kb_us;
            const double cost = (c > 1 ? 6.5 + 0.2 * c : 4.0) + (waves - 1) * (c > 1 ? 6.0 : 1.0) + (busy > stream_us ? busy : stream_us);
            if (cost < best_cost - 1e-9) {
                best_cost = cost;
                best = SmallPlan{bn, c, cost};
            }
        }
    }
    // One row block: whole tiles as the intake model sees them, where that is clearly ahead of what
    // this estimate found (the wide projections, which it takes for bound by one streaming rate
    // whatever the width; on small problems the intake model runs low and does not get the say).
    if (M <= BM && !force_s) {
        const SmallPlan whole = small_plan_whole(M, N, K, info);
        if (whole.us < 0.85 * best_cost) return whole;
    }
    return best;
}

// Plan for the pair kernel: the column-block width (a multiple of 32) and how the k-blocks
// are handed out -- whole tiles, `splits` equal parts per tile, or one contiguous run of all
// tiles' k-blocks per pair -- by an estimate in microseconds built from measurements (4B- and
// 27B-shaped projections at 1024 and 4096 rows, widths 64 to 256, all three schedules): a
// k-block of a 256 x bn tile takes 0.00115 (bn + 28) us (the tensor pipe at 85 % of its peak: the
// width is what counts), a wave of tiles about 5 us beside its k-blocks (fill, drain and the
// ragged end of a wave), a launch 3; sharing a tile between s pairs costs about 1.7 s^2 for the
// float32 partial tiles summed by the last piece, and a k-block of a run 1.3 times a tile's
// (pairs at different k share no operand tiles in L2). Sharing needs float32 room for every
// partial tile.
struct PairPlan {
    int bn, splits, mode;
    double us;  // the estimate it was chosen by
};
constexpr double PAIR_KB_US = 0.00115, PAIR_KB_BASE = 28.0, PAIR_WAVE_US = 5.0, PAIR_LAUNCH_US = 3.0;
constexpr double SPLIT_FIXUP_US = 1.7;   // x s^2
constexpr double RUN_KB_COST = 1.3;

PairPlan pair_plan(int M, int N, int K, int pairs, size_t partial_bytes, int counter_slots) {
    const long num_m = (M + 2 * BM - 1) / (2 * BM);
    const int kblocks = (K + BK - 1) / BK;
    const int force_bn = g_override.bn, force_s = g_override.splits, force_run = g_override.runs;
    PairPlan best{256, 1, 0, 1e30};
    for (int bn = 256; bn >= 64; bn -= 32) {
        if (force_bn && bn != force_bn) continue;
        const long tiles = num_m * ((N + bn - 1) / bn);
        const double kb_us = PAIR_KB_US * (bn + PAIR_KB_BASE);
        for (int s = 1; s <= 8 && force_run != 1; s++) {
            if (force_s && s != force_s) continue;
            const int kb_per = (kblocks + s - 1) / s;
            if (s > 1) {
                if ((s - 1) * kb_per >= kblocks) continue;  // an empty part
                if (kb_per < 8) continue;
                if ((size_t)tiles * s * 2 * BM * bn * 4 > partial_bytes || tiles * 2 > counter_slots) continue;
            }
            const long waves = (tiles * s + pairs - 1) / pairs;
            const double cost = (double)waves * (kb_per * kb_us + PAIR_WAVE_US) + PAIR_LAUNCH_US + (s > 1 ? SPLIT_FIXUP_US * s * s : 0.0);
            if (cost < best.us - 1e-9) best = PairPlan{bn, s, 0, cost};
        }
        // contiguous runs: every pair gets total / pairs k-blocks in at most
        // ceil(run / kblocks) + 1 pieces, two of which share their tile
        const long total = tiles * kblocks;
        // Only for problems of at most two tiles per pair: measured, with many tiles the pairs
        // drift apart in k, stop sharing x and w tiles in L2, and every k-block gets slower.
        if (force_run != 0 && total >= pairs && (force_run == 1 || tiles <= 2 * pairs) &&
            (size_t)pairs * 2 * 2 * BM * bn * 4 <= partial_bytes && tiles * 2 <= counter_slots) {
            const long run = (total + pairs - 1) / pairs;
            const long pieces = (run + kblocks - 1) / kblocks + 1;
            // a tile is shared by about kblocks / run + 1 pairs, the last of which sums the others' partial tiles
            const double parts = (double)kblocks / (double)run + 1.0;
            const double cost = (double)run * kb_us * RUN_KB_COST + PAIR_WAVE_US * pieces + PAIR_LAUNCH_US + SPLIT_FIXUP_US * parts * parts;
            if (cost < best.us - 1e-9) best = PairPlan{bn, 1, 1, cost};
        }
    }
    return best;
}

// Row blocks walked per column block. 16 where that many blocks' rows of x (16 x 256 x K bf16) fit
// in a good third of the 126 MB L2 beside the w and y streams, else 8: the energy of the second
// HBM pass over w is what the wider walk saves (the kernel is tensor-bound either way, and runs
// under the board's power limit in long steps).
#ifndef PAIR_WALK_WIDE
#define PAIR_WALK_WIDE 1
#endif
int pair_walk(int M, int K) {
    const long num_m = (M + 2 * BM - 1) / (2 * BM);
    return PAIR_WALK_WIDE && num_m > 8 && (size_t)16 * 2 * BM * K * 2 <= ((size_t)48 << 20) ? 16 : 8;
}

int launch_pair(const void* x, const void* w, void* y, int M, int N, int K, int ldy, DeviceInfo* info,
                void* partials, size_t partial_bytes, int* counters, int counter_slots, cudaStream_t st) {
    if (!info->pair_smem_set) {
        const cudaError_t e =
            cudaFuncSetAttribute(gemm_tc5_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM);
        if (e != cudaSuccess) return e;
        info->pair_smem_set = true;
    }
    const int pairs = info->sms / 2;
    const PairPlan plan = pair_plan(M, N, K, pairs, partials && counters ? partial_bytes : 0, counter_slots);
    const int bn = plan.bn;
    CUtensorMap mx, mw;
    if (!tensor_map(x, M, K, BM, &mx) || !tensor_map(w, N, K, bn / 2, &mw)) return CS1_ERR_TENSOR_MAP;
    const int units = ((M + 2 * BM - 1) / (2 * BM)) * ((N + bn - 1) / bn) * plan.splits;
    const int grid = plan.mode == 1 ? 2 * pairs : 2 * (units < pairs ? units : pairs);
    const int vec_ok = store_width(y, ldy);
    return launch_dep_gemm(gemm_tc5_pair_kernel, grid, GEMM_THREADS, PAIR_SMEM, st, mx, mw, static_cast<bf16*>(y), M, N, K, ldy,
                      vec_ok, bn, plan.splits, plan.mode, static_cast<float*>(partials), counters, 0, pair_walk(M, K));
}

// Width of the gate/up tile (half of it gate columns, half up columns) for the fused kernel.
PairPlan swiglu_plan(int M, int I, int K, int pairs) {
    const long num_m = (M + 2 * BM - 1) / (2 * BM);
    const int kblocks = (K + BK - 1) / BK;
    PairPlan best{256, 1, 0, 1e30};
    for (int c = 256; c >= 64; c -= 64) {  // half of it a multiple of 32
        const long tiles = num_m * ((I + c / 2 - 1) / (c / 2));
        const double cost = (double)((tiles + pairs - 1) / pairs) * (kblocks * PAIR_KB_US * (c + PAIR_KB_BASE) + PAIR_WAVE_US) + PAIR_LAUNCH_US;
        if (cost < best.us - 1e-9) best = PairPlan{c, 1, 0, cost};
    }
    return best;
}

// act [M, I] = silu(x w_gate^T) * (x w_up^T) with w = [gate; up] stacked, [2 I, K]: both
// projections rounded to bf16 before the activation, as when they are stored and read back.
int launch_pair_swiglu(const void* x, const void* w, void* act, int M, int I, int K, int ld, DeviceInfo* info,
                       cudaStream_t st) {
    if (!info->pair_smem_set) {
        const cudaError_t e =
            cudaFuncSetAttribute(gemm_tc5_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM);
        if (e != cudaSuccess) return e;
        info->pair_smem_set = true;
    }
    const int pairs = info->sms / 2;
    const long num_m = (M + 2 * BM - 1) / (2 * BM);
    const int bn = swiglu_plan(M, I, K, pairs).bn;
    CUtensorMap mx, mw;
    if (!tensor_map(x, M, K, BM, &mx) || !tensor_map(w, 2 * I, K, bn / 2, &mw)) return CS1_ERR_TENSOR_MAP;
    const long tiles = num_m * ((I + bn / 2 - 1) / (bn / 2));
    const int grid = 2 * (int)(tiles < pairs ? tiles : pairs);
    const int vec_ok = store_width(act, ld);
    return launch_dep_gemm(gemm_tc5_pair_kernel, grid, GEMM_THREADS, PAIR_SMEM, st, mx, mw, static_cast<bf16*>(act), M, I, K, ld,
                      vec_ok, bn, 1, 0, static_cast<float*>(nullptr), static_cast<int*>(nullptr), 1, pair_walk(M, K));
}

// Which kernel takes a problem of more than 128 rows: the pair kernel, or the single-block kernel
// whose clusters share K. By the two planners' estimates; with few rows and a narrow result
// (N = 2560 ... 5120 at up to some 700 rows) the pair kernel has too few 256-row tiles to fill the
// GPU and its shared-tile schedules pay for partial tiles in global memory. The single-block
// estimate runs up to 20 % low with several row blocks (measured against both kernels on the
// projections of the three model sizes at 192 to 1024 rows), so it has to win by 15 %.
bool single_block_wins(double single_us, double pair_us, int M) {
    if (g_override.small_rows > 0) return M <= g_override.small_rows;
    return single_us < 0.85 * pair_us;
}

}  // namespace
}  // namespace s1

using namespace s1;

bool s1_gemm_tc5_supported(const void* x, const void* w, const void* y, int M, int N, int K, int ldy) {
    (void)y;
    (void)ldy;
    return M > 0 && N > 0 && K >= 64 && K % 8 == 0 && aligned16(x) && aligned16(w);
}

int s1_gemm_tc5(const void* x, const void* w, void* y, int M, int N, int K, int ldy, const S1GemmScratch* scratch,
                cudaStream_t st) {
    cudaError_t err;
    DeviceInfo* info = device_info(&err);
    if (!info) return err;
    // No scratch means the caller wants a sum over k whose order does not depend on the number of
    // rows, so the k-blocks of a tile stay in one block.
    const SmallPlan plan = small_plan(M, N, K, info, scratch != nullptr);
    // More than one row block: the CTA-pair kernel unless the single-block one is estimated faster
    if (M > BM) {
        const bool fix = scratch && scratch->partials && scratch->counters;
        const PairPlan pair = pair_plan(M, N, K, info->sms / 2, fix ? scratch->partial_bytes : 0, fix ? scratch->counter_slots : 0);
        if (!single_block_wins(plan.us, pair.us, M))
            return launch_pair(x, w, y, M, N, K, ldy, info, scratch ? scratch->partials : nullptr,
                               scratch ? scratch->partial_bytes : 0, scratch ? scratch->counters : nullptr,
                               scratch ? scratch->counter_slots : 0, st);
    }
    if (plan.bn == 256) return launch<256>(x, w, y, M, N, K, ldy, info, 0, plan.splits, st);
    if (plan.bn == 128) return launch<128>(x, w, y, M, N, K, ldy, info, 1, plan.splits, st);
    return launch<64>(x, w, y, M, N, K, ldy, info, 2, plan.splits, st);
}

bool s1_gemm_tc5_swiglu_supported(const void* x, const void* w, int M, int I, int K) {
    if (!(M > BM && I > 0 && K >= 64 && K % 8 == 0 && aligned16(x) && aligned16(w))) return false;
    cudaError_t err;
    DeviceInfo* info = device_info(&err);
    if (!info) return false;
    // the fused kernel is the pair kernel: against the single-block kernel on [gate | up] followed by
    // the SiLU-multiply as a kernel of its own (a launch and 6 bytes per element at about 3 TB/s)
    const double two_ops = small_plan(M, 2 * I, K, info, true).us + 2.5 + 6.0 * M * I / 3e6;
    return !single_block_wins(two_ops, swiglu_plan(M, I, K, info->sms / 2).us, M);
}

int s1_gemm_tc5_swiglu(const void* x, const void* w, void* act, int M, int I, int K, int ld, cudaStream_t st) {
    cudaError_t err;
    DeviceInfo* info = device_info(&err);
    if (!info) return err;
    return launch_pair_swiglu(x, w, act, M, I, K, ld, info, st);
}

// y = bf16(x w^T + bias) on the single-block kernel with whole tiles (the bias joins the float32
// sum in the epilogue), for any number of rows.
int s1_gemm_tc5_bias(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, int ldy, cudaStream_t st) {
    cudaError_t err;
    DeviceInfo* info = device_info(&err);
    if (!info) return err;
    const bf16* b = static_cast<const bf16*>(bias);
    const long t256 = (long)((M + BM - 1) / BM) * ((N + 255) / 256);
    if (t256 >= info->sms || N % 256 == 0) return launch<256>(x, w, y, M, N, K, ldy, info, 0, 1, st, b);
    const long t128 = (long)((M + BM - 1) / BM) * ((N + 127) / 128);
    if (t128 >= info->sms) return launch<128>(x, w, y, M, N, K, ldy, info, 1, 1, st, b);
    return launch<64>(x, w, y, M, N, K, ldy, info, 2, 1, st, b);
}

// Planner overrides for the schedule tests and for tuning runs: tile width (0 = planner's
// choice), K shares per tile (0 = planner's), contiguous runs in the pair kernel (0 never, 1
// always, 2 by the estimate), and the row count up to which the single-block kernel takes
// problems of more than 128 rows (0 = by the estimates). Process-wide.
extern "C" int s1_gemm_plan_override(int bn, int splits, int runs, int small_rows) {
    g_override.bn = bn > 0 ? bn : 0;
    g_override.splits = splits > 0 ? splits : 0;
    g_override.runs = runs == 0 || runs == 1 ? runs : 2;
    g_override.small_rows = small_rows > 0 ? small_rows : 0;
    return 0;
}

// Diagnostics: how many clusters of c blocks of the single-block kernel of width bn the current
// device holds at once (0 when that shape of launch is not possible).
extern "C" int s1_gemm_tc5_cluster_room(int bn, int c) {
    cudaError_t err;
    DeviceInfo* info = device_info(&err);
    if (!info) return 0;
    return bn == 256 ? cluster_room<256>(info, 0, c) : bn == 128 ? cluster_room<128>(info, 1, c) : bn == 64 ? cluster_room<64>(info, 2, c) : 0;
}

// Returns the device error word of the current device (0 = no bounded wait ever gave up)
// after waiting for all queued work, and clears it.
extern "C" int s1_gemm_tc5_status(int* code) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return e;
    int v = 0;
    e = cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int));
    if (e != cudaSuccess) return e;
    if (v != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
    }
    *code = v;
    return e;
}

// Device address of this device's error word, for the executor's status copy.
int s1::gemm_error_address(int** p) {
    void* a = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&a, s1::g_gemm_error);
    *p = static_cast<int*>(a);
    return e;
}

namespace s1 {
namespace {
// One block, one thread: waits on an mbarrier that nothing ever completes. The bounded wait
// runs out after limit_ns, the thread records code 99 in the GEMM's error word the way the
// kernels above do, and the kernel returns. No copy, tensor memory or MMA is in flight.
__global__ void wait_runs_out_kernel(uint64_t limit_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    tc5::mbar_init(&bar, 1);
    abort_flag = 0;
    tc5::mbar_init_fence();
    if (!tc5::mbar_wait(&bar, 0, &abort_flag, limit_ns)) atomicCAS(&g_gemm_error, 0, 99);
}
}  // namespace
}  // namespace s1

// Self-test of the give-up path of the bounded waits: queues a one-thread kernel whose wait is
// made to run out after limit_us microseconds (clamped to [1, 100000]) and which then records
// code 99 in the GEMM's error word and returns. The next status read (s1_device_status,
// s1_gemm_tc5_status, or any executor call that reads results back) reports it; the context
// stays usable.
extern "C" int s1_selftest_wait_runs_out(int limit_us, void* stream) {
    if (limit_us < 1) limit_us = 1;
    if (limit_us > 100000) limit_us = 100000;
    wait_runs_out_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>((uint64_t)limit_us * 1000ull);
    return cudaGetLastError();
}
