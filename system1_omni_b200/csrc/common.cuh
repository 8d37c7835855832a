// Device helpers shared by the sm_100a kernels: bf16 conversion, 128-bit packs, warp and
// block reductions, and the launch-argument checks every entry point performs.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace s1 {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float f32(bf16 x) { return __bfloat162float(x); }
__device__ __forceinline__ bf16 to_bf16(float x) { return __float2bfloat16(x); }
// A float rounded through bf16 (round to nearest even), where the model stores a bf16 result.
__device__ __forceinline__ float rbf(float x) { return __bfloat162float(__float2bfloat16(x)); }

__device__ __forceinline__ float silu(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float sigmoid(float x) { return 1.f / (1.f + expf(-x)); }
// SiLU for the bandwidth-bound kernels whose result is rounded to bf16 right away: hardware
// exp2 and reciprocal approximations (relative error about 1e-6, against a bf16 step of 4e-3)
// instead of the IEEE division and the accurate expf, which cost about four times the
// instructions and kept those kernels instruction-bound. The rounded bf16 result differs from
// the exact-division one in rare ties only, by one step.
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.f + __expf(-x)); }

// Eight bf16 values moved as one 16-byte access.
struct alignas(16) Pack8 {
    uint4 raw;
};

__device__ __forceinline__ void unpack8(const uint4& p, float (&out)[8]) {
    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ uint4 pack8(const float (&in)[8]) {
    uint4 p;
    p.x = pack2(in[0], in[1]);
    p.y = pack2(in[2], in[3]);
    p.z = pack2(in[4], in[5]);
    p.w = pack2(in[6], in[7]);
    return p;
}

__device__ __forceinline__ uint4 ld16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void st16(void* p, const uint4& v) { *reinterpret_cast<uint4*>(p) = v; }
// 32 bytes (a whole sector) in one store; p must be 32-byte aligned.
__device__ __forceinline__ void st32(void* p, const uint4& a, const uint4& b) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w),
                 "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
                 : "memory");
}
// Streaming variants for data touched once: keep it out of L1 and mark it evict-first.
__device__ __forceinline__ uint4 ld16_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <int WIDTH = 32>
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = WIDTH / 2; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// Sum over a block of up to 1024 threads; scratch holds 32 floats; every thread gets the sum.
__device__ __forceinline__ float block_sum(float x, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    x = warp_sum(x);
    if (lane == 0) scratch[warp] = x;
    __syncthreads();
    float t = lane < warps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    __syncthreads();
    return t;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

// ---- programmatic dependent launch ----
// A kernel launched with launch_dep while the switch is on is queued as a programmatic dependent
// of the kernel before it on the stream: its blocks may become resident as soon as every block of
// that kernel has called grid_dep_trigger() (the first thing each hot-path kernel does) or has
// exited, and it calls grid_dep_sync() before it touches anything that kernel wrote or still
// reads. What a kernel does before grid_dep_sync() - barriers, tensor memory, descriptor
// prefetch, and in the GEMMs the first stages of weight tiles, which no kernel of a forward pass
// writes - overlaps the kernels before it; the order of all other memory effects is that of
// ordinary stream order, since grid_dep_sync() returns only when the kernel before is complete
// and its writes are visible, and that kernel in turn waited for the one before it.
// The switch is per host thread and has three settings: nearly every hot-path kernel (the
// executor's choice for short prompts issued eagerly, where launch gaps, prologues and the first
// trip to HBM are a large part of every kernel), the GEMMs and the norms after them (its choice
// otherwise: measured at 1024 tokens +3 %, where making every kernel a dependent costs 1 %: blocks
// that only wait take room from the running kernel, while a GEMM's blocks that arrive early fetch
// their first ring of weight tiles under the short kernel ahead), or none.
// Both instructions are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void grid_dep_sync() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// The switch: 0 = plain stream order, 1 = every hot-path kernel but the delta-rule pair, 2 = the GEMMs and norms.
inline int& dep_launch_switch() {
    static thread_local int mode = 0;
    return mode;
}

inline int dep_launch_mode() { return dep_launch_switch(); }
// Kernel families, for the choice of which launches become dependents.
enum DepFamily { DEP_GEMM = 1, DEP_GDN = 2, DEP_ATTENTION = 4, DEP_NORM = 8, DEP_OTHER = 16 };
// What the two modes cover, from measurements on the 4B-shaped decoder: the delta-rule kernels are
// never launched as dependents (their blocks take most of an SM's shared memory while they wait:
// -4 % at 1024 tokens, and short passes are faster without them too); mode 1 takes everything
// else, mode 2 the GEMMs and the norms that follow them.
inline int dep_launch_mask(int mode) {
    return mode == 1 ? (int)(DEP_GEMM | DEP_ATTENTION | DEP_NORM | DEP_OTHER) : mode == 2 ? (int)(DEP_GEMM | DEP_NORM) : 0;
}
inline bool dep_launch_family(int family) { return (dep_launch_mask(dep_launch_mode()) & family) != 0; }
inline bool dep_launch_enabled() { return dep_launch_family(DEP_OTHER); }
inline bool dep_launch_gemm() { return dep_launch_family(DEP_GEMM); }

template <typename... KArgs, typename... Args>
cudaError_t launch_maybe_dep(bool dependent, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                             Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
template <typename... KArgs, typename... Args>
cudaError_t launch_dep(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    return launch_maybe_dep(dep_launch_enabled(), kernel, grid, block, smem, st, args...);
}
template <typename... KArgs, typename... Args>
cudaError_t launch_dep_family(int family, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args... args) {
    return launch_maybe_dep(dep_launch_family(family), kernel, grid, block, smem, st, args...);
}
template <typename... KArgs, typename... Args>
cudaError_t launch_dep_gemm(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    return launch_maybe_dep(dep_launch_gemm(), kernel, grid, block, smem, st, args...);
}

}  // namespace s1
