// Warp-level tensor-core building blocks (mma.sync with register accumulators), ldmatrix
// and cp.async. These serve the latency-bound kernels whose accumulators must be rescaled
// every step (the delta-rule state scan, online-softmax attention); the throughput-bound
// GEMM uses tcgen05 with TMEM accumulators instead (tc5.cuh).
//
// Fragment layouts (PTX ISA, mma.m16n8k16), with g = lane / 4 and t = lane % 4:
//   A (16x16, row):  a0 (g, 2t..2t+1)  a1 (g+8, 2t..)  a2 (g, 2t+8..)  a3 (g+8, 2t+8..)
//   B (16x8, col):   b0 (k = 2t..2t+1, n = g)          b1 (k = 2t+8.., n = g)
//   C (16x8):        c0,c1 (g, 2t..2t+1)               c2,c3 (g+8, 2t..2t+1)
#pragma once

#include "common.cuh"

namespace s1 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte asynchronous global->shared copy; writes zeros when !valid (src must still be a
// mapped address).
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid = true) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src),
                 "r"(valid ? 16 : 0));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(p)));
}

// A fragment (16x16 at row0, col0) of a row-major bf16 matrix M[row][col], ld in elements.
__device__ __forceinline__ void load_a_rm(uint32_t (&a)[4], const bf16* m, int ld, int row0, int col0, int lane) {
    ldsm_x4(a, m + (size_t)(row0 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + col0 + (lane >> 4) * 8);
}
// A fragment A[m][k] (m0.., k0..) when memory holds the transpose M[k][m] (m contiguous).
__device__ __forceinline__ void load_a_tr(uint32_t (&a)[4], const bf16* m, int ld, int m0, int k0, int lane) {
    ldsm_x4_t(a, m + (size_t)(k0 + (lane & 7) + (lane >> 4) * 8) * ld + m0 + ((lane >> 3) & 1) * 8);
}
// B fragments for two adjacent 8-column tiles (n0, n0+8) at k0 when memory holds
// M[n][k] (k contiguous): b[0],b[1] -> tile n0; b[2],b[3] -> tile n0+8.
__device__ __forceinline__ void load_b_nk(uint32_t (&b)[4], const bf16* m, int ld, int n0, int k0, int lane) {
    ldsm_x4(b, m + (size_t)(n0 + (lane & 7) + (lane >> 4) * 8) * ld + k0 + ((lane >> 3) & 1) * 8);
}
// The same two tiles when memory holds M[k][n] (n contiguous).
__device__ __forceinline__ void load_b_kn(uint32_t (&b)[4], const bf16* m, int ld, int k0, int n0, int lane) {
    ldsm_x4_t(b, m + (size_t)(k0 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + n0 + (lane >> 4) * 8);
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// TF32 m16n8k8: A a0 (g, t) a1 (g+8, t) a2 (g, t+4) a3 (g+8, t+4); B b0 (k=t, n=g) b1 (k=t+4, n=g).
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;\n" : "=r"(r) : "f"(x));
    return r;
}

}  // namespace s1
