// Comparison arm of the GEMM microbenchmark only: the vendor library's bf16 GEMM (cuBLASLt, first
// heuristic algorithm, 32 MiB workspace) behind one call, built into its own shared object
// (libs1_compare.so). Nothing in libqwen3_5_cuda.so links or loads it; the product's GEMM is the
// tcgen05 kernel it is measured against.
#include <cublasLt.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <unordered_map>

namespace {

struct Problem {
    cublasLtMatmulDesc_t op = nullptr;
    cublasLtMatrixLayout_t wl = nullptr, xl = nullptr, yl = nullptr;
    cublasLtMatmulHeuristicResult_t pick{};
    bool usable = false;
    ~Problem() {
        if (wl) cublasLtMatrixLayoutDestroy(wl);
        if (xl) cublasLtMatrixLayoutDestroy(xl);
        if (yl) cublasLtMatrixLayoutDestroy(yl);
        if (op) cublasLtMatmulDescDestroy(op);
    }
};

struct Library {
    cublasLtHandle_t lt = nullptr;
    void* room = nullptr;
    size_t room_bytes = 32u << 20;
    std::unordered_map<uint64_t, std::unique_ptr<Problem>> known;

    bool ready() {
        if (lt) return true;
        if (cublasLtCreate(&lt) != CUBLAS_STATUS_SUCCESS) return false;
        return cudaMalloc(&room, room_bytes) == cudaSuccess;
    }

    // Row-major y [M, N] = x [M, K] w[N, K]^T, seen by the column-major library as y^T = w^T-view * x-view.
    Problem* lookup(int M, int N, int K) {
        const uint64_t key = ((uint64_t)M << 42) ^ ((uint64_t)N << 21) ^ (uint64_t)K;
        auto& slot = known[key];
        if (slot) return slot.get();
        slot = std::make_unique<Problem>();
        Problem& p = *slot;
        const cublasOperation_t yes = CUBLAS_OP_T, no = CUBLAS_OP_N;
        bool ok = cublasLtMatmulDescCreate(&p.op, CUBLAS_COMPUTE_32F, CUDA_R_32F) == CUBLAS_STATUS_SUCCESS;
        ok = ok && cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_TRANSA, &yes, sizeof(yes)) == CUBLAS_STATUS_SUCCESS;
        ok = ok && cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_TRANSB, &no, sizeof(no)) == CUBLAS_STATUS_SUCCESS;
        ok = ok && cublasLtMatrixLayoutCreate(&p.wl, CUDA_R_16BF, K, N, K) == CUBLAS_STATUS_SUCCESS;
        ok = ok && cublasLtMatrixLayoutCreate(&p.xl, CUDA_R_16BF, K, M, K) == CUBLAS_STATUS_SUCCESS;
        ok = ok && cublasLtMatrixLayoutCreate(&p.yl, CUDA_R_16BF, N, M, N) == CUBLAS_STATUS_SUCCESS;
        cublasLtMatmulPreference_t want = nullptr;
        ok = ok && cublasLtMatmulPreferenceCreate(&want) == CUBLAS_STATUS_SUCCESS;
        if (ok) {
            cublasLtMatmulPreferenceSetAttribute(want, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &room_bytes, sizeof(room_bytes));
            int n = 0;
            ok = cublasLtMatmulAlgoGetHeuristic(lt, p.op, p.wl, p.xl, p.yl, p.yl, want, 1, &p.pick, &n) == CUBLAS_STATUS_SUCCESS && n > 0;
        }
        if (want) cublasLtMatmulPreferenceDestroy(want);
        p.usable = ok;
        return &p;
    }
};

Library g_library;

}  // namespace

// 0 on success, 1 when the library refuses the problem or cannot be set up.
extern "C" int s1_compare_library_gemm(const void* x, const void* w, void* y, int M, int N, int K, void* stream) {
    if (!g_library.ready()) return 1;
    Problem* p = g_library.lookup(M, N, K);
    if (!p->usable) return 1;
    const float one = 1.f, zero = 0.f;
    return cublasLtMatmul(g_library.lt, p->op, &one, w, p->wl, x, p->xl, &zero, y, p->yl, y, p->yl, &p->pick.algo,
                          g_library.room, g_library.room_bytes, static_cast<cudaStream_t>(stream)) == CUBLAS_STATUS_SUCCESS
               ? 0
               : 1;
}
