// y [M, N] (rows of ldy) = x [M, K] * w [N, K]^T in bf16 with float32 accumulation: every
// projection of the decoder (reference entry: src/backends/cuda/qwen3_5/gemm.cu:103-135).
//
// Two engines sit behind cs1_gemm and are chosen per handle when it is created:
//   * the hand-written tcgen05 kernel of gemm_tc5.cu (TMA-fed, TMEM accumulators), used for
//     every shape it supports (K % 64 == 0, 16-byte aligned rows);
//   * cuBLASLt with its first heuristic choice, excluding split-K schemes that reduce into
//     the output in place, exactly as the reference configures it. It serves the shapes the
//     tcgen05 kernel declines and is the comparison arm of the GEMM benchmark.
// S1_GEMM=cublaslt in the environment forces the library engine for a whole process.
#include <cublasLt.h>
#include <cuda_runtime.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <mutex>
#include <tuple>

#include "cs1_ops.h"
#include "gemm_tc5.h"
#include "s1_executor.h"

namespace {

struct Plan {
    cublasLtMatmulDesc_t op = nullptr;
    cublasLtMatrixLayout_t a = nullptr, b = nullptr, c = nullptr;
    cublasLtMatmulAlgo_t algo{};
};

using Key = std::tuple<int, int, int, int, int>;  // M, N, K, ldy, kind (0 bf16, 1 bf16 + bias epilogue, 2 float32)
constexpr int COUNTER_SLOTS = 16384;
constexpr size_t PARTIAL_BYTES = (size_t)48 << 20;

struct Gemm {
    cublasLtHandle_t handle = nullptr;
    void* workspace = nullptr;
    size_t workspace_bytes = 0;
    bool use_tc5 = true;
    int* counters = nullptr;
    void* partials = nullptr;  // float32 partial tiles of the tcgen05 kernel's shared-tile paths
    size_t partial_bytes = 0;
    std::map<Key, Plan> plans;
    std::mutex lock;
};

int status(cublasStatus_t s) { return s == CUBLAS_STATUS_SUCCESS ? 0 : CS1_ERR_GEMM_BASE + (int)s; }

void destroy(Plan& p) {
    if (p.a) cublasLtMatrixLayoutDestroy(p.a);
    if (p.b) cublasLtMatrixLayoutDestroy(p.b);
    if (p.c) cublasLtMatrixLayoutDestroy(p.c);
    if (p.op) cublasLtMatmulDescDestroy(p.op);
    p = Plan{};
}

// Row-major y = x w^T is the column-major product y^T [N, M] = (w as [K, N])^T (x as [K, M]).
int make_plan(Gemm& g, int M, int N, int K, int ldy, Plan& p, int kind = 0) {
    const cudaDataType_t dt = kind == 2 ? CUDA_R_32F : CUDA_R_16BF;
    cublasStatus_t s = cublasLtMatmulDescCreate(&p.op, CUBLAS_COMPUTE_32F, CUDA_R_32F);
    if (s != CUBLAS_STATUS_SUCCESS) return status(s);
    const cublasOperation_t ta = CUBLAS_OP_T, tb = CUBLAS_OP_N;
    cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof(ta));
    cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof(tb));
    if (kind == 1) {  // bias added to the float32 sum before the one bf16 rounding (gemm.cu:137-151 of the reference)
        const cublasLtEpilogue_t ep = CUBLASLT_EPILOGUE_BIAS;
        const cudaDataType_t bias_type = CUDA_R_16BF;
        cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_EPILOGUE, &ep, sizeof(ep));
        cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_BIAS_DATA_TYPE, &bias_type, sizeof(bias_type));
    }
    if ((s = cublasLtMatrixLayoutCreate(&p.a, dt, K, N, K)) != CUBLAS_STATUS_SUCCESS) return status(s);
    if ((s = cublasLtMatrixLayoutCreate(&p.b, dt, K, M, K)) != CUBLAS_STATUS_SUCCESS) return status(s);
    if ((s = cublasLtMatrixLayoutCreate(&p.c, dt, N, M, ldy)) != CUBLAS_STATUS_SUCCESS) return status(s);
    cublasLtMatmulPreference_t pref;
    if ((s = cublasLtMatmulPreferenceCreate(&pref)) != CUBLAS_STATUS_SUCCESS) return status(s);
    cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &g.workspace_bytes,
                                         sizeof(g.workspace_bytes));
    const uint32_t schemes = CUBLASLT_REDUCTION_SCHEME_MASK & ~CUBLASLT_REDUCTION_SCHEME_INPLACE;
    cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_REDUCTION_SCHEME_MASK, &schemes, sizeof(schemes));
    cublasLtMatmulHeuristicResult_t r{};
    int found = 0;
    s = cublasLtMatmulAlgoGetHeuristic(g.handle, p.op, p.a, p.b, p.c, p.c, pref, 1, &r, &found);
    cublasLtMatmulPreferenceDestroy(pref);
    if (s != CUBLAS_STATUS_SUCCESS) return status(s);
    if (found == 0 || r.state != CUBLAS_STATUS_SUCCESS) return status(CUBLAS_STATUS_NOT_SUPPORTED);
    p.algo = r.algo;
    return 0;
}

int lt_gemm(Gemm& g, const void* x, const void* w, void* y, int M, int N, int K, int ldy, cudaStream_t st, int kind = 0,
            const void* bias = nullptr) {
    Plan* p = nullptr;
    {
        std::lock_guard<std::mutex> hold(g.lock);
        const Key key{M, N, K, ldy, kind};
        auto it = g.plans.find(key);
        if (it == g.plans.end()) {
            Plan fresh;
            const int rc = make_plan(g, M, N, K, ldy, fresh, kind);
            if (rc != 0) {
                destroy(fresh);
                return rc;
            }
            it = g.plans.emplace(key, fresh).first;
        }
        p = &it->second;
    }
    const float alpha = 1.f, beta = 0.f;
    if (kind == 1) {
        // the pointer lives in the shared descriptor: one stream per handle, as for everything else here
        std::lock_guard<std::mutex> hold(g.lock);
        const cublasStatus_t s = cublasLtMatmulDescSetAttribute(p->op, CUBLASLT_MATMUL_DESC_BIAS_POINTER, &bias, sizeof(bias));
        if (s != CUBLAS_STATUS_SUCCESS) return status(s);
        return status(cublasLtMatmul(g.handle, p->op, &alpha, w, p->a, x, p->b, &beta, y, p->c, y, p->c, &p->algo,
                                     g.workspace, g.workspace_bytes, st));
    }
    return status(cublasLtMatmul(g.handle, p->op, &alpha, w, p->a, x, p->b, &beta, y, p->c, y, p->c, &p->algo,
                                 g.workspace, g.workspace_bytes, st));
}

}  // namespace

extern "C" void* cs1_gemm_create(size_t workspace_bytes) {
    Gemm* g = new Gemm();
    if (cublasLtCreate(&g->handle) != CUBLAS_STATUS_SUCCESS ||
        (workspace_bytes > 0 && cudaMalloc(&g->workspace, workspace_bytes) != cudaSuccess)) {
        if (g->handle) cublasLtDestroy(g->handle);
        delete g;
        return nullptr;
    }
    g->workspace_bytes = workspace_bytes;
    // counters of the tcgen05 kernel's K-split path; zero between launches
    if (cudaMalloc(reinterpret_cast<void**>(&g->counters), COUNTER_SLOTS * sizeof(int)) != cudaSuccess ||
        cudaMemset(g->counters, 0, COUNTER_SLOTS * sizeof(int)) != cudaSuccess) {
        if (g->counters) cudaFree(g->counters);
        if (g->workspace) cudaFree(g->workspace);
        cublasLtDestroy(g->handle);
        delete g;
        return nullptr;
    }
    const char* engine = getenv("S1_GEMM");
    g->use_tc5 = !(engine && strcmp(engine, "cublaslt") == 0);
    // Room for two 256 x 256 float32 partial tiles per block pair (37 MiB on 148 SMs). Without
    // it (allocation refused) the kernel keeps to whole tiles.
    if (g->use_tc5 && cudaMalloc(&g->partials, PARTIAL_BYTES) == cudaSuccess)
        g->partial_bytes = PARTIAL_BYTES;
    else
        cudaGetLastError();
    return g;
}

extern "C" void cs1_gemm_destroy(void* gemm) {
    Gemm* g = static_cast<Gemm*>(gemm);
    if (!g) return;
    for (auto& kv : g->plans) destroy(kv.second);
    if (g->workspace) cudaFree(g->workspace);
    if (g->counters) cudaFree(g->counters);
    if (g->partials) cudaFree(g->partials);
    cublasLtDestroy(g->handle);
    delete g;
}

namespace {
S1GemmScratch scratch_of(Gemm* g) {
    return S1GemmScratch{g->partials, g->partial_bytes, g->counters, COUNTER_SLOTS};
}
}  // namespace

extern "C" int cs1_gemm(void* gemm, const void* x, const void* w, void* y, int M, int N, int K, int ldy,
                        void* stream) {
    Gemm* g = static_cast<Gemm*>(gemm);
    if (!g || M < 0 || N <= 0 || K <= 0 || ldy < N) return cudaErrorInvalidValue;
    if (M == 0) return cudaSuccess;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (g->use_tc5 && s1_gemm_tc5_supported(x, w, y, M, N, K, ldy)) {
        const S1GemmScratch scratch = scratch_of(g);
        return s1_gemm_tc5(x, w, y, M, N, K, ldy, &scratch, st);
    }
    return lt_gemm(*g, x, w, y, M, N, K, ldy, st);
}

// cs1_gemm without the K-split path: every row's sum runs over K in one fixed order, whatever M is.
extern "C" int s1_gemm_unsplit(void* gemm, const void* x, const void* w, void* y, int M, int N, int K, int ldy,
                               void* stream) {
    Gemm* g = static_cast<Gemm*>(gemm);
    if (!g || M < 0 || N <= 0 || K <= 0 || ldy < N) return cudaErrorInvalidValue;
    if (M == 0) return cudaSuccess;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (g->use_tc5 && s1_gemm_tc5_supported(x, w, y, M, N, K, ldy)) return s1_gemm_tc5(x, w, y, M, N, K, ldy, nullptr, st);
    return lt_gemm(*g, x, w, y, M, N, K, ldy, st);
}

extern "C" int s1_gemm_engine(void* gemm, const void* x, const void* w, int M, int N, int K) {
    Gemm* g = static_cast<Gemm*>(gemm);
    return g && g->use_tc5 && s1_gemm_tc5_supported(x, w, nullptr, M, N, K, N) ? 1 : 0;
}

// The MLP's first half as one kernel on the tcgen05 engine: act [M, I] (rows of ld) =
// silu(x w[0:I]^T) * (x w[I:2I]^T), bit-identical to cs1_gemm into a [M, 2 I] buffer followed by
// cs1_silu_mul. Returns CS1_ERR_UNSUPPORTED when the engine cannot take the problem (other
// engine selected, at most 128 rows, K not a multiple of 8); the caller then runs the two operators.
extern "C" int s1_gemm_swiglu(void* gemm, const void* x, const void* w, void* act, int M, int I, int K, int ld,
                              void* stream) {
    Gemm* g = static_cast<Gemm*>(gemm);
    if (!g || M < 0 || I <= 0 || K <= 0 || ld < I) return cudaErrorInvalidValue;
    if (M == 0) return cudaSuccess;
    if (!g->use_tc5 || !s1_gemm_tc5_swiglu_supported(x, w, M, I, K)) return CS1_ERR_UNSUPPORTED;
    return s1_gemm_tc5_swiglu(x, w, act, M, I, K, ld, static_cast<cudaStream_t>(stream));
}

// Engine-pinned entry points for the GEMM benchmark and the parity tests.
extern "C" int s1_gemm_cublaslt(void* gemm, const void* x, const void* w, void* y, int M, int N, int K, int ldy,
                                void* stream) {
    Gemm* g = static_cast<Gemm*>(gemm);
    if (!g || M < 0 || N <= 0 || K <= 0 || ldy < N) return cudaErrorInvalidValue;
    if (M == 0) return cudaSuccess;
    return lt_gemm(*g, x, w, y, M, N, K, ldy, static_cast<cudaStream_t>(stream));
}

extern "C" int s1_gemm_tcgen05(void* gemm, const void* x, const void* w, void* y, int M, int N, int K, int ldy,
                               void* stream) {
    if (M < 0 || N <= 0 || K <= 0 || ldy < N) return cudaErrorInvalidValue;
    if (M == 0) return cudaSuccess;
    if (!s1_gemm_tc5_supported(x, w, y, M, N, K, ldy)) return CS1_ERR_UNSUPPORTED;
    Gemm* g = static_cast<Gemm*>(gemm);  // null: no scratch, so no K split
    if (!g) return s1_gemm_tc5(x, w, y, M, N, K, ldy, nullptr, static_cast<cudaStream_t>(stream));
    const S1GemmScratch scratch = scratch_of(g);
    return s1_gemm_tc5(x, w, y, M, N, K, ldy, &scratch, static_cast<cudaStream_t>(stream));
}

// ---- the vision tower's two library GEMMs (gemm.cu:137-163 of the reference), on cuBLASLt as there ----
// y [M, N] = bf16(x w^T + bias): the bias joins the float32 sum before the rounding.
extern "C" int cs1_vision_linear(void* gemm, const void* x, const void* w, const void* bias, void* y, int M, int N, int K,
                                 void* stream) {
    Gemm* g = static_cast<Gemm*>(gemm);
    if (!g || !bias || !x || !w || !y || M <= 0 || N <= 0 || K <= 0) return cudaErrorInvalidValue;
    return lt_gemm(*g, x, w, y, M, N, K, N, static_cast<cudaStream_t>(stream), 1, bias);
}

// float32 in, float32 out, float32 arithmetic (unmerged LoRA factors; no TF32).
extern "C" int cs1_gemm_f32(void* gemm, const float* x, const float* w, float* y, int M, int N, int K, void* stream) {
    Gemm* g = static_cast<Gemm*>(gemm);
    if (!g || !x || !w || !y || M <= 0 || N <= 0 || K <= 0) return cudaErrorInvalidValue;
    return lt_gemm(*g, x, w, y, M, N, K, N, static_cast<cudaStream_t>(stream), 2);
}
