/* C interface of libqwen3_5_cuda.so, the sm_100a build.
 *
 * This is the boundary the reference project's native workers bind at run time: its Rust
 * loader (src/models/qwen3_5/native/src/cuda.rs:24-47,50-133) dlopens a library of this
 * name, resolves every symbol below and refuses to start unless cs1_abi_version() returns
 * 6 (cuda.rs:12,161-166). Names, argument order, types and error behaviour follow the
 * reference header src/backends/cuda/qwen3_5/ops.h:24-138 declaration for declaration; each
 * group cites the lines it replaces.
 *
 * Conventions (ops.h:1-9): tensors are row-major bfloat16 device memory unless typed
 * otherwise; every operation only queues work on `stream` (a cudaStream_t, always the last
 * argument) and returns 0, a cudaError_t, or a library code >= 1000; invalid shapes return
 * cudaErrorInvalidValue (1) before any launch; zero rows succeed without touching pointers.
 */
#ifndef CS1_OPS_H
#define CS1_OPS_H

#include <stddef.h>
#include <stdint.h>

#define CS1_ABI_VERSION 6

/* Library-defined error codes (>= 1000, as src/backends/cuda/contract.md:145-148 reserves). */
#define CS1_ERR_GEMM_BASE 1000      /* 1000 + cublasStatus_t, as the reference (gemm.cu:34) */
#define CS1_ERR_UNSUPPORTED 2000    /* this engine does not take the problem (see s1_gemm_swiglu, s1_gemm_tcgen05) */
#define CS1_ERR_DEVICE_CHECK 2001   /* a device-side bounded wait gave up */
#define CS1_ERR_TENSOR_MAP 2002     /* a TMA tensor map could not be encoded */
#define CS1_ERR_STATIC_SCRATCH 2003 /* the window does not fit the fixed scratch of cs1_gdn_prefill_static */

#ifdef __cplusplus
extern "C" {
#endif

/* ---- runtime: ops.h:24-44 (runtime.cu:9-74) ---- */
uint32_t cs1_abi_version(void);
const char* cs1_error_string(int code);
int cs1_set_device(int device);
int cs1_malloc(void** ptr, size_t bytes);
int cs1_free(void* ptr);
int cs1_stream_create(void** stream);
int cs1_stream_sync(void* stream);
int cs1_stream_destroy(void* stream);
int cs1_graph_begin(void* stream);
int cs1_graph_end(void* stream, void** exec);
int cs1_graph_launch(void* exec, void* stream);
int cs1_graph_destroy(void* exec);
/* Copy and wait for the copy (ops.h:36-38). */
int cs1_upload(void* dst, const void* src, size_t bytes, void* stream);
int cs1_download(void* dst, const void* src, size_t bytes, void* stream);
/* Queue-only device-to-device copies (ops.h:39-44). */
int cs1_copy_dd(void* dst, const void* src, size_t bytes, void* stream);
int cs1_copy2d(void* dst, size_t dpitch, const void* src, size_t spitch, size_t width, size_t height, void* stream);

/* ---- operations ---- */

/* ops.h:48-49: out[t] = table[ids[t]], rows of D (D % 8 == 0). */
int cs1_embed(const int32_t* ids, const void* table, void* out, int T, int D, void* stream);

/* ops.h:51-52: out = bf16(x * rsqrt(mean(x^2) + eps) * (1 + w)), float32 inside. */
int cs1_rms_norm(const void* x, const void* w, void* out, int rows, int D, float eps, void* stream);

/* ops.h:54-56: residual = bf16(residual + delta) in place, then cs1_rms_norm(residual). */
int cs1_add_rms_norm(void* residual, const void* delta, const void* w, void* out, int rows, int D, float eps,
                     void* stream);

/* ops.h:58-61: gated RMSNorm of x [T, H, 128] with z [T, H*128] in rows of ldz:
 * out = bf16(bf16(w * bf16(x * inv)) * silu(z)). */
int cs1_gated_rms_norm(const void* x, const void* z, int ldz, const void* w, void* out, int T, int H, int D,
                       float eps, void* stream);

/* ops.h:63-66: depthwise causal conv1d (kernel 4) + SiLU over qkv [T, ld], split into
 * q [T, key_dim], k [T, key_dim], v [T, value_dim]; w is [2*key_dim + value_dim, 4]. */
int cs1_gdn_conv(const void* qkv, int ld, const void* w, void* q, void* k, void* v, int T, int key_dim,
                 int value_dim, void* stream);

/* ops.h:68-71: beta = bf16(sigmoid(b)), g = -exp(A_log) * softplus(a + dt_bias) (float32), [T, H]. */
int cs1_gdn_gates(const void* b, const void* a, int ld, const void* A_log, const void* dt_bias, void* beta,
                  float* g, int T, int H, void* stream);

/* ops.h:73-78: chunked gated delta rule; q, k [T, HK, 128], v, o [T, H, 128], g float [T, H],
 * beta [T, H]. The workspace holds cs1_gdn_workspace_floats(T', H) floats for any T' >= T. */
size_t cs1_gdn_workspace_floats(int T, int H);
int cs1_gdn_prefill(const void* q, const void* k, const void* v, const float* g, const void* beta, void* o,
                    float* workspace, int T, int H, int HK, float scale, void* stream);

/* ops.h:80-87: the same scan with an explicit float32 state [H, 128, 128] before (s_in, null =
 * zero) and after (s_out, null = skip) the window; a continuation that starts on a multiple
 * of 64 tokens repeats the one-shot arithmetic bit for bit. T == 0 copies s_in (or zeros) to s_out. */
int cs1_gdn_prefill_x(const void* q, const void* k, const void* v, const float* g, const void* beta, void* o,
                      float* workspace, int T, int H, int HK, float scale, const void* s_in, void* s_out,
                      void* stream);

/* No counterpart in the reference. cs1_gdn_prefill for callers that cannot provide the
 * workspace because they cannot allocate device memory (a worker confined to buffers it was
 * handed, a plugin inside a process whose memory pool it does not own, a path where
 * cudaMalloc is forbidden because it synchronises the device): the workspace is a fixed
 * CS1_GDN_STATIC_SCRATCH_BYTES array inside the library, one per GPU, held until the library
 * is unloaded. The call allocates nothing. It fails with CS1_ERR_STATIC_SCRATCH when
 * cs1_gdn_workspace_floats(T, H) * 4 exceeds that size. All calls on a GPU share the array:
 * calls that can overlap on the GPU race; the array keeps the last call's contents, and
 * none of it has to be cleared. The first call on each GPU resolves the array's device
 * address and should be made before any stream capture. */
#define CS1_GDN_STATIC_SCRATCH_BYTES (64u << 20)
int cs1_gdn_prefill_static(const void* q, const void* k, const void* v, const float* g, const void* beta, void* o,
                           int T, int H, int HK, float scale, void* stream);

/* ops.h:89-94: per-head RMSNorm(1+w) of q and k and rotary embedding on the first 2*half
 * dims; qg [T, Hq, 2*Dh] (query | gate per head) and kr [T, Hk, Dh] in rows of ld. The
 * reference accepts Dh == 256 only; this build accepts Dh in {128, 256}. */
int cs1_attn_prep(const void* qg, const void* kr, int ld, const void* qw, const void* kw, const void* cos,
                  const void* sin, void* q, void* gate, void* k, int T, int Hq, int Hk, int Dh, int half,
                  float eps, void* stream);

/* ops.h:96-99: causal grouped-query attention, v in rows of ldv; Dh in {128, 256}. */
int cs1_attention(const void* q, const void* k, const void* v, int ldv, void* out, int T, int Hq, int Hk, int Dh,
                  float scale, void* stream);
/* ops.h:101-105: the same with out = bf16(bf16(o) * bf16(sigmoid(gate))) fused. */
int cs1_attention_gated(const void* q, const void* k, const void* v, int ldv, const void* gate, void* out, int T,
                        int Hq, int Hk, int Dh, float scale, void* stream);
/* ops.h:107-112: q, gate, out cover rows [q_base, T) only; q_base % 64 == 0. */
int cs1_attention_gated_prefix(const void* q, const void* k, const void* v, int ldv, const void* gate, void* out,
                               int T, int Hq, int Hk, int Dh, float scale, int q_base, void* stream);

/* ops.h:114-115 */
int cs1_sigmoid_gate(void* x, const void* gate, size_t n, void* stream);
/* ops.h:117-118: out [T, I] = bf16(bf16(silu(gate)) * up) from gate_up [T, 2*I] in rows of ld. */
int cs1_silu_mul(const void* gate_up, int ld, void* out, int T, int I, void* stream);

/* ops.h:120-125: y [M, N] (rows of ldy) = x [M, K] * w [N, K]^T, float32 accumulation. */
void* cs1_gemm_create(size_t workspace_bytes);
void cs1_gemm_destroy(void* gemm);
int cs1_gemm(void* gemm, const void* x, const void* w, void* y, int M, int N, int K, int ldy, void* stream);

/* ---- vision tower (single image, hidden 1024, 16 heads of 64): ops.h:125-138, vision.cu, gemm.cu:137-163.
 * linear: y = bf16(x w^T + bias), the bias joining the float32 sum (a library call in the reference, the tcgen05 kernel's bias epilogue here);
 * gemm_f32: float32 throughout; norm: LayerNorm eps 1e-6; position: x += bf16(sum of four table rows times
 * their weights), separate float32 multiplies and adds; rope: q, k out of the fused [n, 3072] projection, cos / sin
 * [n, 32] float32, both products rounded before the add; attention: every query over all n keys, v a slice of
 * the projection with rows 3072 apart (tcgen05 kernel); bias / gelu / add / lora_add: in place, one bf16
 * rounding; to_float: widening copy. ---- */
int cs1_vision_linear(void* gemm, const void* x, const void* w, const void* bias, void* y, int M, int N, int K,
                      void* stream);
int cs1_gemm_f32(void* gemm, const float* x, const float* w, float* y, int M, int N, int K, void* stream);
int cs1_vision_norm(const void* x, const void* w, const void* b, void* y, int rows, int d, void* stream);
int cs1_vision_position(void* x, const void* table, const int* indices, const float* weights, int n, void* stream);
int cs1_vision_rope(const void* qkv, const float* co, const float* si, void* q, void* k, int n, void* stream);
int cs1_vision_attention(const void* q, const void* k, const void* v, void* out, int n, void* stream);
int cs1_vision_bias(void* x, const void* bias, size_t n, int d, void* stream);
int cs1_vision_gelu(void* x, size_t n, int exact, void* stream);
int cs1_vision_add(void* x, const void* delta, size_t n, void* stream);
int cs1_vision_to_float(const void* x, float* out, size_t n, void* stream);
int cs1_vision_lora_add(void* x, const float* delta, size_t n, float scale, void* stream);

#ifdef __cplusplus
}
#endif
#endif
