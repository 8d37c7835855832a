/* Additions to the cs1_* C ABI exported by the same libqwen3_5_cuda.so: runtime helpers a
 * host needs for timing and pinned staging, engine-pinned GEMM entry points, and the host
 * executor (the decoder layer loop the reference keeps in Rust,
 * src/models/qwen3_5/native/src/model.rs). Plain pointers and sizes only.
 */
#ifndef S1_EXECUTOR_H
#define S1_EXECUTOR_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- runtime helpers (no counterpart in the reference ABI; its host links none of these
 * because it never times on the device or stages through pinned memory) ---- */
int s1_device_count(int* count);
int s1_event_create(void** event);
int s1_event_destroy(void* event);
int s1_event_record(void* event, void* stream);
int s1_event_sync(void* event);
int s1_event_elapsed_ms(void* start, void* stop, float* ms);
int s1_host_alloc(void** ptr, size_t bytes);
int s1_host_free(void* ptr);
int s1_upload_async(void* dst, const void* src, size_t bytes, void* stream);
int s1_download_async(void* dst, const void* src, size_t bytes, void* stream);
int s1_memset_async(void* dst, int value, size_t bytes, void* stream);
int s1_device_sync(void);
/* Programmatic dependent launch for the calling host thread's later launches of this library's
 * kernels: mode 1 = every hot-path kernel but the two delta-rule kernels, 2 = the GEMMs and the
 * norms, 0 = plain stream order. A kernel
 * launched so may become resident while the kernel before it on the stream still runs, sets up
 * (the GEMMs also fetch their first weight tiles) and waits for that kernel to complete before it
 * touches activations. Results are the same bits in every mode. Returns the previous mode. The
 * executor picks per forward pass by the number of tokens (s1_model_set_overlap_tokens). */
int s1_set_dependent_launch(int mode);
int s1_mem_info(size_t* free_bytes, size_t* total_bytes);

/* ---- Attention over a window that continues a shared prefix ----
 * Gated causal attention of positions [prefix_len, prefix_len + rows): q, gate, out [rows, Hq, Dh],
 * k [rows, Hk, Dh] and v (row stride ldv) hold the window only; the prefix's post-prep keys
 * [prefix_len, Hk, Dh] and values (row stride ldv_prefix) are read where they lie, so several
 * windows share one copy. Same tiles and arithmetic as cs1_attention_gated_prefix on the
 * concatenated rows, which is how the reference does it after copying the prefix rows back
 * into its scratch (model.rs:1516-1523). prefix_len: a multiple of 64, 0 = no prefix. */
int s1_attention_gated_shared_prefix(const void* q, const void* k, const void* v, int ldv, const void* gate, void* out,
                                     const void* k_prefix, const void* v_prefix, int ldv_prefix, int prefix_len,
                                     int rows, int Hq, int Hk, int Dh, float scale, void* stream);

/* Per-head L2 norm as an operator of its own (inside cs1_gdn_prefill it is part of the chunk kernel,
 * gdn_prefill.cu:170-203): out = bf16(x * rsqrt(sum x^2 + 1e-6) * scale) over `rows` rows of 128 bf16;
 * for the elementwise benchmark sweep and for checks. x and out 16-byte aligned. */
int s1_l2norm_heads(const void* x, void* out, long long rows, float scale, void* stream);
/* cs1_gdn_conv and cs1_gdn_gates of the same T rows (of pitch ld) in one launch: b and a point at
 * the two gate columns of the first row, as in cs1_gdn_gates. The same bits as the two operators
 * (the reference runs them one after the other, model.rs:640-668). CS1_ERR_UNSUPPORTED where
 * cs1_gdn_conv would take its scalar path (widths not multiples of 8, unaligned): run the two. */
int s1_gdn_conv_gates(const void* qkv, int ld, const void* w, void* q, void* k, void* v, int T, int key_dim,
                      int value_dim, const void* b, const void* a, const void* A_log, const void* dt_bias, void* beta,
                      float* g, int H, void* stream);

/* cs1_attn_prep for the sequences of one pack in one launch (the reference calls it once per
 * sequence, model.rs:1244-1254): every pointer is that of packed row 0 and T counts the packed
 * rows in all; sequence i is rows [row0[i], row0[i] + rows[i]) and its first row takes the first
 * row of the tables (cos and sin point at the position the sequences start from). Rows outside
 * every sequence are left as they are. nseq <= 16. The same bits as one call per sequence. */
int s1_attn_prep_batch(const void* qg, const void* kr, int ld, const void* qw, const void* kw, const void* cos,
                       const void* sin, void* q, void* gate, void* k, int T, const int* row0, const int* rows, int nseq,
                       int Hq, int Hk, int Dh, int half, float eps, void* stream);

/* s1_attention_gated_shared_prefix for the sequences of one pack in one launch: sequence i owns
 * rows [row0[i], row0[i] + rows[i]) of q, gate, out, k and v and sits at positions
 * [prefix_len, prefix_len + rows[i]) behind the shared prefix (prefix_len 0: none - the plain
 * packed pass, where the reference calls cs1_attention_gated once per sequence,
 * model.rs:1255-1268). nseq <= 16, rows[i] > 0. The same bits as one call per sequence. */
int s1_attention_gated_batch(const void* q, const void* k, const void* v, int ldv, const void* gate, void* out,
                             const void* k_prefix, const void* v_prefix, int ldv_prefix, int prefix_len, const int* row0,
                             const int* rows, int nseq, int Hq, int Hk, int Dh, float scale, void* stream);

/* cs1_gdn_prefill_x for the sequences of one pack in one pair of launches (the reference calls it
 * once per sequence, model.rs:690-712). Sequence i is rows [row0[i], row0[i] + len[i]) of the
 * packed q, k, v, g, beta and o; nseq <= 16 (the pack limit of s1_batch_ranges), len[i] > 0. All
 * sequences start from the same state s_in (nullable = zero: the candidates of one captured
 * prefix share theirs) and sequence i leaves its state in s_out + i * H * 128 * 128 floats
 * (nullable). The same bits as nseq calls. workspace_floats: what the workspace holds; it must be
 * at least cs1_gdn_workspace_floats(64 * sum ceil(len[i] / 64), H). */
int s1_gdn_prefill_batch(const void* q, const void* k, const void* v, const float* g, const void* beta, void* o,
                         float* workspace, size_t workspace_floats, const int* row0, const int* len, int nseq, int H,
                         int HK, float scale, const void* s_in, void* s_out, void* stream);

/* s1_gdn_conv_gates for the sequences of one pack in one launch: every pointer is that of packed
 * row 0 (b and a: the two gate columns of row 0); sequence i is rows [row0[i], row0[i] + len[i]) and
 * its convolution sees zeros before its first row. nseq <= 16, len[i] > 0. The same bits as one
 * call per sequence, CS1_ERR_UNSUPPORTED under the same conditions. */
int s1_gdn_conv_gates_batch(const void* qkv, int ld, const void* w, void* q, void* k, void* v, const int* row0,
                            const int* len, int nseq, int key_dim, int value_dim, const void* b, const void* a,
                            const void* A_log, const void* dt_bias, void* beta, float* g, int H, void* stream);

/* The attention kernel's counterpart of s1_gemm_tc5_status: its device error word (0 = no bounded
 * wait ever gave up), read after waiting for all queued work, then cleared. */
int s1_attn_tc5_status(int* code);

/* The same for the delta-rule kernels (a bounded wait for a TMA or bulk copy gave up). */
int s1_gdn_status(int* code);
/* All three words of the current device with one wait for the device (each out pointer nullable);
 * cleared when any is set. The executor's calls that read results back (s1_model_forward_batch,
 * s1_model_forward_continue, s1_model_prefix_capture, s1_model_read_rows) check them themselves
 * and return CS1_ERR_DEVICE_CHECK, the way the reference turns every device failure into an
 * error (src/models/qwen3_5/native/src/cuda.rs:177-187). */
int s1_device_status(int* gemm, int* attention, int* gdn);
/* Self-test of that path, without any fault: queues a one-thread kernel that waits on a barrier
 * nothing completes; its bounded wait gives up after limit_us microseconds, records code 99 in
 * the GEMM's error word and the kernel returns. The context stays usable. */
int s1_selftest_wait_runs_out(int limit_us, void* stream);

/* ---- the two kernels behind cs1_gemm, pinned (benchmark arms and parity tests) ---- */
/* The plain CUDA-core kernel that serves what TMA cannot address (K below 64 or not a multiple
 * of 8, unaligned operands): float32 FMAs over k in order, any sizes. */
int s1_gemm_plain(void* gemm, const void* x, const void* w, void* y, int M, int N, int K, int ldy, void* stream);
/* Planner overrides of the tcgen05 kernels, for the schedule tests and tuning runs: tile width
 * (0 = the planner's choice), K shares per tile (0 = the planner's), contiguous runs in the pair
 * kernel (0 never, 1 always, 2 by the estimate), and the row count up to which the single-block
 * kernel takes problems of more than 128 rows (0 = by the estimates). Process-wide. */
int s1_gemm_plan_override(int bn, int splits, int runs, int small_rows);
/* cs1_gemm with the K-split path switched off for this call. */
int s1_gemm_unsplit(void* gemm, const void* x, const void* w, void* y, int M, int N, int K, int ldy, void* stream);
/* gemm: a cs1_gemm_create handle whose workspace the K-split path may use, or null (no split). */
int s1_gemm_tcgen05(void* gemm, const void* x, const void* w, void* y, int M, int N, int K, int ldy, void* stream);
/* act [M, I] (rows of ld) = silu(x w[0:I]^T) * (x w[I:2I]^T) in one kernel, bit-identical to cs1_gemm
 * into [M, 2 I] followed by cs1_silu_mul (the reference's MLP sequence, model.rs:1301-1316).
 * CS1_ERR_UNSUPPORTED when the pair kernel cannot take the problem (M <= 128, K % 8 != 0): run the
 * two operators then. */
int s1_gemm_swiglu(void* gemm, const void* x, const void* w, void* act, int M, int I, int K, int ld, void* stream);
/* Waits for the device, returns in *code the error word of the tcgen05 GEMM (0 = no bounded
 * wait gave up) and clears it. */
int s1_gemm_tc5_status(int* code);
/* Diagnostics: how many clusters of c blocks of the tcgen05 GEMM's single-block kernel of column
 * width bn (64, 128 or 256) the current device holds at once; 0 = such a launch is not possible.
 * With at most 128 rows a tile's k-blocks are shared by the blocks of one cluster. */
int s1_gemm_tc5_cluster_room(int bn, int c);

/* ---- host executor: the decoder prefill the reference keeps in Rust ---- */

/* Model shape, the fields of the reference's Config (model.rs:28-48) that the text path uses. */
typedef struct S1Config {
    int hidden, intermediate, n_layers;
    int heads, kv_heads, head_dim, rotary_half;   /* full attention; head_dim 128 or 256 */
    int lin_k_heads, lin_v_heads;                 /* Gated DeltaNet, head dims fixed at 128 */
    int vocab, max_positions;
    float eps;
    double rope_theta;
    const unsigned char* full_attention;          /* n_layers flags: 1 = full attention, 0 = Gated DeltaNet */
} S1Config;

/* Model::load (model.rs:622-705) without the file reading: allocates the weight arena for
 * `cfg` on `device` (one allocation, stacked GEMM groups contiguous, 256-byte aligned parts),
 * a stream and a GEMM handle. Tensors arrive through s1_model_set_tensor under their
 * checkpoint names without the model prefix ("layers.3.mlp.down_proj.weight", ...), or all
 * at once from the seeded device-side generator. Returns 0 or an error code. */
int s1_model_create(const S1Config* cfg, int device, void** model);
void s1_model_destroy(void* model);
int s1_model_set_tensor(void* model, const char* name, const void* host_bf16, size_t bytes);
int s1_model_tensor(void* model, const char* name, void** device_ptr, size_t* bytes);
/* The shape a checkpoint must give that tensor (Weights::get, model.rs:306-320): rank and up to
 * 8 extents, each nullable. */
int s1_model_tensor_shape(void* model, const char* name, int* rank, uint64_t* shape8);
/* Random weights of the shape, generated on the device: matrices and zero-centred norm
 * weights N(0, std), the gated norm weight 1 + N(0, std), A_log U(0, ln 16), dt_bias N(0, 0.1). */
int s1_model_init_random(void* model, uint64_t seed, float std);
size_t s1_model_weight_bytes(void* model);
/* The model's shape (full_attention points into the model). */
int s1_model_config(void* model, S1Config* out);
/* Grows the scratch to hold passes of up to `tokens` tokens now (the reference grows on demand in
 * 1024-token steps, model.rs:747-761, which drops recorded graphs): a host that knows its largest
 * pack calls this once, before it queues passes. */
int s1_model_reserve(void* model, int tokens);
void* s1_model_stream(void* model);
/* CUDA-graph replay per ordered length vector (64 entries, first in first out; a failed capture
 * switches replay off): model.rs:797-897. Off by default, or on when CUA_S1_GRAPH=1 is in the
 * environment at creation, as in the reference (model.rs:695). Unlike the reference, which
 * records every new vector right after running it, a vector is recorded when it is seen for the
 * second time (the pass is recorded and the recording launched, with no wait for the stream):
 * ragged request sets rarely repeat a vector, and a first sight then costs one eager pass only. */
int s1_model_enable_graphs(void* model, int on);
/* Exact packing (on by default): a prompt's hidden states come out bit-identical whether it
 * runs alone, inside a pack, or as a continuation of a captured prefix. Every GEMM then runs on
 * whole tiles (no K range shared between blocks), which makes a row's result independent of the
 * call's row count, so the out/down projections need not run per sequence as they do in the
 * reference (model.rs:723-739). Off: the planner may share K between blocks by the row count,
 * which is faster with few rows (2-3x on the narrow projections at 32-128 tokens) but changes the
 * summation order with the row count: measured on a 4-layer 9B-width decoder with random weights,
 * packed and alone logits then differ by up to 0.02, twice the reference's gate of 0.01
 * (tests/open_jev/prefill_batch.rs:57-64) - hence the default. */
int s1_model_set_exact_packing(void* model, int on);
/* The executor's fused kernels, on by default, each with the same bits as the operators it
 * replaces: the MLP's gate/up projection and SiLU-multiply as one kernel (s1_gemm_swiglu), and the
 * convolution and the gates of a GDN layer as one launch (s1_gdn_conv_gates). Off: always the
 * reference's operator sequence. */
int s1_model_set_fused_mlp(void* model, int on);
/* Forward passes of at most `tokens` tokens that are issued eagerly launch every kernel as a
 * programmatic dependent of the one before it (s1_set_dependent_launch mode 1); longer ones, and
 * every pass recorded into a CUDA graph, only the GEMMs and norms (mode 2); tokens < 0: plain stream order
 * always. Default 128. With few tokens and
 * eager issue the gaps between launches are what there is to hide; otherwise short kernels' blocks
 * that only wait take room from the running GEMM, while a GEMM's early blocks fetch their first
 * weight tiles under the short kernel ahead. The result's bits do not depend on it. */
int s1_model_set_overlap_tokens(void* model, int tokens);
int s1_model_graph_stats(void* model, int* replays, int* captures, int* enabled);

/* Model::forward_batch (model.rs:769-823): prefill a pack of independent prompts
 * (ids concatenated, lengths[nseq]) and return the final-norm hidden state of each prompt's
 * last token as float32 [nseq, hidden] in host memory. Validates like the reference: empty
 * batch, empty or oversized prompt and out-of-vocabulary ids are errors (S1_ERR_ARGUMENT).
 * layer_out (nullable, host, bf16 [n_layers, T, hidden]) receives the residual stream after
 * every layer; it forces eager execution and is meant for parity tests. */
int s1_model_forward_batch(void* model, const int32_t* ids, const int* lengths, int nseq, float* last_hidden,
                           void* layer_out);
/* The same pass with ids already on the device (int32 [T]) and the last-token rows left on
 * the device as bf16 [nseq, hidden] at *last_rows (owned by the model, valid until the next
 * call); queue-only, no host synchronisation. */
int s1_model_forward_device(void* model, const int32_t* ids_device, const int* lengths, int nseq, void** last_rows);
int s1_model_sync(void* model);
/* The same pass, queue-only, for a host that keeps several packs in flight: ids in host memory
 * (pinned, if the copy is to overlap; they must stay unchanged until the pass has run), the
 * last-token rows written as bf16 [nseq, hidden] to rows_device, a device buffer of the caller.
 * Validates like s1_model_forward_batch. No host synchronisation. */
int s1_model_forward_queue(void* model, const int32_t* ids_host, const int* lengths, int nseq, void* rows_device);
/* Copies `bytes` from rows_device to dst_host behind everything queued, waits for the stream and
 * checks the device error words as of the last pass: 0, or CS1_ERR_DEVICE_CHECK when a bounded
 * wait gave up (the rows must not be used then). bytes == 0 only waits and checks. */
int s1_model_read_rows(void* model, void* dst_host, const void* rows_device, size_t bytes);

/* ---- Prefix capture and continuation (PrefixState, alloc_prefix, forward_multimodal_capture /
 * _continue, model.rs:557-588, 954-1073; run_window, model.rs:1340-1638), for text positions.
 * A prefix is rows [0, len) of a prompt, len a positive multiple of 64 (the delta rule's chunk):
 * per full-attention layer the post-prep keys and raw values, per Gated DeltaNet layer the
 * float32 state and the last three pre-conv rows. Capture runs those rows once; a continuation
 * runs rows [len, len + c) seeded from them and repeats the one-shot arithmetic (bit for bit
 * when the GEMMs do not split K, i.e. under exact packing; within rounding otherwise - the
 * reference has the same caveat for cuBLASLt's row-count-dependent plans, model.rs:1349-1351).
 * Unlike the reference, which continues one window per call, s1_model_forward_continue takes
 * all candidates of a request at once and packs them through every GEMM. ---- */
int s1_prefix_create(void* model, int len, void** prefix);
void s1_prefix_destroy(void* prefix);
size_t s1_prefix_bytes(void* prefix); /* device bytes held, for a cache budget */
int s1_prefix_len(void* prefix);
/* Run ids[0, len) (len == the prefix's length) and fill the prefix; waits for the device. */
int s1_model_prefix_capture(void* model, const int32_t* ids, int len, void* prefix);
/* nseq continuations of one captured prefix: ids concatenated, lengths[nseq]; candidate i sits at
 * positions [len, len + lengths[i]). last_hidden: float32 [nseq, hidden] in host memory, the
 * final-norm hidden state of each candidate's last token. S1_ERR_ARGUMENT for a prefix of
 * another model, one not yet captured, an empty candidate or one that passes max_positions. */
int s1_model_forward_continue(void* model, const void* prefix, const int32_t* ids, const int* lengths, int nseq,
                              float* last_hidden);


/* Operator families of the layer loop, for launch counts and per-family device time. */
enum {
    S1_FAMILY_GEMM = 0, S1_FAMILY_GDN = 1, S1_FAMILY_ATTENTION = 2, S1_FAMILY_CONV = 3, S1_FAMILY_GATES = 4,
    S1_FAMILY_NORM = 5, S1_FAMILY_GATED_NORM = 6, S1_FAMILY_SILU_MUL = 7, S1_FAMILY_ATTN_PREP = 8,
    S1_FAMILY_OTHER = 9, S1_FAMILIES = 10
};
/* ---- Safetensors checkpoints (Weights::load, model.rs:239-315) ----
 * dir holds model.safetensors, or model.safetensors.index.json and the files it names. The
 * language model's tensors are those under the first of the prefixes "model.language_model.",
 * "model.", "" that has embed_tokens.weight. */
/* Host only (no GPU needed): the prefix, the number of language-model tensors and, for
 * index >= 0, that tensor's name without the prefix, dtype string, rank, shape (up to 8 extents)
 * and byte size. Every out pointer is nullable. */
int s1_checkpoint_inspect(const char* dir, char* prefix_out, size_t prefix_cap, int* n_tensors, int index,
                          char* name_out, size_t name_cap, char* dtype_out, size_t dtype_cap, int* rank,
                          uint64_t* shape8, uint64_t* bytes);
/* Upload every tensor of the decoder from the checkpoint into the model's arena (tensors under
 * the prefix that the decoder has no place for - lm_head, MTP - are skipped). Every tensor under
 * the prefix must be bfloat16 (model.rs:291-295), every tensor of the decoder must have exactly
 * the planned shape (model.rs:306-320: a transposed matrix has the same bytes), and all planned
 * tensors must be present. offender (nullable) receives the name of the tensor an error is about. */
int s1_model_load_checkpoint(void* model, const char* dir, char* offender, size_t offender_cap);
/* open_jev_export.json of a merged Open-Jev export (recipe/open_jev/export_merged.py:82-90,
 * engine.rs:21-46, executor.rs:21-54), host only: format tag "open-jev-text-merged/1",
 * temperature (finite, > 0), max_length (1..=16384), chat_prefix / chat_suffix (strings) and
 * the trained scalar head: `hidden` finite weights into head_weight and a finite bias, rounded
 * from the file's float64 to float32. With s1_head_logits (n_classes = 1) and s1_decide they
 * give a request's scores and decision as the worker computes them. Every out pointer but
 * head_weight is nullable. S1_ERR_CHECKPOINT_IO / _FORMAT, or S1_ERR_EXPORT_FIELD for a missing
 * or invalid field. */
int s1_export_read(const char* dir, int hidden, float* head_weight, float* head_bias, double* temperature,
                   int* max_length, char* model_id, size_t model_id_cap);
/* Number of planned tensors not yet given a value; the first one's name in name_out (nullable). */
int s1_model_unfilled(void* model, char* name_out, size_t cap);

/* Profile mode brackets every operator of eager passes with events on the model's stream. */
int s1_model_profile(void* model, int on);
/* Waits for the stream, then returns and resets: device milliseconds per family since the
 * last read (profile mode only; ms nullable), kernels of this library launched per family
 * (nullable, a graph replay counts the kernels it holds); *library_launches (nullable) is always 0:
 * no vendor library is linked. */
int s1_model_profile_read(void* model, float* ms, long long* launches, long long* library_launches);
/* 1 if cs1_gemm would run this problem on the tcgen05 kernels, 0 if on the plain kernel. */
int s1_gemm_engine(void* gemm, const void* x, const void* w, int M, int N, int K);

/* DecisionHead::score (open_jev executor.rs:56-68) and letter_logits (cua_s1 executor.rs:61-78):
 * float64 accumulation on the host rounded to float32, bias added in float32 (bias nullable).
 * weights [n_classes, hidden] float32, last [hidden] float32, logits [n_classes].
 * Returns 0, or S1_ERR_NONFINITE when a logit is not finite. */
int s1_head_logits(const float* weights, const float* bias, const float* last, int hidden, int n_classes,
                   float* logits);
/* contract::answer's softmax over (x - max) / temperature in float64 and its decision: the
 * first maximum wins (contract.rs:227-247). probs nullable. Returns the argmax or -1. */
int s1_decide(const float* logits, int n, double temperature, double* probs);
/* batching::ranges (open_jev batching.rs:9-25): order-preserving groups of at most 16
 * prompts and 4096 tokens. Writes group starts and returns the number of groups. */
int s1_batch_ranges(const int* lengths, int n, int* starts);
/* Token-balanced assignment of whole requests to n_ranks GPUs: longest processing time
 * first on the cost a*T + b*T^2. rank_of [n]. No counterpart in the reference (single GPU). */
int s1_assign_requests(const int* lengths, int n, int n_ranks, double a, double b, int* rank_of);
/* The same with ranks of unequal speed (speed [n_ranks], relative, > 0; null = all equal): each
 * request, longest first, goes to the rank on which it would finish earliest,
 * (load + cost) / speed. GPUs of one box differ by a few per cent in sustained clock under the
 * board power limit, which is more than the residue of the token balance. */
int s1_assign_requests_weighted(const int* lengths, int n, int n_ranks, double a, double b, const double* speed,
                                int* rank_of);

#define S1_ERR_ARGUMENT 3000
#define S1_ERR_NONFINITE 3001
#define S1_ERR_UNKNOWN_TENSOR 3002
#define S1_ERR_TENSOR_SIZE 3003
#define S1_ERR_CHECKPOINT_IO 3004      /* a checkpoint file cannot be opened or mapped */
#define S1_ERR_CHECKPOINT_FORMAT 3005  /* not a safetensors file / index */
#define S1_ERR_CHECKPOINT_DTYPE 3006   /* a language-model tensor is not bfloat16 (model.rs:291-295) */
#define S1_ERR_CHECKPOINT_MISSING 3007 /* no embed_tokens.weight, or a tensor of the decoder is absent */
#define S1_ERR_EXPORT_FIELD 3008       /* open_jev_export.json lacks a field or holds an invalid value */

#ifdef __cplusplus
}
#endif
#endif
