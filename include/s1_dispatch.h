/* Request dispatcher of libqwen3_5_cuda.so for the GPUs of one box: one process (rank) per GPU,
 * weights replicated, whole requests assigned to ranks by estimated cost, each rank prefilling
 * its share in packs through the host executor (s1_executor.h), the decision logits of all
 * requests gathered to rank 0 with one NCCL all-gather. The forward pass itself never
 * communicates.
 *
 * No counterpart in the reference, which serves from one device (model.rs:625 pins device 0);
 * what a rank runs is the reference's own sequence: packs of at most 16 prompts / 4096 tokens
 * (open_jev batching.rs:5-25) through Model::forward_batch (model.rs:769-823), then the float64
 * host head (open_jev executor.rs:56-68). NCCL is loaded at run time (dlopen of libnccl.so.2)
 * and only when world > 1, so a single-GPU host needs no NCCL at all.
 */
#ifndef S1_DISPATCH_H
#define S1_DISPATCH_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define S1_ERR_DISPATCH_NCCL 3100       /* libnccl.so.2 cannot be loaded or lacks a symbol */
#define S1_ERR_DISPATCH_RENDEZVOUS 3101 /* the communicator id could not be exchanged through the file */
#define S1_ERR_DISPATCH_COMM 3102       /* an NCCL call failed */
#define S1_ERR_DISPATCH_STATE 3103      /* call out of order (no plan, nothing staged, ...) */

/* Joins `world` ranks. device: this rank's GPU. rendezvous: a path on a file system all ranks
 * share (one box: /dev/shm or /tmp), unique to this job; rank 0 writes the NCCL id there and
 * removes the file once every rank has joined; ignored when world == 1. nccl_library: path of
 * libnccl.so.2, or null for the loader's default search. */
int s1_dispatch_create(int rank, int world, int device, const char* rendezvous, const char* nccl_library, void** out);
void s1_dispatch_destroy(void* dispatch);

/* Cost of a request of T tokens for the assignment: a T + b T^2 (default a = 1, b = 4e-6: the
 * attention layers' quadratic share on the 27B-shaped decoder). Every rank must set the same. */
int s1_dispatch_set_cost(void* dispatch, double a, double b);

/* Relative speed of every rank's GPU for the assignment (speed [world], > 0; null puts all back
 * to equal): requests go where they finish earliest, (load + cost) / speed
 * (s1_assign_requests_weighted). A host measures it as planned cost / busy time of a few passes.
 * Every rank must set the same values. Takes effect at the next s1_dispatch_plan. */
int s1_dispatch_set_speed(void* dispatch, const double* speed, int world);

/* The plan alone, on the host (no GPU, no communicator): rank_of [n] for all requests and, for
 * `rank`, its requests in run order (local_index, up to n entries) with their count in *n_local
 * and the first local request of each pack (pack_start, up to n entries). Returns the number of
 * packs, or a negative error code. */
int s1_dispatch_layout(const int* lengths, int n, int world, double a, double b, int rank, int* rank_of,
                       int* local_index, int* n_local, int* pack_start);

/* s1_dispatch_layout with per-rank speeds (speed [world] or null), as s1_dispatch_set_speed takes them. */
int s1_dispatch_layout_weighted(const int* lengths, int n, int world, double a, double b, const double* speed, int rank,
                                int* rank_of, int* local_index, int* n_local, int* pack_start);

/* Plans a request set (every rank passes the same lengths): s1_assign_requests_weighted over all ranks,
 * each rank's requests ordered by length (so that short prompts share packs), packs by
 * s1_batch_ranges. Allocates the staging buffers for `model` (hidden size, stream) and
 * n_classes logits per request. */
int s1_dispatch_plan(void* dispatch, void* model, const int* lengths, int n, int n_classes);
/* What the plan gave this rank (every out pointer nullable): requests, tokens, packs; rank_of [n]. */
int s1_dispatch_info(void* dispatch, int* n_local, long long* local_tokens, int* n_packs, int* rank_of);
/* Request indices of this rank in the order it runs them, local_index [n_local], and the first
 * local request of each pack, pack_start [n_packs]. */
int s1_dispatch_local(void* dispatch, int* local_index, int* pack_start);

/* Copies this rank's prompts out of ids_all (all n requests concatenated in request order, host)
 * into the dispatcher's pinned buffer: the state "ids in pinned host memory" an end-to-end step
 * starts from. */
int s1_dispatch_stage(void* dispatch, const int32_t* ids_all);
/* Makes the staged ids resident on the device too (waits), for steps timed without the copy. */
int s1_dispatch_upload(void* dispatch);

/* Queues every pack of this rank on the model's stream, nothing else: resident = 0 copies each
 * pack's ids from the pinned buffer first (s1_model_forward_queue), 1 uses the device copy
 * (s1_model_forward_device). Last-token rows land in the dispatcher's device buffer. */
int s1_dispatch_enqueue(void* dispatch, int resident);
/* Device milliseconds of each pack of the last s1_dispatch_enqueue (events around it), after
 * waiting for the stream. pack_ms [n_packs]. */
int s1_dispatch_pack_ms(void* dispatch, float* pack_ms);

/* After s1_dispatch_enqueue: reads the rows back (checking the device error words), applies the
 * head to each (s1_head_logits: float64 accumulation, float32 result, bias nullable), and gathers
 * all ranks' logits. Rank 0 receives logits [n, n_classes] in request order; on other ranks
 * `logits` may be null. gather_us (nullable): host microseconds of the exchange, which include
 * the wait for the slowest rank. */
int s1_dispatch_collect(void* dispatch, const float* head_weights, const float* head_bias, float* logits,
                        double* gather_us);

/* Small collectives for the harness around it (timing protocol, statistics): all ranks. */
/* One multi-candidate request over the ranks: n candidates continue one shared prefix that every
 * rank has captured itself (weights and prefix are replicated: s1_prefix_create +
 * s1_model_prefix_capture on each rank's model). The candidates are assigned to ranks by length
 * (s1_assign_requests_weighted with the speeds set), each rank continues its share in packed
 * passes (s1_model_forward_continue), applies the head, and the logits are gathered to rank 0 in
 * candidate order: logits [n, n_classes] there, may be null elsewhere. ids: all candidates
 * concatenated, lengths [n], the same on every rank. rank_of_out (nullable): where each went.
 * Waits for the device. The single-GPU form of this in the reference is
 * forward_multimodal_capture / _continue (model.rs:954-1073), one candidate per call. */
int s1_dispatch_candidates(void* dispatch, void* model, const void* prefix, const int32_t* ids, const int* lengths, int n,
                           const float* head_weights, const float* head_bias, int n_classes, float* logits,
                           int* rank_of_out);

int s1_dispatch_barrier(void* dispatch);
int s1_dispatch_allreduce_max(void* dispatch, double* values, int n);
int s1_dispatch_allgather(void* dispatch, const double* values, int n, double* all /* [world, n] */);

#ifdef __cplusplus
}
#endif
#endif
