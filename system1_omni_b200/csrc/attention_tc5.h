// Internal interface of the tcgen05 attention kernel (attention_tc5.cu), used by attention.cu.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

// Causal GQA attention of positions [q_base, T) over keys [0, T). q, gate, out, k and v hold the
// positions from own_base on (indexed from zero); keys and values of positions below own_base are
// read from kpre / vpre (row stride ldvpre). gate null = ungated. Dh 128 or 256; q, k, v, kpre, vpre
// 16-byte aligned, ldv and ldvpre multiples of 8. Returns 0, a cudaError_t or CS1_ERR_TENSOR_MAP.
int s1_attn_tc5(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v, int ldv,
                const __nv_bfloat16* gate, __nv_bfloat16* out, int T, int Hq, int Hk, int Dh, float scale, int q_base,
                const __nv_bfloat16* kpre, const __nv_bfloat16* vpre, int ldvpre, int own_base, cudaStream_t stream);
// The same for nseq <= 16 sequences in one launch: sequence i has positions [0, T[i]), T[i] > q_base, and its own
// rows (positions from own_base on) start at row row0[i] of q, k, v, gate and out; the prefix below own_base
// (kpre, vpre) is shared by all of them. The same bits as one call per sequence.
int s1_attn_tc5_batch(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v, int ldv,
                      const __nv_bfloat16* gate, __nv_bfloat16* out, const int* row0, const int* T, int nseq, int Hq, int Hk,
                      int Dh, float scale, int q_base, const __nv_bfloat16* kpre, const __nv_bfloat16* vpre, int ldvpre,
                      int own_base, cudaStream_t stream);
// Non-causal attention over all n positions with head dim 64 and heads == key-value heads (the
// vision tower): q, k, out [n, heads, 64], v rows ldv elements apart. Same return codes.
int s1_attn_tc5_full64(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v, int ldv,
                       __nv_bfloat16* out, int n, int heads, float scale, cudaStream_t stream);
