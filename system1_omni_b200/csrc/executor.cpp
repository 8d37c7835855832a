// Host executor of the Qwen3.5-style hybrid decoder prefill: weight arena, scratch plan,
// layer loop, packed batches, CUDA-graph cache, last-token readout, decision heads, packing
// policy and the multi-GPU request assignment. It drives the device only through the
// cs1_* C ABI of this library, the way the reference's Rust executor does
// (src/models/qwen3_5/native/src/model.rs); citations below are to that file unless noted.
#include <cuda_runtime.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <cmath>
#include <deque>
#include <initializer_list>
#include <numeric>
#include <string>
#include <unordered_map>
#include <vector>

#include "cs1_ops.h"
#include "exec_kernels.h"
#include "s1_executor.h"
#include "status.h"

namespace {

constexpr int PACK_SEQS = 16;  // sequences of one pack (s1_batch_ranges); what the batched operators take per launch


constexpr size_t ALIGN = 256;  // model.rs:23
constexpr size_t BF16 = 2, F32 = 4;
constexpr size_t GEMM_WORKSPACE = 32u << 20;  // model.rs:26
constexpr int GRAPH_CACHE = 64;               // model.rs:879-882
constexpr int ENDS_RING = 16;

#define S1_TRY(expr)            \
    do {                        \
        const int rc_ = (expr); \
        if (rc_ != 0) return rc_; \
    } while (0)

struct Tensor {
    size_t offset = 0, bytes = 0;
    bool filled = false;
    int rank = 0;
    uint64_t shape[3] = {};  // the checkpoint tensor's shape (Weights::get, model.rs:306-320)
};

// Byte offsets into one scratch allocation for up to `cap` tokens (model.rs:415-555).
struct Scratch {
    size_t cap = 0;
    void* buf = nullptr;
    size_t ws_floats = 0;  // floats the delta rule's workspace holds
    size_t ids, res, x, delta, gdn_in, beta, g, lq, lk, lv, lo, ln, workspace, attn_in, aq, agate, ak, ao, gate_up,
        act, cos, sin, ends, last, status, total;
    char* at(size_t off) const { return static_cast<char*>(buf) + off; }
};

struct Layer {
    bool full = false;
    Tensor input_norm, post_norm, gate_up, down;
    Tensor in_proj, conv, a_log, dt_bias, norm, out;  // Gated DeltaNet
    Tensor qkv, o, q_norm, k_norm;                    // full attention
};

struct ProfRecord {
    int family;
    cudaEvent_t start, stop;
};

struct Model {
    S1Config cfg{};
    bool profiling = false;
    std::vector<ProfRecord> prof;
    std::vector<cudaEvent_t> events;
    size_t events_used = 0;
    long long launches[S1_FAMILIES] = {};
    long long library_launches = 0;
    std::vector<unsigned char> full;
    int device = 0;
    void* arena = nullptr;
    size_t arena_bytes = 0;
    std::unordered_map<std::string, Tensor> named;  // every checkpoint tensor
    std::vector<std::pair<std::string, Tensor>> order;
    Tensor embed, final_norm;
    std::vector<Layer> layers;
    void* stream = nullptr;
    void* gemm = nullptr;
    Scratch s;
    bool graph_enabled = false;
    bool exact_packing = true;  // whole-tile GEMMs: a prompt's bits do not depend on what it is packed with
    bool fuse_swiglu = true;  // gate/up GEMM and SiLU-multiply as one kernel where the engine supports it
    int overlap_tokens = 128;  // eager passes of at most this many tokens launch every kernel as a programmatic dependent
    bool capturing = false;    // the pass being issued is recorded into a graph
    int replays = 0, captures = 0;
    struct Recorded {
        std::vector<int> key;
        void* exec;
        long long kernels[S1_FAMILIES];  // what one replay launches, per family
    };
    std::deque<Recorded> graphs;
    int* ends_host = nullptr;  // pinned ring of ENDS_RING slots of cap ints
    size_t ends_slot = 0;
    cudaEvent_t ends_event[ENDS_RING] = {};  // recorded behind the copy out of a slot; awaited before the slot is rewritten
    int* status_host = nullptr;               // pinned: the three device error words as of the last pass read back
    std::deque<std::vector<int>> seen_once;   // length vectors run eagerly once, captured when they come again
    void* last_host = nullptr;  // pinned staging of the last rows
    size_t last_host_bytes = 0;

    int key_dim() const { return cfg.lin_k_heads * 128; }
    int value_dim() const { return cfg.lin_v_heads * 128; }
    int conv_w() const { return 2 * key_dim() + value_dim(); }
    int gdn_in_w() const { return conv_w() + value_dim() + 2 * cfg.lin_v_heads; }
    int attn_q_w() const { return cfg.heads * cfg.head_dim * 2; }
    int attn_in_w() const { return attn_q_w() + 2 * cfg.kv_heads * cfg.head_dim; }
    char* w(const Tensor& t) const { return static_cast<char*>(arena) + t.offset; }
};

void clear_graphs(Model* m) {
    for (auto& g : m->graphs) cs1_graph_destroy(g.exec);
    m->graphs.clear();
    m->seen_once.clear();
}

// What the kernels implement (model.rs:134-180), with head_dim 128 accepted besides 256.
int validate(const S1Config& c) {
    if (c.hidden <= 0 || c.hidden % 8 || c.intermediate <= 0 || c.intermediate % 8 || c.n_layers <= 0 || c.vocab <= 0)
        return S1_ERR_ARGUMENT;
    if (c.head_dim != 128 && c.head_dim != 256) return S1_ERR_ARGUMENT;
    if (c.kv_heads <= 0 || c.heads <= 0 || c.heads % c.kv_heads) return S1_ERR_ARGUMENT;
    if (c.lin_k_heads <= 0 || c.lin_v_heads <= 0 || c.lin_v_heads % c.lin_k_heads) return S1_ERR_ARGUMENT;
    if (c.rotary_half <= 0 || c.rotary_half % 8 || 2 * c.rotary_half > c.head_dim ||
        ((c.rotary_half / 8) & (c.rotary_half / 8 - 1)))
        return S1_ERR_ARGUMENT;
    if (c.max_positions <= 0 || c.max_positions > (1 << 24)) return S1_ERR_ARGUMENT;
    if (!(c.rope_theta > 0.0) || !isfinite(c.rope_theta) || !c.full_attention) return S1_ERR_ARGUMENT;
    return 0;
}

// Arena plan: by layer, the members of a stacked GEMM group back to back (model.rs:205-231).
void plan_arena(Model* m) {
    const S1Config& c = m->cfg;
    size_t at = 0;
    auto place = [&](const std::string& name, std::initializer_list<size_t> shape, bool aligned) {
        if (aligned) at = (at + ALIGN - 1) / ALIGN * ALIGN;
        Tensor t;
        size_t elems = 1;
        for (size_t extent : shape) {
            t.shape[t.rank++] = extent;
            elems *= extent;
        }
        t.offset = at;
        t.bytes = elems * BF16;
        at += t.bytes;
        m->named[name] = t;
        m->order.emplace_back(name, t);
        return t;
    };
    auto join = [](const Tensor& first, const Tensor& last) {
        Tensor t;
        t.offset = first.offset;
        t.bytes = last.offset + last.bytes - first.offset;
        return t;
    };
    const size_t h = c.hidden, I = c.intermediate, kd = m->key_dim(), vd = m->value_dim(), hv = c.lin_v_heads;
    const size_t hq = c.heads, hk = c.kv_heads, hd = c.head_dim;
    m->embed = place("embed_tokens.weight", {(size_t)c.vocab, h}, true);
    m->final_norm = place("norm.weight", {h}, true);
    m->layers.resize(c.n_layers);
    for (int i = 0; i < c.n_layers; i++) {
        const std::string p = "layers." + std::to_string(i) + ".";
        Layer& ly = m->layers[i];
        ly.full = m->full[i] != 0;
        if (!ly.full) {
            const Tensor a = place(p + "linear_attn.in_proj_qkv.weight", {2 * kd + vd, h}, true);
            place(p + "linear_attn.in_proj_z.weight", {vd, h}, false);
            place(p + "linear_attn.in_proj_b.weight", {hv, h}, false);
            const Tensor d = place(p + "linear_attn.in_proj_a.weight", {hv, h}, false);
            ly.in_proj = join(a, d);
        } else {
            const Tensor a = place(p + "self_attn.q_proj.weight", {hq * hd * 2, h}, true);
            place(p + "self_attn.k_proj.weight", {hk * hd, h}, false);
            const Tensor d = place(p + "self_attn.v_proj.weight", {hk * hd, h}, false);
            ly.qkv = join(a, d);
        }
        {
            const Tensor a = place(p + "mlp.gate_proj.weight", {I, h}, true);
            const Tensor d = place(p + "mlp.up_proj.weight", {I, h}, false);
            ly.gate_up = join(a, d);
        }
        ly.down = place(p + "mlp.down_proj.weight", {h, I}, true);
        ly.input_norm = place(p + "input_layernorm.weight", {h}, true);
        ly.post_norm = place(p + "post_attention_layernorm.weight", {h}, true);
        if (!ly.full) {
            ly.conv = place(p + "linear_attn.conv1d.weight", {2 * kd + vd, 1, 4}, true);
            ly.a_log = place(p + "linear_attn.A_log", {hv}, true);
            ly.dt_bias = place(p + "linear_attn.dt_bias", {hv}, true);
            ly.norm = place(p + "linear_attn.norm.weight", {128}, true);
            ly.out = place(p + "linear_attn.out_proj.weight", {h, vd}, true);
        } else {
            ly.o = place(p + "self_attn.o_proj.weight", {h, hq * hd}, true);
            ly.q_norm = place(p + "self_attn.q_norm.weight", {hd}, true);
            ly.k_norm = place(p + "self_attn.k_norm.weight", {hd}, true);
        }
    }
    m->arena_bytes = (at + ALIGN - 1) / ALIGN * ALIGN;
}

inline uint16_t f2bf(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
inline float bf2f(uint16_t b) {
    const uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

// cos/sin tables [positions, half] in bf16 for text positions 0..n-1 (all three rotary axes
// equal): float32 inverse frequencies and products, float64 trigonometry (inputs.rs:69-95).
void rotary_tables(int n, int half, double theta, std::vector<uint16_t>& cos_t, std::vector<uint16_t>& sin_t) {
    std::vector<float> inv(half);
    for (int i = 0; i < half; i++) inv[i] = 1.0f / powf((float)theta, (float)(2 * i) / (float)(2 * half));
    cos_t.resize((size_t)n * half);
    sin_t.resize((size_t)n * half);
    for (int t = 0; t < n; t++)
        for (int i = 0; i < half; i++) {
            const double angle = (double)(inv[i] * (float)t);
            cos_t[(size_t)t * half + i] = f2bf((float)cos(angle));
            sin_t[(size_t)t * half + i] = f2bf((float)sin(angle));
        }
}

int make_scratch(Model* m, size_t cap) {
    const S1Config& c = m->cfg;
    Scratch& s = m->s;
    if (s.buf) {
        S1_TRY(cs1_stream_sync(m->stream));
        S1_TRY(cs1_free(s.buf));
        s.buf = nullptr;
        s.cap = 0;
    }
    if (m->ends_host) {
        cudaFreeHost(m->ends_host);
        m->ends_host = nullptr;
    }
    const size_t h = c.hidden, kd = m->key_dim(), vd = m->value_dim(), hv = c.lin_v_heads;
    const size_t hq = c.heads, hk = c.kv_heads, hd = c.head_dim;
    size_t next = 0;
    auto take = [&](size_t bytes) {
        const size_t off = next;
        next = (off + bytes + ALIGN - 1) / ALIGN * ALIGN;
        return off;
    };
    // every sequence of a pack rounds its own last chunk up: at most one more chunk per sequence
    const size_t ws_floats = cs1_gdn_workspace_floats((int)cap + 64 * PACK_SEQS, (int)hv);
    s.ws_floats = ws_floats;
    s.ids = take(cap * 4);
    s.res = take(cap * h * BF16);
    s.x = take(cap * h * BF16);
    s.delta = take(cap * h * BF16);
    s.gdn_in = take(cap * m->gdn_in_w() * BF16);
    s.beta = take(cap * hv * BF16);
    s.g = take(cap * hv * F32);
    s.lq = take(cap * kd * BF16);
    s.lk = take(cap * kd * BF16);
    s.lv = take(cap * vd * BF16);
    s.lo = take(cap * vd * BF16);
    s.ln = take(cap * vd * BF16);
    s.workspace = take(ws_floats * F32);
    s.attn_in = take(cap * m->attn_in_w() * BF16);
    s.aq = take(cap * hq * hd * BF16);
    s.agate = take(cap * hq * hd * BF16);
    s.ak = take(cap * hk * hd * BF16);
    s.ao = take(cap * hq * hd * BF16);
    s.gate_up = take(cap * 2 * c.intermediate * BF16);
    s.act = take(cap * c.intermediate * BF16);
    s.cos = take(cap * c.rotary_half * BF16);
    s.sin = take(cap * c.rotary_half * BF16);
    s.ends = take(cap * 4);
    s.last = take(cap * h * BF16);  // at most one row per prompt, at most cap prompts
    s.status = take(4 * sizeof(int));
    s.total = next;
    S1_TRY(cs1_malloc(&s.buf, s.total));
    s.cap = cap;
    std::vector<uint16_t> cos_t, sin_t;
    const size_t npos = std::min(cap, (size_t)c.max_positions);
    rotary_tables((int)npos, c.rotary_half, c.rope_theta, cos_t, sin_t);
    S1_TRY(cs1_upload(s.at(s.cos), cos_t.data(), cos_t.size() * 2, m->stream));
    S1_TRY(cs1_upload(s.at(s.sin), sin_t.data(), sin_t.size() * 2, m->stream));
    S1_TRY((int)cudaHostAlloc(reinterpret_cast<void**>(&m->ends_host), ENDS_RING * cap * sizeof(int),
                              cudaHostAllocDefault));
    return 0;
}

// Grow to the next multiple of 1024 tokens; a new scratch invalidates captured graphs (model.rs:747-761).
int prepare_scratch(Model* m, size_t t) {
    S1_TRY(cs1_set_device(m->device));
    if (m->s.buf == nullptr || t > m->s.cap) {
        clear_graphs(m);
        S1_TRY(make_scratch(m, (t + 1023) / 1024 * 1024));
    }
    return 0;
}

cudaEvent_t next_event(Model* m) {
    if (m->events_used == m->events.size()) {
        cudaEvent_t e = nullptr;
        if (cudaEventCreate(&e) != cudaSuccess) return nullptr;
        m->events.push_back(e);
    }
    return m->events[m->events_used++];
}

// Every device operator of the layer loop goes through here: counts the kernels it launches
// per operator family and, in profile mode, brackets it with events on the model's stream.
template <typename F>
int op(Model* m, int family, int kernels, F&& call) {
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaStream_t st = static_cast<cudaStream_t>(m->stream);
    if (m->profiling && (e0 = next_event(m))) cudaEventRecord(e0, st);
    const int rc = call();
    if (m->profiling && e0 && (e1 = next_event(m))) {
        cudaEventRecord(e1, st);
        m->prof.push_back({family, e0, e1});
    }
    m->launches[family] += kernels;
    return rc;
}
#define S1_OP(family, kernels, expr) S1_TRY(op(m, family, kernels, [&] { return (expr); }))

int gemm(Model* m, size_t x, const Tensor& w, size_t y, int rows, int n, int k) {
    return op(m, S1_FAMILY_GEMM, 1, [&] {
        // exact packing: whole tiles only, so a row's sum over K runs in one fixed order
        // whatever the row count of the call (packed, alone, or continuing a prefix)
        if (m->exact_packing)
            return s1_gemm_unsplit(m->gemm, m->s.at(x), m->w(w), m->s.at(y), rows, n, k, n, m->stream);
        return cs1_gemm(m->gemm, m->s.at(x), m->w(w), m->s.at(y), rows, n, k, n, m->stream);
    });
}

// The projections back to the hidden size (out / o / down). The reference runs them per
// sequence (gemm_sequences, model.rs:723-739) so that a prompt sees the same GEMM shape, hence
// the same library plan, packed or alone. Here a row's result does not depend on the call's row
// count once the tiles are whole (exact packing; the plain kernel always sums k in order), so
// the projection runs once over the pack in every mode.
int gemm_rows(Model* m, size_t x, const Tensor& w, size_t y, const int* lengths, int nseq, int n, int k) {
    int t = 0;
    for (int i = 0; i < nseq; i++) t += lengths[i];
    return gemm(m, x, w, y, t, n, k);
}

// Second half of a layer (model.rs:1287-1336): residual add + post norm, SwiGLU MLP, residual
// add + the next layer's input norm (the final norm after the last layer).
int mlp_block(Model* m, size_t li, const int* lengths, int nseq, int t) {
    const S1Config& c = m->cfg;
    const Scratch& s = m->s;
    void* st = m->stream;
    const Layer& ly = m->layers[li];
    const int h = c.hidden, I = c.intermediate;
    const float eps = c.eps;
    S1_OP(S1_FAMILY_NORM, 1,
          cs1_add_rms_norm(s.at(s.res), s.at(s.delta), m->w(ly.post_norm), s.at(s.x), t, h, eps, st));
    // gate/up projection and SiLU-multiply: one kernel where the tcgen05 engine takes it
    // (same bits as the two operators), else the reference's sequence
    int fused = CS1_ERR_UNSUPPORTED;
    if (m->fuse_swiglu) {
        S1_TRY(op(m, S1_FAMILY_GEMM, 0, [&] {
            fused = s1_gemm_swiglu(m->gemm, s.at(s.x), m->w(ly.gate_up), s.at(s.act), t, I, h, I, st);
            return fused == CS1_ERR_UNSUPPORTED ? 0 : fused;
        }));
        if (fused == 0) m->launches[S1_FAMILY_GEMM] += 1;
    }
    if (fused == CS1_ERR_UNSUPPORTED) {
        S1_TRY(gemm(m, s.x, ly.gate_up, s.gate_up, t, 2 * I, h));
        S1_OP(S1_FAMILY_SILU_MUL, 1, cs1_silu_mul(s.at(s.gate_up), 2 * I, s.at(s.act), t, I, st));
    }
    S1_TRY(gemm_rows(m, s.act, ly.down, s.delta, lengths, nseq, h, I));
    const Tensor& next = li + 1 < m->layers.size() ? m->layers[li + 1].input_norm : m->final_norm;
    S1_OP(S1_FAMILY_NORM, 1, cs1_add_rms_norm(s.at(s.res), s.at(s.delta), m->w(next), s.at(s.x), t, h, eps, st));
    return 0;
}

// Convolution and gates of rows [off, off + len) of the input projection's output: one launch
// where the fused kernel takes the shapes (same bits), else the reference's two operators.
int conv_gates(Model* m, const Layer& ly, size_t off, int len) {
    const Scratch& s = m->s;
    void* st = m->stream;
    const int kd = m->key_dim(), vd = m->value_dim(), hv = m->cfg.lin_v_heads, gdn_in = m->gdn_in_w(), conv = m->conv_w();
    const size_t row = s.gdn_in + off * gdn_in * BF16;
    const size_t b = row + (size_t)(conv + vd) * BF16, a = b + (size_t)hv * BF16;
    float* g = reinterpret_cast<float*>(s.at(s.g + off * hv * F32));
    int fused = CS1_ERR_UNSUPPORTED;
    if (m->fuse_swiglu) {
        S1_TRY(op(m, S1_FAMILY_CONV, 0, [&] {
            fused = s1_gdn_conv_gates(s.at(row), gdn_in, m->w(ly.conv), s.at(s.lq + off * kd * BF16),
                                      s.at(s.lk + off * kd * BF16), s.at(s.lv + off * vd * BF16), len, kd, vd, s.at(b),
                                      s.at(a), m->w(ly.a_log), m->w(ly.dt_bias), s.at(s.beta + off * hv * BF16), g, hv, st);
            return fused == CS1_ERR_UNSUPPORTED ? 0 : fused;
        }));
        if (fused == 0) m->launches[S1_FAMILY_CONV] += 1;
    }
    if (fused == CS1_ERR_UNSUPPORTED) {
        S1_OP(S1_FAMILY_CONV, 1,
              cs1_gdn_conv(s.at(row), gdn_in, m->w(ly.conv), s.at(s.lq + off * kd * BF16), s.at(s.lk + off * kd * BF16),
                           s.at(s.lv + off * vd * BF16), len, kd, vd, st));
        S1_OP(S1_FAMILY_GATES, 1,
              cs1_gdn_gates(s.at(b), s.at(a), gdn_in, m->w(ly.a_log), m->w(ly.dt_bias), s.at(s.beta + off * hv * BF16), g,
                            len, hv, st));
    }
    return 0;
}

// conv_gates of every sequence of the pack: one launch where the fused kernel takes the shapes,
// else sequence by sequence.
int conv_gates_pack(Model* m, const Layer& ly, const int* lengths, int nseq) {
    const Scratch& s = m->s;
    const int kd = m->key_dim(), vd = m->value_dim(), hv = m->cfg.lin_v_heads, gdn_in = m->gdn_in_w(), conv = m->conv_w();
    const size_t b = s.gdn_in + (size_t)(conv + vd) * BF16, a = b + (size_t)hv * BF16;
    for (int first = 0, off = 0; first < nseq;) {
        const int n = std::min(nseq - first, PACK_SEQS);
        int row0[PACK_SEQS];
        for (int i = 0, at = off; i < n; i++) {
            row0[i] = at;
            at += lengths[first + i];
        }
        int fused = CS1_ERR_UNSUPPORTED;
        if (m->fuse_swiglu && n > 1) {
            S1_TRY(op(m, S1_FAMILY_CONV, 0, [&] {
                fused = s1_gdn_conv_gates_batch(s.at(s.gdn_in), gdn_in, m->w(ly.conv), s.at(s.lq), s.at(s.lk), s.at(s.lv), row0,
                                                lengths + first, n, kd, vd, s.at(b), s.at(a), m->w(ly.a_log), m->w(ly.dt_bias),
                                                s.at(s.beta), reinterpret_cast<float*>(s.at(s.g)), hv, m->stream);
                return fused == CS1_ERR_UNSUPPORTED ? 0 : fused;
            }));
            if (fused == 0) m->launches[S1_FAMILY_CONV] += 1;
        }
        for (int i = 0; i < n; i++) {
            if (fused == CS1_ERR_UNSUPPORTED) S1_TRY(conv_gates(m, ly, (size_t)row0[i], lengths[first + i]));
            off += lengths[first + i];
        }
        first += n;
    }
    return 0;
}

// The delta rule of every sequence of the pack in one pair of launches (the reference calls its
// operator once per sequence, model.rs:690-712): sequence q owns lengths[q] packed rows of which
// the first `lead` are skipped. s_in: the state all of them start from (null = zero); s_out: where
// the state after the sequence goes (capture; one sequence then).
int delta_rule(Model* m, const int* lengths, int nseq, int lead, const void* s_in, void* s_out) {
    const Scratch& s = m->s;
    const S1Config& c = m->cfg;
    const int hv = c.lin_v_heads;
    for (int first = 0, off = 0; first < nseq;) {  // a pack has at most PACK_SEQS sequences; callers of the layer loop may pass more
        const int n = std::min(nseq - first, PACK_SEQS);
        int row0[PACK_SEQS], len[PACK_SEQS];
        for (int i = 0; i < n; i++) {
            row0[i] = off + lead;
            len[i] = lengths[first + i] - lead;
            off += lengths[first + i];
        }
        S1_OP(S1_FAMILY_GDN, 2,
              s1_gdn_prefill_batch(s.at(s.lq), s.at(s.lk), s.at(s.lv), reinterpret_cast<const float*>(s.at(s.g)), s.at(s.beta),
                                   s.at(s.lo), reinterpret_cast<float*>(s.at(s.workspace)), s.ws_floats, row0, len, n, hv,
                                   c.lin_k_heads, 1.0f / sqrtf(128.0f), s_in, s_out, m->stream));
        first += n;
    }
    return 0;
}

// Norm, rotary and gate split, then gated causal attention, of every sequence of the pack in one
// launch each (the reference calls both operators once per sequence, model.rs:1244-1268). Sequence
// q owns lengths[q] of the t packed rows, the first `lead` of them skipped, and sits at positions
// from qb on behind the shared prefix k_pre / v_pre (null: none). keep_k / keep_v (capture; one
// sequence then): where the keys after norm and rotary and the values as projected are copied to.
int attention_pack(Model* m, const Layer& ly, const int* lengths, int nseq, int t, int lead, int qb, const void* k_pre,
                   const void* v_pre, void* keep_k, void* keep_v) {
    const Scratch& s = m->s;
    const S1Config& c = m->cfg;
    void* st = m->stream;
    const int hq = c.heads, hk = c.kv_heads, hd = c.head_dim, attn_in = m->attn_in_w(), attn_q = m->attn_q_w();
    const size_t kv_row = (size_t)hk * hd * BF16;
    const size_t k = s.attn_in + (size_t)attn_q * BF16, v = k + kv_row;
    for (int first = 0, off = 0; first < nseq;) {
        const int n = std::min(nseq - first, PACK_SEQS);
        int row0[PACK_SEQS], rows[PACK_SEQS];
        for (int i = 0; i < n; i++) {
            row0[i] = off + lead;
            rows[i] = lengths[first + i] - lead;
            off += lengths[first + i];
        }
        // the tables from position qb on: every sequence restarts there (model.rs:1244-1251)
        S1_OP(S1_FAMILY_ATTN_PREP, 1,
              s1_attn_prep_batch(s.at(s.attn_in), s.at(k), attn_in, m->w(ly.q_norm), m->w(ly.k_norm),
                                 s.at(s.cos + (size_t)qb * c.rotary_half * BF16), s.at(s.sin + (size_t)qb * c.rotary_half * BF16),
                                 s.at(s.aq), s.at(s.agate), s.at(s.ak), t, row0, rows, n, hq, hk, hd, c.rotary_half, c.eps, st));
        if (keep_k) {
            S1_TRY(cs1_copy_dd(keep_k, s.at(s.ak + (size_t)row0[0] * kv_row), (size_t)rows[0] * kv_row, st));
            S1_TRY(cs1_copy2d(keep_v, kv_row, s.at(v + (size_t)row0[0] * attn_in * BF16), (size_t)attn_in * BF16, kv_row, rows[0], st));
        }
        S1_OP(S1_FAMILY_ATTENTION, 1,
              s1_attention_gated_batch(s.at(s.aq), s.at(s.ak), s.at(v), attn_in, s.at(s.agate), s.at(s.ao), k_pre, v_pre, hk * hd,
                                       qb, row0, rows, n, hq, hk, hd, 1.0f / sqrtf((float)hd), st));
        first += n;
    }
    return 0;
}

// The layer loop (model.rs:1119-1338). Pointwise operators and the input / gate-up GEMMs run
// once over the packed rows; conv, delta rule, attention prep and attention run per sequence.
// dump (nullable, host) receives the residual stream after each layer.
// Dependent launch for the launches of one pass, put back on every way out. Short passes make
// (nearly) every kernel a programmatic dependent of the one before it, longer ones the GEMMs and norms (a GEMM's
// blocks arrive under the short kernel ahead and fetch their first ring of weight tiles there);
// overlap_tokens < 0 keeps plain stream order. Measured on the 4B-shaped decoder (ms per pass,
// plain / every kernel / GEMMs only; leaving out the delta-rule kernels and adding the norms gained 2-5 % more): issued eagerly 3.81 / 3.29 / 3.45 at 64 tokens, 4.22 / 3.72 /
// 3.78 at 128, 4.70 / 4.41 / 4.27 at 256, 9.34 / 9.06 / 9.09 at 1024; replayed from a graph, where
// the gaps between launches are small already, 3.11 / 3.17 / 2.93 at 64, 4.02 / 4.29 / 3.85 at 256,
// 8.69 / 8.88 / 8.50 at 1024, no difference from 4096 on. So an eager pass of up to overlap_tokens
// tokens makes every kernel a dependent, every other pass the GEMMs only.
struct OverlapScope {
    int before;
    static int mode(const Model* m, int tokens) {
        if (m->overlap_tokens < 0) return 0;
        return !m->capturing && tokens <= m->overlap_tokens ? 1 : 2;
    }
    OverlapScope(const Model* m, int tokens) : before(s1_set_dependent_launch(mode(m, tokens))) {}
    ~OverlapScope() { s1_set_dependent_launch(before); }
};

int run(Model* m, const int* lengths, int nseq, char* dump) {
    const S1Config& c = m->cfg;
    const Scratch& s = m->s;
    void* st = m->stream;
    int t = 0;
    for (int i = 0; i < nseq; i++) t += lengths[i];
    const OverlapScope overlap(m, t);
    const int h = c.hidden, vd = m->value_dim(), hv = c.lin_v_heads;
    const int hq = c.heads, hd = c.head_dim;
    const int gdn_in = m->gdn_in_w(), attn_in = m->attn_in_w(), conv = m->conv_w();
    const float eps = c.eps;
    S1_OP(S1_FAMILY_NORM, 1, cs1_rms_norm(s.at(s.res), m->w(m->layers[0].input_norm), s.at(s.x), t, h, eps, st));
    for (size_t li = 0; li < m->layers.size(); li++) {
        const Layer& ly = m->layers[li];
        if (!ly.full) {
            S1_TRY(gemm(m, s.x, ly.in_proj, s.gdn_in, t, gdn_in, h));
            const size_t z = s.gdn_in + (size_t)conv * BF16;
            S1_TRY(conv_gates_pack(m, ly, lengths, nseq));
            S1_TRY(delta_rule(m, lengths, nseq, 0, nullptr, nullptr));
            S1_OP(S1_FAMILY_GATED_NORM, 1,
                  cs1_gated_rms_norm(s.at(s.lo), s.at(z), gdn_in, m->w(ly.norm), s.at(s.ln), t, hv, 128, eps, st));
            S1_TRY(gemm_rows(m, s.ln, ly.out, s.delta, lengths, nseq, h, vd));
        } else {
            S1_TRY(gemm(m, s.x, ly.qkv, s.attn_in, t, attn_in, h));
            S1_TRY(attention_pack(m, ly, lengths, nseq, t, 0, 0, nullptr, nullptr, nullptr, nullptr));
            S1_TRY(gemm_rows(m, s.ao, ly.o, s.delta, lengths, nseq, h, hq * hd));
        }
        S1_TRY(mlp_block(m, li, lengths, nseq, t));
        if (dump) S1_TRY(cs1_download(dump + li * (size_t)t * h * BF16, s.at(s.res), (size_t)t * h * BF16, st));
    }
    return 0;
}

// The device-side state of one token prefix, rows [0, len) of a prompt (PrefixState,
// model.rs:557-576): per full-attention layer the post-prep keys and the raw values, per Gated
// DeltaNet layer the float32 recurrent state and the last three pre-conv projection rows.
struct Prefix {
    Model* owner = nullptr;
    bool ready = false;
    int len = 0;
    std::vector<void*> k, v;         // [len, Hk * Dh] bf16 each
    std::vector<void*> state, tail;  // [H, 128, 128] float32; [3, gdn_in] bf16
    void* arena = nullptr;           // the one allocation they are carved from
    size_t bytes = 0;
};

constexpr int TAIL_ROWS = 3;  // conv kernel 4: a row needs the three rows before it

// The layer loop over a window that captures or continues a prefix (run_window,
// model.rs:1340-1638), for a pack of windows instead of one.
//   capture: one sequence, rows [0, len); the per-layer state is copied out as it is produced.
//   prefix:  nseq continuations of the same prefix, each at positions [len, len + c_i). The
//            reference runs one continuation per call; here the candidates of a request share
//            every GEMM and pointwise launch, which is what keeps the weights' one pass over
//            HBM amortised over all of them. A continuation owns lengths[i] = 3 + c_i packed
//            rows: three lead rows that receive the prefix's conv tail in every Gated DeltaNet
//            layer (so the convolution over the whole pack sees the right history; what the
//            lead rows themselves compute is never read), then its c_i token rows.
int run_window(Model* m, const int* lengths, int nseq, Prefix* capture, const Prefix* prefix) {
    const S1Config& c = m->cfg;
    const Scratch& s = m->s;
    void* st = m->stream;
    int t = 0;
    for (int i = 0; i < nseq; i++) t += lengths[i];
    const OverlapScope overlap(m, t);
    const int lead = prefix ? TAIL_ROWS : 0, qb = prefix ? prefix->len : 0;
    const int h = c.hidden, vd = m->value_dim(), hv = c.lin_v_heads;
    const int hq = c.heads, hd = c.head_dim;
    const int gdn_in = m->gdn_in_w(), attn_in = m->attn_in_w(), conv = m->conv_w();
    const size_t tail_bytes = (size_t)TAIL_ROWS * gdn_in * BF16;
    const float eps = c.eps;
    if (prefix) {
        // the lead rows skip the per-sequence operators; give what those would have written a value
        S1_TRY(s1_memset_async(s.at(s.lo), 0, (size_t)t * vd * BF16, st));
        S1_TRY(s1_memset_async(s.at(s.ao), 0, (size_t)t * hq * hd * BF16, st));
    }
    S1_OP(S1_FAMILY_NORM, 1, cs1_rms_norm(s.at(s.res), m->w(m->layers[0].input_norm), s.at(s.x), t, h, eps, st));
    size_t la = 0, fa = 0;
    for (size_t li = 0; li < m->layers.size(); li++) {
        const Layer& ly = m->layers[li];
        if (!ly.full) {
            S1_TRY(gemm(m, s.x, ly.in_proj, s.gdn_in, t, gdn_in, h));
            const size_t z = s.gdn_in + (size_t)conv * BF16;
            if (capture)
                S1_TRY(cs1_copy_dd(capture->tail[la], s.at(s.gdn_in + (size_t)(t - TAIL_ROWS) * gdn_in * BF16), tail_bytes,
                                   st));
            for (int first = 0, off = 0; prefix && first < nseq;) {  // the prefix's conv tail in front of every continuation
                const int n = std::min(nseq - first, PACK_SEQS);
                int row0[PACK_SEQS];
                for (int i = 0; i < n; i++) {
                    row0[i] = off;
                    off += lengths[first + i];
                }
                if (gdn_in % 8 == 0) {
                    S1_TRY(s1::spread_block(s.at(s.gdn_in), (size_t)gdn_in * BF16 / 16, row0, n, prefix->tail[la], tail_bytes / 16,
                                            static_cast<cudaStream_t>(st)));
                } else {
                    for (int i = 0; i < n; i++)
                        S1_TRY(cs1_copy_dd(s.at(s.gdn_in + (size_t)row0[i] * gdn_in * BF16), prefix->tail[la], tail_bytes, st));
                }
                first += n;
            }
            // one convolution over the pack: a continuation's first token row sees its lead rows
            S1_TRY(conv_gates(m, ly, 0, t));
            S1_TRY(delta_rule(m, lengths, nseq, lead, prefix ? prefix->state[la] : nullptr,
                              capture ? capture->state[la] : nullptr));
            S1_OP(S1_FAMILY_GATED_NORM, 1,
                  cs1_gated_rms_norm(s.at(s.lo), s.at(z), gdn_in, m->w(ly.norm), s.at(s.ln), t, hv, 128, eps, st));
            S1_TRY(gemm_rows(m, s.ln, ly.out, s.delta, lengths, nseq, h, vd));
            la++;
        } else {
            S1_TRY(gemm(m, s.x, ly.qkv, s.attn_in, t, attn_in, h));
            S1_TRY(attention_pack(m, ly, lengths, nseq, t, lead, qb, prefix ? prefix->k[fa] : nullptr,
                                  prefix ? prefix->v[fa] : nullptr, capture ? capture->k[fa] : nullptr,
                                  capture ? capture->v[fa] : nullptr));
            S1_TRY(gemm_rows(m, s.ao, ly.o, s.delta, lengths, nseq, h, hq * hd));
            fa++;
        }
        S1_TRY(mlp_block(m, li, lengths, nseq, t));
    }
    return 0;
}

// Replay a captured graph for this ordered length vector (model.rs:797-813, 862-897). A vector
// seen for the first time runs eagerly and is only remembered: ragged request sets rarely repeat
// a vector, and recording one costs a second host pass over the layer loop. When a remembered
// vector comes again the pass is recorded first and the recording launched (one host pass, no
// wait for the stream); if recording fails the pass runs eagerly and replay is switched off.
int run_or_replay(Model* m, const int* lengths, int nseq) {
    if (!m->graph_enabled) return run(m, lengths, nseq, nullptr);
    const std::vector<int> key(lengths, lengths + nseq);
    auto replay = [m](const Model::Recorded& g) {
        m->replays++;
        for (int f = 0; f < S1_FAMILIES; f++) m->launches[f] += g.kernels[f];
        return cs1_graph_launch(g.exec, m->stream);
    };
    for (auto& g : m->graphs)
        if (g.key == key) return replay(g);
    auto seen = std::find(m->seen_once.begin(), m->seen_once.end(), key);
    if (seen == m->seen_once.end()) {
        if ((int)m->seen_once.size() == GRAPH_CACHE) m->seen_once.pop_front();
        m->seen_once.push_back(key);
        return run(m, lengths, nseq, nullptr);
    }
    m->seen_once.erase(seen);
    Model::Recorded rec{key, nullptr, {}};
    void*& exec = rec.exec;
    long long before[S1_FAMILIES];
    memcpy(before, m->launches, sizeof(before));
    int rc = cs1_graph_begin(m->stream);
    if (rc == 0) {
        m->capturing = true;
        const int body = run(m, lengths, nseq, nullptr);
        m->capturing = false;
        for (int f = 0; f < S1_FAMILIES; f++) rec.kernels[f] = m->launches[f] - before[f];  // recorded, not launched
        memcpy(m->launches, before, sizeof(before));
        rc = cs1_graph_end(m->stream, &exec);
        if (rc == 0 && body != 0) {
            cs1_graph_destroy(exec);
            rc = body;
        }
    }
    if (rc != 0) {
        // nothing of the pass has run yet: run it eagerly and stop trying to record
        m->graph_enabled = false;
        clear_graphs(m);
        return run(m, lengths, nseq, nullptr);
    }
    if ((int)m->graphs.size() == GRAPH_CACHE) {
        cs1_graph_destroy(m->graphs.front().exec);
        m->graphs.pop_front();
    }
    m->graphs.push_back(rec);
    m->captures++;
    return replay(m->graphs.back());
}

int check_batch(const Model* m, const int* lengths, int nseq, long* total) {
    if (nseq <= 0 || !lengths) return S1_ERR_ARGUMENT;
    long t = 0;
    for (int i = 0; i < nseq; i++) {
        if (lengths[i] <= 0 || lengths[i] > m->cfg.max_positions) return S1_ERR_ARGUMENT;
        t += lengths[i];
    }
    if (t > 0x7fffffffL) return S1_ERR_ARGUMENT;
    *total = t;
    return 0;
}

// The end offsets of a pack, through a ring of pinned slots. A slot is rewritten only after the
// copy queued out of it ENDS_RING passes ago has run, so any number of passes may be queued
// without waiting for the stream.
int stage_ends(Model* m, const int* lengths, int nseq) {
    const size_t k = m->ends_slot++ % ENDS_RING;
    cudaStream_t st = static_cast<cudaStream_t>(m->stream);
    if (!m->ends_event[k]) {
        S1_TRY((int)cudaEventCreateWithFlags(&m->ends_event[k], cudaEventDisableTiming));
    } else {
        S1_TRY((int)cudaEventSynchronize(m->ends_event[k]));
    }
    int* slot = m->ends_host + k * m->s.cap;
    int end = 0;
    for (int i = 0; i < nseq; i++) {
        end += lengths[i];
        slot[i] = end;
    }
    S1_TRY((int)cudaMemcpyAsync(m->s.at(m->s.ends), slot, (size_t)nseq * sizeof(int), cudaMemcpyHostToDevice, st));
    return (int)cudaEventRecord(m->ends_event[k], st);
}

// Behind a pass: each prompt's last-token row gathered into `rows` (bf16 [nseq, hidden], device)
// and the three device error words copied into the scratch's status slot.
int finish_pass(Model* m, int nseq, void* rows) {
    const Scratch& s = m->s;
    cudaStream_t st = static_cast<cudaStream_t>(m->stream);
    S1_OP(S1_FAMILY_OTHER, 1,
          s1::gather_rows(s.at(s.x), reinterpret_cast<const int*>(s.at(s.ends)), rows, nseq, m->cfg.hidden, st));
    S1_OP(S1_FAMILY_OTHER, 1, s1::collect_status(reinterpret_cast<int*>(s.at(s.status)), st));
    return 0;
}

// Reads `bytes` of last rows (nullable dst) and the status slot back, waits for the stream, and
// turns a non-zero error word into CS1_ERR_DEVICE_CHECK (clearing the words so that the next
// pass starts clean): a bounded wait that gave up left rows that must not be used.
int read_back(Model* m, void* dst, const void* src, size_t bytes) {
    cudaStream_t st = static_cast<cudaStream_t>(m->stream);
    if (!m->status_host) S1_TRY((int)cudaHostAlloc(reinterpret_cast<void**>(&m->status_host), 4 * sizeof(int), cudaHostAllocDefault));
    if (dst && bytes) S1_TRY((int)cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, st));
    S1_TRY((int)cudaMemcpyAsync(m->status_host, m->s.at(m->s.status), 3 * sizeof(int), cudaMemcpyDeviceToHost, st));
    S1_TRY(cs1_stream_sync(m->stream));
    if (m->status_host[0] | m->status_host[1] | m->status_host[2]) {
        S1_TRY(s1::clear_status());
        return CS1_ERR_DEVICE_CHECK;
    }
    return 0;
}

}  // namespace

extern "C" {

int s1_model_create(const S1Config* cfg, int device, void** out) {
    if (!cfg || !out) return S1_ERR_ARGUMENT;
    S1_TRY(validate(*cfg));
    S1_TRY(cs1_set_device(device));
    Model* m = new Model();
    m->cfg = *cfg;
    m->full.assign(cfg->full_attention, cfg->full_attention + cfg->n_layers);
    m->cfg.full_attention = m->full.data();
    m->device = device;
    plan_arena(m);
    int rc = cs1_stream_create(&m->stream);
    if (rc == 0) rc = cs1_malloc(&m->arena, m->arena_bytes);
    if (rc == 0) {
        m->gemm = cs1_gemm_create(GEMM_WORKSPACE);
        if (!m->gemm) rc = CS1_ERR_GEMM_BASE + 1;
    }
    if (rc != 0) {
        s1_model_destroy(m);
        return rc;
    }
    const char* flag = getenv("CUA_S1_GRAPH");
    m->graph_enabled = flag && strcmp(flag, "1") == 0;
    *out = m;
    return 0;
}

void s1_model_destroy(void* model) {
    Model* m = static_cast<Model*>(model);
    if (!m) return;
    cs1_set_device(m->device);
    if (m->stream) cs1_stream_sync(m->stream);
    clear_graphs(m);
    if (m->gemm) cs1_gemm_destroy(m->gemm);
    if (m->s.buf) cs1_free(m->s.buf);
    if (m->arena) cs1_free(m->arena);
    if (m->ends_host) cudaFreeHost(m->ends_host);
    if (m->last_host) cudaFreeHost(m->last_host);
    if (m->status_host) cudaFreeHost(m->status_host);
    for (cudaEvent_t e : m->ends_event)
        if (e) cudaEventDestroy(e);
    for (cudaEvent_t e : m->events) cudaEventDestroy(e);
    if (m->stream) cs1_stream_destroy(m->stream);
    delete m;
}

int s1_model_set_tensor(void* model, const char* name, const void* host_bf16, size_t bytes) {
    Model* m = static_cast<Model*>(model);
    if (!m || !name || !host_bf16) return S1_ERR_ARGUMENT;
    auto it = m->named.find(name);
    if (it == m->named.end()) return S1_ERR_UNKNOWN_TENSOR;
    if (it->second.bytes != bytes) return S1_ERR_TENSOR_SIZE;
    S1_TRY(cs1_set_device(m->device));
    S1_TRY(cs1_upload(m->w(it->second), host_bf16, bytes, m->stream));
    it->second.filled = true;
    return 0;
}

int s1_model_tensor(void* model, const char* name, void** device_ptr, size_t* bytes) {
    Model* m = static_cast<Model*>(model);
    if (!m || !name) return S1_ERR_ARGUMENT;
    auto it = m->named.find(name);
    if (it == m->named.end()) return S1_ERR_UNKNOWN_TENSOR;
    if (device_ptr) *device_ptr = m->w(it->second);
    if (bytes) *bytes = it->second.bytes;
    return 0;
}

int s1_model_tensor_shape(void* model, const char* name, int* rank, uint64_t* shape8) {
    Model* m = static_cast<Model*>(model);
    if (!m || !name) return S1_ERR_ARGUMENT;
    auto it = m->named.find(name);
    if (it == m->named.end()) return S1_ERR_UNKNOWN_TENSOR;
    if (rank) *rank = it->second.rank;
    for (int i = 0; shape8 && i < it->second.rank; i++) shape8[i] = it->second.shape[i];
    return 0;
}

int s1_model_unfilled(void* model, char* name_out, size_t cap) {
    Model* m = static_cast<Model*>(model);
    if (!m) return -1;
    int n = 0;
    for (const auto& entry : m->order) {
        if (m->named[entry.first].filled) continue;
        if (n++ == 0 && name_out && cap) {
            const size_t len = std::min(cap - 1, entry.first.size());
            memcpy(name_out, entry.first.data(), len);
            name_out[len] = 0;
        }
    }
    return n;
}

int s1_model_init_random(void* model, uint64_t seed, float std) {
    Model* m = static_cast<Model*>(model);
    if (!m) return S1_ERR_ARGUMENT;
    S1_TRY(cs1_set_device(m->device));
    cudaStream_t st = static_cast<cudaStream_t>(m->stream);
    uint64_t index = 0;
    auto ends_with = [](const std::string& s, const char* tail) {
        const size_t n = strlen(tail);
        return s.size() >= n && s.compare(s.size() - n, n, tail) == 0;
    };
    for (auto& entry : m->order) {
        const std::string& name = entry.first;
        const Tensor& t = entry.second;
        const uint64_t sd = seed * 0x100000001b3ull + (++index) * 0x9e3779b97f4a7c15ull;
        const size_t n = t.bytes / BF16;
        int rc;
        if (ends_with(name, "linear_attn.A_log"))
            rc = s1::fill_bf16(m->w(t), n, sd, 0.f, logf(16.f), 1, st);
        else if (ends_with(name, "linear_attn.dt_bias"))
            rc = s1::fill_bf16(m->w(t), n, sd, 0.f, 0.1f, 0, st);
        else if (ends_with(name, "linear_attn.norm.weight"))
            rc = s1::fill_bf16(m->w(t), n, sd, 1.f, std, 0, st);
        else
            rc = s1::fill_bf16(m->w(t), n, sd, 0.f, std, 0, st);
        S1_TRY(rc);
    }
    for (auto& kv : m->named) kv.second.filled = true;
    return cs1_stream_sync(m->stream);
}

int s1_model_config(void* model, S1Config* out) {
    Model* m = static_cast<Model*>(model);
    if (!m || !out) return S1_ERR_ARGUMENT;
    *out = m->cfg;  // full_attention points into the model and lives as long as it
    return 0;
}

int s1_model_reserve(void* model, int tokens) {
    Model* m = static_cast<Model*>(model);
    if (!m || tokens <= 0) return S1_ERR_ARGUMENT;
    return prepare_scratch(m, (size_t)tokens);
}

size_t s1_model_weight_bytes(void* model) { return model ? static_cast<Model*>(model)->arena_bytes : 0; }
void* s1_model_stream(void* model) { return model ? static_cast<Model*>(model)->stream : nullptr; }

int s1_model_set_exact_packing(void* model, int on) {
    Model* m = static_cast<Model*>(model);
    if (!m) return S1_ERR_ARGUMENT;
    if (m->exact_packing != (on != 0)) clear_graphs(m);
    m->exact_packing = on != 0;
    return 0;
}

int s1_model_set_overlap_tokens(void* model, int tokens) {
    Model* m = static_cast<Model*>(model);
    if (!m) return S1_ERR_ARGUMENT;
    if (tokens < 0) tokens = -1;
    if (m->overlap_tokens != tokens) clear_graphs(m);
    m->overlap_tokens = tokens;
    return 0;
}

int s1_model_set_fused_mlp(void* model, int on) {
    Model* m = static_cast<Model*>(model);
    if (!m) return S1_ERR_ARGUMENT;
    if (m->fuse_swiglu != (on != 0)) clear_graphs(m);
    m->fuse_swiglu = on != 0;
    return 0;
}

int s1_model_enable_graphs(void* model, int on) {
    Model* m = static_cast<Model*>(model);
    if (!m) return S1_ERR_ARGUMENT;
    m->graph_enabled = on != 0;
    if (!on) clear_graphs(m);
    return 0;
}

int s1_model_graph_stats(void* model, int* replays, int* captures, int* enabled) {
    Model* m = static_cast<Model*>(model);
    if (!m) return S1_ERR_ARGUMENT;
    if (replays) *replays = m->replays;
    if (captures) *captures = m->captures;
    if (enabled) *enabled = m->graph_enabled ? 1 : 0;
    return 0;
}

int s1_model_forward_batch(void* model, const int32_t* ids, const int* lengths, int nseq, float* last_hidden,
                           void* layer_out) {
    Model* m = static_cast<Model*>(model);
    if (!m || !ids || !last_hidden) return S1_ERR_ARGUMENT;
    long total = 0;
    S1_TRY(check_batch(m, lengths, nseq, &total));
    for (long i = 0; i < total; i++)
        if (ids[i] < 0 || ids[i] >= m->cfg.vocab) return S1_ERR_ARGUMENT;
    S1_TRY(prepare_scratch(m, (size_t)total));
    const Scratch& s = m->s;
    const int h = m->cfg.hidden;
    S1_TRY(cs1_upload(s.at(s.ids), ids, (size_t)total * 4, m->stream));
    S1_TRY(stage_ends(m, lengths, nseq));
    S1_OP(S1_FAMILY_OTHER, 1,
          cs1_embed(reinterpret_cast<const int32_t*>(s.at(s.ids)), m->w(m->embed), s.at(s.res), (int)total, h,
                    m->stream));
    if (layer_out)
        S1_TRY(run(m, lengths, nseq, static_cast<char*>(layer_out)));
    else
        S1_TRY(run_or_replay(m, lengths, nseq));
    S1_TRY(finish_pass(m, nseq, s.at(s.last)));
    const size_t bytes = (size_t)nseq * h * BF16;
    if (m->last_host_bytes < bytes) {
        if (m->last_host) cudaFreeHost(m->last_host);
        m->last_host = nullptr;
        m->last_host_bytes = 0;
        S1_TRY((int)cudaHostAlloc(&m->last_host, bytes, cudaHostAllocDefault));
        m->last_host_bytes = bytes;
    }
    S1_TRY(read_back(m, m->last_host, s.at(s.last), bytes));
    const uint16_t* rows = static_cast<const uint16_t*>(m->last_host);
    for (size_t i = 0; i < (size_t)nseq * h; i++) last_hidden[i] = bf2f(rows[i]);
    return 0;
}

int s1_model_forward_device(void* model, const int32_t* ids_device, const int* lengths, int nseq, void** last_rows) {
    Model* m = static_cast<Model*>(model);
    if (!m || !ids_device) return S1_ERR_ARGUMENT;
    long total = 0;
    S1_TRY(check_batch(m, lengths, nseq, &total));
    S1_TRY(prepare_scratch(m, (size_t)total));
    const Scratch& s = m->s;
    const int h = m->cfg.hidden;
    S1_TRY(stage_ends(m, lengths, nseq));
    S1_OP(S1_FAMILY_OTHER, 1, cs1_embed(ids_device, m->w(m->embed), s.at(s.res), (int)total, h, m->stream));
    S1_TRY(run_or_replay(m, lengths, nseq));
    S1_TRY(finish_pass(m, nseq, s.at(s.last)));
    if (last_rows) *last_rows = s.at(s.last);
    return 0;
}

int s1_model_forward_queue(void* model, const int32_t* ids_host, const int* lengths, int nseq, void* rows_device) {
    Model* m = static_cast<Model*>(model);
    if (!m || !ids_host || !rows_device) return S1_ERR_ARGUMENT;
    long total = 0;
    S1_TRY(check_batch(m, lengths, nseq, &total));
    for (long i = 0; i < total; i++)
        if (ids_host[i] < 0 || ids_host[i] >= m->cfg.vocab) return S1_ERR_ARGUMENT;
    S1_TRY(prepare_scratch(m, (size_t)total));
    const Scratch& s = m->s;
    S1_TRY(s1_upload_async(s.at(s.ids), ids_host, (size_t)total * 4, m->stream));
    S1_TRY(stage_ends(m, lengths, nseq));
    S1_OP(S1_FAMILY_OTHER, 1,
          cs1_embed(reinterpret_cast<const int32_t*>(s.at(s.ids)), m->w(m->embed), s.at(s.res), (int)total,
                    m->cfg.hidden, m->stream));
    S1_TRY(run_or_replay(m, lengths, nseq));
    return finish_pass(m, nseq, rows_device);
}

int s1_model_read_rows(void* model, void* dst_host, const void* rows_device, size_t bytes) {
    Model* m = static_cast<Model*>(model);
    if (!m || (bytes && (!dst_host || !rows_device))) return S1_ERR_ARGUMENT;
    S1_TRY(cs1_set_device(m->device));
    if (!m->s.buf) return bytes ? S1_ERR_ARGUMENT : cs1_stream_sync(m->stream);
    return read_back(m, dst_host, rows_device, bytes);
}

// ---- prefix capture / continuation (alloc_prefix, forward_multimodal_capture / _continue,
// model.rs:954-1073, for text positions) ----

void s1_prefix_destroy(void* prefix) {
    Prefix* p = static_cast<Prefix*>(prefix);
    if (!p) return;
    if (p->owner) cs1_set_device(p->owner->device);
    if (p->arena) cs1_free(p->arena);
    delete p;
}

int s1_prefix_create(void* model, int len, void** out) {
    Model* m = static_cast<Model*>(model);
    if (!m || !out || len < 64 || len % 64 || len > m->cfg.max_positions) return S1_ERR_ARGUMENT;
    S1_TRY(cs1_set_device(m->device));
    Prefix* p = new Prefix();
    p->owner = m;
    p->len = len;
    const size_t kv = (size_t)len * m->cfg.kv_heads * m->cfg.head_dim * BF16;
    const size_t state = (size_t)m->cfg.lin_v_heads * 128 * 128 * F32, tail = (size_t)TAIL_ROWS * m->gdn_in_w() * BF16;
    // one allocation, carved at 256-byte boundaries (the reference allocates each buffer, model.rs:968-989)
    size_t at = 0;
    auto take = [&](std::vector<void*>& list, size_t bytes) {
        list.push_back(reinterpret_cast<void*>(at));
        at += (bytes + ALIGN - 1) / ALIGN * ALIGN;
    };
    for (const Layer& ly : m->layers) {
        if (ly.full) {
            take(p->k, kv);
            take(p->v, kv);
        } else {
            take(p->state, state);
            take(p->tail, tail);
        }
    }
    p->bytes = at;
    const int rc = cs1_malloc(&p->arena, at);
    if (rc != 0) {
        delete p;
        return rc;
    }
    for (auto* list : {&p->k, &p->v, &p->state, &p->tail})
        for (void*& b : *list) b = static_cast<char*>(p->arena) + reinterpret_cast<size_t>(b);
    *out = p;
    return 0;
}

size_t s1_prefix_bytes(void* prefix) { return prefix ? static_cast<Prefix*>(prefix)->bytes : 0; }
int s1_prefix_len(void* prefix) { return prefix ? static_cast<Prefix*>(prefix)->len : 0; }

int s1_model_prefix_capture(void* model, const int32_t* ids, int len, void* prefix) {
    Model* m = static_cast<Model*>(model);
    Prefix* p = static_cast<Prefix*>(prefix);
    if (!m || !ids || !p || p->owner != m || len != p->len) return S1_ERR_ARGUMENT;
    for (int i = 0; i < len; i++)
        if (ids[i] < 0 || ids[i] >= m->cfg.vocab) return S1_ERR_ARGUMENT;
    p->ready = false;
    S1_TRY(prepare_scratch(m, (size_t)len));
    const Scratch& s = m->s;
    S1_TRY(cs1_upload(s.at(s.ids), ids, (size_t)len * 4, m->stream));
    S1_OP(S1_FAMILY_OTHER, 1,
          cs1_embed(reinterpret_cast<const int32_t*>(s.at(s.ids)), m->w(m->embed), s.at(s.res), len, m->cfg.hidden,
                    m->stream));
    S1_TRY(run_window(m, &len, 1, p, nullptr));
    S1_OP(S1_FAMILY_OTHER, 1, s1::collect_status(reinterpret_cast<int*>(s.at(s.status)), static_cast<cudaStream_t>(m->stream)));
    S1_TRY(read_back(m, nullptr, nullptr, 0));
    p->ready = true;
    return 0;
}

int s1_model_forward_continue(void* model, const void* prefix, const int32_t* ids, const int* lengths, int nseq,
                              float* last_hidden) {
    Model* m = static_cast<Model*>(model);
    const Prefix* p = static_cast<const Prefix*>(prefix);
    if (!m || !p || p->owner != m || !p->ready || !ids || !last_hidden || nseq <= 0 || !lengths) return S1_ERR_ARGUMENT;
    long tokens = 0, longest = 0;
    for (int i = 0; i < nseq; i++) {
        if (lengths[i] <= 0 || (long)p->len + lengths[i] > m->cfg.max_positions) return S1_ERR_ARGUMENT;
        tokens += lengths[i];
        longest = std::max<long>(longest, lengths[i]);
    }
    for (long i = 0; i < tokens; i++)
        if (ids[i] < 0 || ids[i] >= m->cfg.vocab) return S1_ERR_ARGUMENT;
    // packed rows: three lead rows in front of every continuation (see run_window)
    const long rows = tokens + (long)TAIL_ROWS * nseq;
    if (rows > 0x7fffffffL) return S1_ERR_ARGUMENT;
    std::vector<int32_t> packed_ids;
    std::vector<int> packed_len(nseq);
    packed_ids.reserve(rows);
    long at = 0;
    for (int i = 0; i < nseq; i++) {
        packed_ids.insert(packed_ids.end(), TAIL_ROWS, ids[at]);
        packed_ids.insert(packed_ids.end(), ids + at, ids + at + lengths[i]);
        packed_len[i] = lengths[i] + TAIL_ROWS;
        at += lengths[i];
    }
    // the rotary tables are as long as the scratch: cover the last position too
    S1_TRY(prepare_scratch(m, (size_t)std::max<long>(rows, p->len + longest)));
    const Scratch& s = m->s;
    const int h = m->cfg.hidden;
    S1_TRY(cs1_upload(s.at(s.ids), packed_ids.data(), (size_t)rows * 4, m->stream));
    S1_TRY(stage_ends(m, packed_len.data(), nseq));
    S1_OP(S1_FAMILY_OTHER, 1,
          cs1_embed(reinterpret_cast<const int32_t*>(s.at(s.ids)), m->w(m->embed), s.at(s.res), (int)rows, h, m->stream));
    S1_TRY(run_window(m, packed_len.data(), nseq, nullptr, p));
    S1_TRY(finish_pass(m, nseq, s.at(s.last)));
    std::vector<uint16_t> out((size_t)nseq * h);
    S1_TRY(read_back(m, out.data(), s.at(s.last), out.size() * BF16));
    for (size_t i = 0; i < out.size(); i++) last_hidden[i] = bf2f(out[i]);
    return 0;
}

int s1_model_profile(void* model, int on) {
    Model* m = static_cast<Model*>(model);
    if (!m) return S1_ERR_ARGUMENT;
    m->profiling = on != 0;
    return 0;
}

int s1_model_profile_read(void* model, float* ms, long long* launches, long long* library_launches) {
    Model* m = static_cast<Model*>(model);
    if (!m) return S1_ERR_ARGUMENT;
    S1_TRY(cs1_set_device(m->device));
    S1_TRY(cs1_stream_sync(m->stream));
    if (ms) {
        for (int f = 0; f < S1_FAMILIES; f++) ms[f] = 0.f;
        for (const ProfRecord& r : m->prof) {
            float t = 0.f;
            if (cudaEventElapsedTime(&t, r.start, r.stop) == cudaSuccess) ms[r.family] += t;
        }
    }
    if (launches) memcpy(launches, m->launches, sizeof(m->launches));
    if (library_launches) *library_launches = m->library_launches;
    m->prof.clear();
    m->events_used = 0;
    memset(m->launches, 0, sizeof(m->launches));
    m->library_launches = 0;
    return 0;
}

int s1_model_sync(void* model) {
    Model* m = static_cast<Model*>(model);
    if (!m) return S1_ERR_ARGUMENT;
    S1_TRY(cs1_set_device(m->device));
    return cs1_stream_sync(m->stream);
}

int s1_head_logits(const float* weights, const float* bias, const float* last, int hidden, int n_classes,
                   float* logits) {
    if (!weights || !last || !logits || hidden <= 0 || n_classes < 0) return S1_ERR_ARGUMENT;
    int bad = 0;
    for (int o = 0; o < n_classes; o++) {
        double acc = 0.0;
        const float* w = weights + (size_t)o * hidden;
        for (int i = 0; i < hidden; i++) acc += (double)w[i] * (double)last[i];
        float v = (float)acc;
        if (bias) v += bias[o];
        logits[o] = v;
        if (!isfinite(v)) bad = 1;
    }
    return bad ? S1_ERR_NONFINITE : 0;
}

int s1_decide(const float* logits, int n, double temperature, double* probs) {
    if (!logits || n <= 0 || !(temperature > 0.0) || !isfinite(temperature)) return -1;
    float mx = -INFINITY;
    for (int i = 0; i < n; i++) {
        if (!isfinite(logits[i])) return -1;
        mx = std::max(mx, logits[i]);
    }
    std::vector<double> p(n);
    double total = 0.0;
    for (int i = 0; i < n; i++) {
        p[i] = exp(((double)logits[i] - (double)mx) / temperature);
        total += p[i];
    }
    int mode = 0;
    for (int i = 0; i < n; i++) {
        p[i] /= total;
        if (i > 0 && p[i] > p[mode]) mode = i;
    }
    if (probs) memcpy(probs, p.data(), sizeof(double) * n);
    return mode;
}

int s1_batch_ranges(const int* lengths, int n, int* starts) {
    const int MAX_SEQUENCES = 16;
    const long MAX_TOKENS = 4096;
    int groups = 0, start = 0;
    long tokens = 0;
    for (int index = 0; index < n; index++) {
        if (index > start && (index - start == MAX_SEQUENCES || tokens + lengths[index] > MAX_TOKENS)) {
            starts[groups++] = start;
            start = index;
            tokens = 0;
        }
        tokens += lengths[index];
    }
    if (start < n) starts[groups++] = start;
    return groups;
}

int s1_assign_requests(const int* lengths, int n, int n_ranks, double a, double b, int* rank_of) {
    return s1_assign_requests_weighted(lengths, n, n_ranks, a, b, nullptr, rank_of);
}

int s1_assign_requests_weighted(const int* lengths, int n, int n_ranks, double a, double b, const double* speed,
                                int* rank_of) {
    if (n < 0 || n_ranks <= 0 || (n > 0 && (!lengths || !rank_of))) return S1_ERR_ARGUMENT;
    for (int r = 0; speed && r < n_ranks; r++)
        if (!(speed[r] > 0.0) || !std::isfinite(speed[r])) return S1_ERR_ARGUMENT;
    std::vector<int> idx(n);
    std::iota(idx.begin(), idx.end(), 0);
    auto cost = [&](int i) { return a * lengths[i] + b * (double)lengths[i] * (double)lengths[i]; };
    std::stable_sort(idx.begin(), idx.end(), [&](int x, int y) { return cost(x) > cost(y); });
    std::vector<double> load(n_ranks, 0.0);
    // each request, longest first, goes where it would finish earliest (the first such rank);
    // with equal speeds that is the rank with the least load
    auto finish = [&](int r, double c) { return speed ? (load[r] + c) / speed[r] : load[r]; };
    for (int i : idx) {
        const double c = cost(i);
        int best = 0;
        for (int r = 1; r < n_ranks; r++)
            if (finish(r, c) < finish(best, c)) best = r;
        rank_of[i] = best;
        load[best] += c;
    }
    return 0;
}

}  // extern "C"
