"""ctypes loader for the CPU oracle (oracle/oracle.cpp). TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg import this
module; the product (the CUDA library and its host executor) never does. bf16 tensors are
numpy uint16 arrays holding the bit patterns.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

u16p = C.POINTER(C.c_uint16)
f32p = C.POINTER(C.c_float)
f64p = C.POINTER(C.c_double)
i32p = C.POINTER(C.c_int32)
i64p = C.POINTER(C.c_int64)


def build():
    """Compile liboracle.so if it is missing or older than its source."""
    so, src = os.path.join(_HERE, "liboracle.so"), os.path.join(_HERE, "oracle.cpp")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True, capture_output=True)
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(build())
        _LIB.orc_head_score.restype = C.c_int
        _LIB.orc_letter_logits.restype = C.c_int
        _LIB.orc_batch_ranges.restype = C.c_int
        _LIB.orc_decide.restype = C.c_int
        _LIB.orc_threads.restype = C.c_int
    return _LIB


def _p(a, t):
    return None if a is None else a.ctypes.data_as(t)


def _u16(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint16, a.dtype
    return a


def threads():
    return lib().orc_threads()


def set_threads(n):
    lib().orc_set_threads(int(n))


def f32_to_bf16(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_bf16(_p(x, f32p), _p(out, u16p), C.c_size_t(x.size))
    return out


def bf16_to_f32(x):
    x = _u16(x)
    out = np.empty(x.shape, np.float32)
    lib().orc_bf16_to_f32(_p(x, u16p), _p(out, f32p), C.c_size_t(x.size))
    return out


def random_bf16(n, seed, amp):
    out = np.empty(int(n), np.uint16)
    lib().orc_random_bf16(_p(out, u16p), C.c_size_t(int(n)), C.c_uint64(seed), C.c_float(amp))
    return out


def embed(ids, table):
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    table = _u16(table)
    D = table.shape[1]
    out = np.empty((ids.size, D), np.uint16)
    lib().orc_embed(_p(ids, i32p), _p(table, u16p), _p(out, u16p), ids.size, D)
    return out


def rms_norm(x, w, eps):
    x, w = _u16(x), _u16(w)
    rows, D = x.shape
    out = np.empty_like(x)
    lib().orc_rms_norm(_p(x, u16p), _p(w, u16p), _p(out, u16p), rows, D, C.c_float(eps))
    return out


def add_rms_norm(residual, delta, w, eps):
    """Returns (new residual, normed)."""
    res = _u16(residual).copy()
    delta, w = _u16(delta), _u16(w)
    rows, D = res.shape
    out = np.empty_like(res)
    lib().orc_add_rms_norm(_p(res, u16p), _p(delta, u16p), _p(w, u16p), _p(out, u16p), rows, D, C.c_float(eps))
    return res, out


def gated_rms_norm(x, z, ldz, w, T, H, eps, D=128):
    x, z, w = _u16(x), _u16(z), _u16(w)
    out = np.empty((T, H * D), np.uint16)
    lib().orc_gated_rms_norm(_p(x, u16p), _p(z, u16p), ldz, _p(w, u16p), _p(out, u16p), T, H, D, C.c_float(eps))
    return out


def gdn_conv(qkv, ld, w, T, key_dim, value_dim):
    qkv, w = _u16(qkv), _u16(w)
    q = np.empty((T, key_dim), np.uint16)
    k = np.empty((T, key_dim), np.uint16)
    v = np.empty((T, value_dim), np.uint16)
    lib().orc_gdn_conv(_p(qkv, u16p), ld, _p(w, u16p), _p(q, u16p), _p(k, u16p), _p(v, u16p), T, key_dim, value_dim)
    return q, k, v


def gdn_gates(b, a, ld, A_log, dt_bias, T, H):
    b, a, A_log, dt_bias = _u16(b), _u16(a), _u16(A_log), _u16(dt_bias)
    beta = np.empty((T, H), np.uint16)
    g = np.empty((T, H), np.float32)
    lib().orc_gdn_gates(_p(b, u16p), _p(a, u16p), ld, _p(A_log, u16p), _p(dt_bias, u16p), _p(beta, u16p),
                        _p(g, f32p), T, H)
    return beta, g


def silu_mul(gate_up, ld, T, I):
    gate_up = _u16(gate_up)
    out = np.empty((T, I), np.uint16)
    lib().orc_silu_mul(_p(gate_up, u16p), ld, _p(out, u16p), T, I)
    return out


def sigmoid_gate(x, gate):
    x = _u16(x).copy()
    gate = _u16(gate)
    lib().orc_sigmoid_gate(_p(x, u16p), _p(gate, u16p), C.c_size_t(x.size))
    return x


def rotary_tables(positions, half, theta):
    positions = np.ascontiguousarray(positions, dtype=np.int64)
    T = positions.size
    cos = np.empty((T, half), np.uint16)
    sin = np.empty((T, half), np.uint16)
    lib().orc_rotary_tables(_p(positions, i64p), T, half, C.c_double(theta), _p(cos, u16p), _p(sin, u16p))
    return cos, sin


def attn_prep(qg, kr_offset, ld, qw, kw, cos, sin, T, Hq, Hk, Dh, half, eps):
    """qg is the whole projection buffer [T, ld]; k rows start kr_offset elements into each row."""
    qg = _u16(qg)
    q = np.empty((T, Hq, Dh), np.uint16)
    gate = np.empty((T, Hq * Dh), np.uint16)
    k = np.empty((T, Hk, Dh), np.uint16)
    base = qg.ctypes.data
    lib().orc_attn_prep(C.cast(base, u16p), C.cast(base + 2 * kr_offset, u16p), ld, _p(_u16(qw), u16p),
                        _p(_u16(kw), u16p), _p(_u16(cos), u16p), _p(_u16(sin), u16p), _p(q, u16p), _p(gate, u16p),
                        _p(k, u16p), T, Hq, Hk, Dh, half, C.c_float(eps))
    return q, gate, k


def gemm(x, w, ldy=None):
    x, w = _u16(x), _u16(w)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K
    ldy = ldy or N
    y = np.zeros((M, ldy), np.uint16)
    lib().orc_gemm(_p(x, u16p), _p(w, u16p), _p(y, u16p), M, N, K, ldy)
    return y


def gdn_recurrent_f64(q, k, v, g, beta, T, H, HK, D=128, s_in=None, want_state=False):
    q, k, v, beta = _u16(q), _u16(k), _u16(v), _u16(beta)
    g = np.ascontiguousarray(g, dtype=np.float32)
    out = np.zeros((T, H, D), np.float64)
    s_out = np.zeros((H, D, D), np.float64) if want_state else None
    if s_in is not None:
        s_in = np.ascontiguousarray(s_in, dtype=np.float64)
    lib().orc_gdn_recurrent_f64(_p(q, u16p), _p(k, u16p), _p(v, u16p), _p(g, f32p), _p(beta, u16p), _p(out, f64p),
                                T, H, HK, D, _p(s_in, f64p), _p(s_out, f64p))
    return (out, s_out) if want_state else out


def gdn_chunked(q, k, v, g, beta, T, H, HK, scale, s_in=None, want_state=False):
    q, k, v, beta = _u16(q), _u16(k), _u16(v), _u16(beta)
    g = np.ascontiguousarray(g, dtype=np.float32)
    o = np.zeros((T, H, 128), np.uint16)
    s_out = np.zeros((H, 128, 128), np.float32) if want_state else None
    if s_in is not None:
        s_in = np.ascontiguousarray(s_in, dtype=np.float32)
    lib().orc_gdn_chunked(_p(q, u16p), _p(k, u16p), _p(v, u16p), _p(g, f32p), _p(beta, u16p), _p(o, u16p), T, H, HK,
                          C.c_float(scale), _p(s_in, f32p), _p(s_out, f32p))
    return (o, s_out) if want_state else o


def attention_f64(q, k, v_buf, v_offset, ldv, T, Hq, Hk, Dh, scale, q_base=0, row_step=1):
    """v_buf is a flat bf16 buffer; V rows start v_offset elements in, with row stride ldv.
    row_step > 1 computes only every row_step-th row and the last one (others stay zero)."""
    q, k, v_buf = _u16(q), _u16(k), _u16(v_buf)
    out = np.zeros((T, Hq, Dh), np.float64)
    lib().orc_attention_f64(_p(q, u16p), _p(k, u16p), C.cast(v_buf.ctypes.data + 2 * v_offset, u16p), ldv,
                            _p(out, f64p), T, Hq, Hk, Dh, C.c_double(scale), q_base, row_step)
    return out


def attention(q, k, v_buf, v_offset, ldv, gate, T, Hq, Hk, Dh, scale, q_base=0):
    q, k, v_buf = _u16(q), _u16(k), _u16(v_buf)
    out = np.zeros((T, Hq, Dh), np.uint16)
    gate = None if gate is None else _u16(gate)
    lib().orc_attention(_p(q, u16p), _p(k, u16p), C.cast(v_buf.ctypes.data + 2 * v_offset, u16p), ldv,
                        _p(gate, u16p), _p(out, u16p), T, Hq, Hk, Dh, C.c_float(scale), q_base)
    return out


def head_score(weights, last, bias):
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    last = np.ascontiguousarray(last, dtype=np.float32)
    s = C.c_float(0)
    bad = lib().orc_head_score(_p(weights, f32p), _p(last, f32p), weights.size, C.c_float(bias), C.byref(s))
    if bad:
        raise ValueError("non-finite decision score")
    return np.float32(s.value)


def letter_logits(letters, last, n_options):
    letters = np.ascontiguousarray(letters, dtype=np.float32)
    last = np.ascontiguousarray(last, dtype=np.float32)
    out = np.zeros(n_options, np.float32)
    bad = lib().orc_letter_logits(_p(letters, f32p), _p(last, f32p), last.size, n_options, _p(out, f32p))
    if bad:
        raise ValueError("non-finite probabilities")
    return out


def batch_ranges(lengths):
    lengths = np.ascontiguousarray(lengths, dtype=np.int32)
    starts = np.zeros(max(1, lengths.size), np.int32)
    n = lib().orc_batch_ranges(_p(lengths, i32p), lengths.size, _p(starts, i32p))
    edges = list(starts[:n]) + [lengths.size]
    return [(int(edges[i]), int(edges[i + 1])) for i in range(n)]


def decide(logits, temperature=1.0):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    probs = np.zeros(logits.size, np.float64)
    mode = lib().orc_decide(_p(logits, f32p), logits.size, C.c_double(temperature), _p(probs, f64p))
    return mode, probs


class _Layer(C.Structure):
    _fields_ = [("full_attention", C.c_int)] + [(n, C.c_void_p) for n in (
        "input_norm", "post_norm", "gate_up", "down", "in_proj", "conv", "a_log", "dt_bias", "norm", "out_proj",
        "qkv", "o_proj", "q_norm", "k_norm")]


class _Model(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("hidden", "intermediate", "n_layers", "heads", "kv_heads", "head_dim",
                                        "rotary_half", "lin_k_heads", "lin_v_heads", "vocab")] + [
        ("eps", C.c_float), ("rope_theta", C.c_double), ("embed", C.c_void_p), ("final_norm", C.c_void_p),
        ("layers", C.POINTER(_Layer))]


def forward(cfg, weights, ids, lengths, max_layers=None, want_layers=False, x_in=None):
    """Prefill a pack of sequences on the CPU.

    cfg: dict with hidden, intermediate, layer_types (list of 'linear_attention'/'full_attention'),
    heads, kv_heads, head_dim, rotary_half, lin_k_heads, lin_v_heads, vocab, eps, rope_theta.
    weights: dict name -> uint16 array using checkpoint tensor names without the model prefix
    (e.g. 'layers.0.linear_attn.in_proj_qkv.weight', 'embed_tokens.weight', 'norm.weight').
    Returns last hidden states float32 [nseq, hidden] (and the per-layer residual streams).
    """
    keep = []

    def w(name):
        a = _u16(weights[name])
        keep.append(a)
        return a.ctypes.data

    def stacked(names):
        a = np.ascontiguousarray(np.concatenate([_u16(weights[n]).reshape(weights[n].shape[0], -1) for n in names], 0))
        keep.append(a)
        return a.ctypes.data

    L = len(cfg["layer_types"])
    layers = (_Layer * L)()
    for i, kind in enumerate(cfg["layer_types"]):
        p = f"layers.{i}."
        ly = layers[i]
        ly.full_attention = int(kind == "full_attention")
        ly.input_norm = w(p + "input_layernorm.weight")
        ly.post_norm = w(p + "post_attention_layernorm.weight")
        ly.gate_up = stacked([p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight"])
        ly.down = w(p + "mlp.down_proj.weight")
        if ly.full_attention:
            ly.qkv = stacked([p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight",
                              p + "self_attn.v_proj.weight"])
            ly.o_proj = w(p + "self_attn.o_proj.weight")
            ly.q_norm = w(p + "self_attn.q_norm.weight")
            ly.k_norm = w(p + "self_attn.k_norm.weight")
        else:
            ly.in_proj = stacked([p + "linear_attn.in_proj_qkv.weight", p + "linear_attn.in_proj_z.weight",
                                  p + "linear_attn.in_proj_b.weight", p + "linear_attn.in_proj_a.weight"])
            ly.conv = w(p + "linear_attn.conv1d.weight")
            ly.a_log = w(p + "linear_attn.A_log")
            ly.dt_bias = w(p + "linear_attn.dt_bias")
            ly.norm = w(p + "linear_attn.norm.weight")
            ly.out_proj = w(p + "linear_attn.out_proj.weight")
    m = _Model()
    for n in ("hidden", "intermediate", "heads", "kv_heads", "head_dim", "rotary_half", "lin_k_heads",
              "lin_v_heads", "vocab"):
        setattr(m, n, int(cfg[n]))
    m.n_layers = L
    m.eps = float(cfg["eps"])
    m.rope_theta = float(cfg["rope_theta"])
    m.embed = w("embed_tokens.weight")
    m.final_norm = w("norm.weight")
    m.layers = layers
    lengths = np.ascontiguousarray(lengths, dtype=np.int32)
    T = int(lengths.sum())
    ids_a = None if ids is None else np.ascontiguousarray(ids, dtype=np.int32)
    x_a = None if x_in is None else _u16(x_in)
    nl = L if max_layers is None else min(L, max_layers)
    last = np.zeros((lengths.size, m.hidden), np.float32)
    layer_out = np.zeros((nl, T, m.hidden), np.uint16) if want_layers else None
    lib().orc_forward(C.byref(m), _p(ids_a, i32p), _p(x_a, u16p), _p(lengths, i32p), lengths.size, nl,
                      _p(last, f32p), _p(layer_out, u16p))
    return (last, layer_out) if want_layers else last
