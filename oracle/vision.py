"""CPU restatement (numpy) of the vision-tower operators of the reference's CUDA backend
(src/backends/cuda/qwen3_5/vision.cu, gemm.cu:137-163): test infrastructure, never on a product path.

bf16 tensors are uint16 bit patterns. float32 arithmetic uses numpy's float32 operations, which round
each multiply and each add once (no fused multiply-add), as the reference spells out with
__fmul_rn / __fadd_rn where the order matters. Parity is pinned by running the reference's own
library beside this one on the GPU (tests/test_vision_gpu.py); the reference has no kernel-level
test vectors for these operators.
"""
import math

import numpy as np

from . import bf16_to_f32, f32_to_bf16

HIDDEN = 1024      # 16 heads of 64 (ops.h:125)
HEADS, HEAD_DIM = 16, 64


def _rbf(x):
    return bf16_to_f32(f32_to_bf16(np.asarray(x, np.float32)))


def norm(x, w, b):
    """LayerNorm, eps 1e-6 (vision.cu:156-167): float32 mean and variance in two passes,
    y = bf16((x - mean) * inv * w + b). Sums are taken in float64 here (the kernel's order is its own)."""
    xf = bf16_to_f32(x).astype(np.float64)
    mean = np.float32(1) * (xf.sum(-1, keepdims=True) / xf.shape[-1]).astype(np.float32)
    a = bf16_to_f32(x) - mean
    var = ((a.astype(np.float64) ** 2).sum(-1, keepdims=True) / xf.shape[-1]).astype(np.float32)
    inv = (1.0 / np.sqrt(var.astype(np.float64) + 1e-6)).astype(np.float32)
    return f32_to_bf16(a * inv * bf16_to_f32(w) + bf16_to_f32(b))


def position(x, table, indices, weights):
    """x [n, 1024] += bf16(sum_j table[indices[:, j]] * weights[:, j]) with separate float32 multiplies and
    adds in j order, the position term rounded to bf16 before the add (vision.cu:168-176)."""
    t = bf16_to_f32(table)
    pos = np.zeros(x.shape, np.float32)
    for j in range(4):
        pos = pos + t[indices[:, j]] * weights[:, j:j + 1].astype(np.float32)
    return f32_to_bf16(bf16_to_f32(x) + _rbf(pos))


def rope(qkv, cos, sin):
    """q, k [n, 1024] from the fused projection [n, 3072] (vision.cu:177-187): per head of 64,
    y[d] = bf16(x[d] * c + sign * x[partner] * s), partner = d +/- 32, sign -1 for d < 32; cos / sin
    [n, 32] float32 indexed by d % 32; both products are rounded to float32 before the add."""
    n = qkv.shape[0]
    x = bf16_to_f32(qkv).reshape(n, 3, HEADS, HEAD_DIM)
    c = np.concatenate([cos, cos], -1).astype(np.float32)[:, None, :]
    s = np.concatenate([sin, sin], -1).astype(np.float32)[:, None, :]
    out = []
    for which in (0, 1):
        a = x[:, which]
        partner = np.concatenate([-a[..., 32:], a[..., :32]], -1)
        out.append(f32_to_bf16((a * c + partner * s).reshape(n, HIDDEN)))
    return out[0], out[1]


def gelu(x, exact):
    """In place in the reference (vision.cu:188-195): 0.5 a (1 + erff(a / sqrt 2)), or the tanh
    approximation, in float32: for a below about -5.9 the float32 erf is exactly -1 and the result is
    a zero, where wider arithmetic would give a denormal-sized negative number."""
    a = bf16_to_f32(x)
    if exact:
        arg = (a * np.float32(0.7071067811865475244)).astype(np.float64)
        inner = np.vectorize(math.erf)(arg).astype(np.float32)
    else:
        cube = a * a * a
        arg = (np.float32(0.7978845608028654) * (a + np.float32(0.044715) * cube)).astype(np.float64)
        inner = np.tanh(arg).astype(np.float32)
    return f32_to_bf16(np.float32(0.5) * a * (np.float32(1) + inner))


def add(x, delta):
    return f32_to_bf16(bf16_to_f32(x) + bf16_to_f32(delta))          # vision.cu:196-199


def bias(x, b):
    flat = bf16_to_f32(x).ravel()
    return f32_to_bf16(flat + bf16_to_f32(b)[np.arange(flat.size) % b.size]).reshape(x.shape)   # vision.cu:200-203


def lora_add(x, delta, scale):
    prod = np.float32(scale) * np.asarray(delta, np.float32)
    return f32_to_bf16(bf16_to_f32(x) + prod)                        # vision.cu:208-211


def attention_f64(q, k, v):
    """Every query attends to all n keys; 16 heads of 64, scale 1/8 (vision.cu:229-235). float64."""
    n = q.shape[0]
    qf = bf16_to_f32(q).astype(np.float64).reshape(n, HEADS, HEAD_DIM)
    kf = bf16_to_f32(k).astype(np.float64).reshape(n, HEADS, HEAD_DIM)
    vf = bf16_to_f32(v).astype(np.float64).reshape(n, HEADS, HEAD_DIM)
    s = np.einsum("qhd,khd->hqk", qf, kf) * 0.125
    s -= s.max(-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(-1, keepdims=True)
    return np.einsum("hqk,khd->qhd", p, vf).reshape(n, HIDDEN)


def linear_f64(x, w, b):
    """y = x w^T + bias before the one bf16 rounding (gemm.cu:137-151). float64, unrounded."""
    return bf16_to_f32(x).astype(np.float64) @ bf16_to_f32(w).astype(np.float64).T + bf16_to_f32(b).astype(np.float64)
