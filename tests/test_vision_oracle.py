"""Known answers of the vision-tower oracle (oracle/vision.py): cases whose result follows from the
operator's definition (vision.cu:156-211 of the reference), checked on the CPU."""
import numpy as np

import oracle as O
from oracle import vision as V
from helpers import bf, f32


def test_layer_norm_of_a_constant_row_is_the_bias():
    x = bf(np.full((3, 1024), 2.5, np.float32))
    w = bf(np.random.default_rng(0).normal(1, 0.1, 1024).astype(np.float32))
    b = bf(np.random.default_rng(1).normal(0, 0.1, 1024).astype(np.float32))
    assert np.array_equal(V.norm(x, w, b), np.tile(b, (3, 1)))


def test_layer_norm_standardises():
    rng = np.random.default_rng(2)
    x = bf(rng.normal(3, 2, (5, 1024)).astype(np.float32))
    y = f32(V.norm(x, bf(np.ones(1024, np.float32)), bf(np.zeros(1024, np.float32))))
    assert np.abs(y.mean(-1)).max() < 1e-2 and np.abs(y.std(-1) - 1).max() < 1e-2


def test_rope_identity_and_quarter_turn():
    rng = np.random.default_rng(3)
    qkv = bf(rng.normal(0, 1, (4, 3072)).astype(np.float32))
    one, zero = np.ones((4, 32), np.float32), np.zeros((4, 32), np.float32)
    q, k = V.rope(qkv, one, zero)
    assert np.array_equal(q, qkv[:, :1024]) and np.array_equal(k, qkv[:, 1024:2048])
    q, _ = V.rope(qkv, zero, one)           # cos 0, sin 1: (a, b) -> (-b, a) within each head
    a = f32(qkv[:, :1024]).reshape(4, 16, 64)
    want = np.concatenate([-a[..., 32:], a[..., :32]], -1).reshape(4, 1024)
    assert np.array_equal(f32(q), want)


def test_position_rounds_the_embedding_before_the_add():
    table = bf(np.zeros((2304, 1024), np.float32))
    table[7] = bf(np.full(1024, 1.0, np.float32))
    table[9] = bf(np.full(1024, 2.0 ** -9, np.float32))
    idx = np.array([[7, 9, 0, 0]], np.int32)
    wts = np.array([[1.0, 1.0, 0.0, 0.0]], np.float32)
    x = bf(np.zeros((1, 1024), np.float32))
    # 1 + 2^-9 is not a bf16 value: the position term rounds to 1.0 first
    assert np.all(f32(V.position(x, table, idx, wts)) == 1.0)


def test_gelu_bias_add_lora():
    x = bf(np.array([-3.0, -1.0, 0.0, 0.5, 2.0, 8.0], np.float32))
    g = f32(V.gelu(x, True))
    assert g[2] == 0 and abs(g[4] - 1.9545) < 1e-2 and abs(g[0] + 0.00405) < 1e-3 and g[5] == 8.0
    assert np.abs(f32(V.gelu(x, False)) - g).max() < 5e-3
    b = bf(np.array([1.0, -1.0], np.float32))
    assert np.array_equal(f32(V.bias(x, b)), f32(x) + np.array([1, -1, 1, -1, 1, -1], np.float32))
    assert np.array_equal(V.add(x, x), bf(2 * f32(x)))
    assert np.array_equal(V.lora_add(x, np.ones(6, np.float32), 0.5), bf(f32(x) + 0.5))


def test_attention_with_one_key_returns_its_value():
    rng = np.random.default_rng(4)
    q, k, v = (bf(rng.normal(0, 1, (1, 1024)).astype(np.float32)) for _ in range(3))
    assert np.allclose(V.attention_f64(q, k, v), f32(v))
    # uniform scores: the mean of the values
    q0 = bf(np.zeros((3, 1024), np.float32))
    k3, v3 = (bf(rng.normal(0, 1, (3, 1024)).astype(np.float32)) for _ in range(2))
    assert np.allclose(V.attention_f64(q0, k3, v3), np.tile(f32(v3).astype(np.float64).mean(0), (3, 1)))
