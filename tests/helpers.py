"""Shared pieces of the parity tests: the seeded inputs of the reference's kernel tests and
bf16 comparisons. bf16 tensors are numpy uint16 bit patterns."""
import numpy as np

import oracle as O


def bf(x):
    return O.f32_to_bf16(np.asarray(x, np.float32))


def f32(x):
    return O.bf16_to_f32(x)


def ulp_diff(a, b):
    """Distance in bf16 steps between two bit-pattern arrays (same-sign finite values)."""
    a = np.asarray(a, np.uint16).astype(np.int32)
    b = np.asarray(b, np.uint16).astype(np.int32)
    # map sign-magnitude to a monotone integer line
    a = np.where(a & 0x8000, 0x8000 - a, a)
    b = np.where(b & 0x8000, 0x8000 - b, b)
    return np.abs(a - b)


def gdn_inputs(t, h, hk, decay_scale, qk_amp, d=128):
    """The input recipe of gated_delta_rule_matches_recurrent_reference
    (reference tests/qwen3_5/kernels.rs:556-572): q close to k, log decays in (-2, 0) * scale,
    learning rates in (0, 1)."""
    k = O.random_bf16(t * hk * d, 12, qk_amp)
    n = O.random_bf16(t * hk * d, 11, qk_amp)
    q = bf(np.float32(0.8) * f32(k) + np.float32(0.2) * f32(n))
    v = O.random_bf16(t * h * d, 13, 1.0)
    g = ((f32(O.random_bf16(t * h, 14, 1.0)) - np.float32(1.0)) * np.float32(decay_scale)).astype(np.float32)
    beta = bf(f32(O.random_bf16(t * h, 15, 0.5)) + np.float32(0.5))
    return q, k, v, g, beta


# (t, h, hk, decay_scale, qk_amp) of the reference test, kernels.rs:533-554
GDN_SHAPES = [
    (1, 4, 2, 1.0, 1.0), (16, 4, 2, 1.0, 1.0), (17, 4, 2, 1.0, 1.0), (32, 4, 2, 1.0, 1.0), (33, 4, 2, 1.0, 1.0),
    (63, 4, 2, 1.0, 1.0), (64, 4, 2, 1.0, 1.0), (65, 4, 2, 1.0, 1.0), (107, 4, 2, 1.0, 1.0), (127, 4, 2, 1.0, 1.0),
    (128, 4, 2, 1.0, 1.0), (129, 4, 2, 1.0, 1.0), (150, 4, 2, 1.0, 1.0), (107, 4, 2, 0.01, 1.0),
    (936, 4, 2, 0.01, 1.0), (936, 6, 2, 0.01, 1.0), (3399, 3, 1, 0.01, 1.0), (65, 4, 2, 0.01, 1e-9),
    (65, 4, 2, 0.01, 1e-18), (65, 4, 2, 0.01, 0.0),
]


def tiny_config(layer_types=("linear_attention", "linear_attention", "linear_attention", "full_attention"),
                head_dim=128, hidden=256, intermediate=512, heads=4, kv_heads=2, lin_k=2, lin_v=4, vocab=512):
    from system1_omni_b200.model import Config
    return Config(hidden=hidden, intermediate=intermediate, layer_types=list(layer_types), heads=heads,
                  kv_heads=kv_heads, head_dim=head_dim, rotary_half=head_dim // 8 if head_dim == 128 else 32,
                  lin_k_heads=lin_k, lin_v_heads=lin_v, vocab=vocab, eps=1e-6, rope_theta=1e7, max_positions=65536)


def random_weights(cfg, seed=0, std=0.02):
    """Seeded synthetic checkpoint: matrices and zero-centred norm weights N(0, std), gated norm
    weight 1 + N(0, std), A_log U(0, ln 16), dt_bias N(0, 0.1); bf16 bit patterns by name."""
    from system1_omni_b200.model import tensor_shapes
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith("linear_attn.A_log"):
            a = rng.uniform(0.0, np.log(16.0), shape)
        elif name.endswith("linear_attn.dt_bias"):
            a = rng.normal(0.0, 0.1, shape)
        elif name.endswith("linear_attn.norm.weight"):
            a = 1.0 + rng.normal(0.0, std, shape)
        elif name == "embed_tokens.weight":
            a = rng.normal(0.0, 1.0, shape)
        else:
            a = rng.normal(0.0, std, shape)
        out[name] = bf(a.astype(np.float32))
    return out
