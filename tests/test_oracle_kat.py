"""Pins the CPU oracle against everything the reference holds for this path that can be
checked without a GPU: its numeric known-answer tests and the figures its own kernel test
run recorded. Citations are file:line in the reference repository."""
import json
import os

import numpy as np
import pytest

import oracle as O
from helpers import GDN_SHAPES, bf, f32, gdn_inputs

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_scalar_head_preserves_accumulation_rounding_and_bias_order():
    # tests/open_jev/head.rs:5-18
    assert O.head_score([16_777_216.0, 1.0, -16_777_216.0], [1.0, 1.0, 1.0], 0.25) == 1.25
    assert O.head_score([16_777_216.0, 1.0], [1.0, 1.0], -16_777_216.0) == 0.0


def test_scalar_head_rejects_nonfinite_scores():
    # tests/open_jev/head.rs:21-29
    with pytest.raises(ValueError):
        O.head_score([np.finfo(np.float32).max], [2.0], 0.0)
    with pytest.raises(ValueError):
        O.head_score([np.finfo(np.float32).max], [np.nan], 0.0)


def test_letter_head_fp64_accumulation_and_fp32_readout():
    # tests/cua_s1/head.rs:4-23: unused letter rows must not be read
    letters = [16_777_216.0, 1.0, -16_777_216.0, 16_777_216.0, 1.0, 0.0, np.nan, np.nan, np.nan]
    assert list(O.letter_logits(letters, [1.0, 1.0, 1.0], 2)) == [1.0, 16_777_216.0]
    assert list(O.letter_logits(letters, [1.0, 1.0, 1.0], 1)) == [1.0]
    with pytest.raises(ValueError):
        O.letter_logits([np.finfo(np.float32).max], [2.0], 1)
    with pytest.raises(ValueError):
        O.letter_logits([np.nan], [1.0], 1)


def test_batching_keeps_all_candidates_across_limits():
    # tests/open_jev/batching.rs:4-17
    lengths = [2048, 2048, 1, 5000, 3] + [4] * 17
    got = O.batch_ranges(lengths)
    assert got == [(0, 2), (2, 3), (3, 4), (4, 20), (20, 22)]
    assert [i for a, b in got for i in range(a, b)] == list(range(len(lengths)))


def test_decision_first_maximum_wins_ties():
    # contract.rs:236-247
    mode, probs = O.decide([1.0, 3.0, 3.0, 0.5], 1.0)
    assert mode == 1 and abs(probs.sum() - 1.0) < 1e-12
    mode, probs = O.decide([0.0, 0.0], 2.0)
    assert mode == 0 and probs[0] == probs[1] == 0.5


def test_generator_matches_its_definition():
    # kernels.rs:25-36 restated independently in Python integers
    n, seed, amp = 64, 12, 1.0
    x = (seed * 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF | 1
    want = []
    for _ in range(n):
        x ^= (x << 13) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 7
        x ^= (x << 17) & 0xFFFFFFFFFFFFFFFF
        want.append((np.float32(x >> 40) / np.float32(1 << 24) * np.float32(2.0) - np.float32(1.0)) * np.float32(amp))
    assert np.array_equal(O.random_bf16(n, seed, amp), bf(np.array(want, np.float32)))


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -1.00390625, 3.4e38, np.inf], np.float32)
    got = f32(bf(x))
    assert list(got[:4]) == [1.0, 1.0, 1.015625, -1.0]
    assert np.isinf(got[4]) and np.isinf(got[5])


@pytest.mark.parametrize("case", json.load(open(os.path.join(GOLDEN, "reference_kernel_log.json")))["gated_delta"],
                         ids=lambda c: f"t{c['t']}h{c['h']}s{c['decay_scale']}a{c['qk_amp']}")
def test_float64_delta_rule_reproduces_the_reference_log(case):
    """The reference's GPU test printed max|reference| of its float64 oracle for each seeded
    shape (3 significant digits). The restated oracle must give the same figure, and the
    chunked float32 restatement must sit as close to it as the reference's kernel did."""
    t, h, hk = case["t"], case["h"], case["hk"]
    if t > 1000:
        pytest.skip("covered by the slow variant below")
    q, k, v, g, beta = gdn_inputs(t, h, hk, case["decay_scale"], case["qk_amp"])
    ref = O.gdn_recurrent_f64(q, k, v, g, beta, t, h, hk)
    scale = np.abs(ref).max()
    assert scale == pytest.approx(case["max_ref"], rel=6e-3, abs=0.0)
    chunked = f32(O.gdn_chunked(q, k, v, g, beta, t, h, hk, 128 ** -0.5)).astype(np.float64)
    diff = np.abs(chunked - ref).max()
    assert diff <= 2e-2 * scale                       # the reference's gate, kernels.rs:620
    if case["diff"] > 0:
        assert diff == pytest.approx(case["diff"], rel=0.25)   # same rounding points, same error


def test_float64_delta_rule_long_shape():
    case = [c for c in json.load(open(os.path.join(GOLDEN, "reference_kernel_log.json")))["gated_delta"]
            if c["t"] == 3399][0]
    q, k, v, g, beta = gdn_inputs(3399, 3, 1, 0.01, 1.0)
    ref = O.gdn_recurrent_f64(q, k, v, g, beta, 3399, 3, 1)
    assert np.abs(ref).max() == pytest.approx(case["max_ref"], rel=6e-3)
    chunked = f32(O.gdn_chunked(q, k, v, g, beta, 3399, 3, 1, 128 ** -0.5)).astype(np.float64)
    assert np.abs(chunked - ref).max() == pytest.approx(case["diff"], rel=0.25)


def test_gdn_shapes_table_matches_the_log():
    log = json.load(open(os.path.join(GOLDEN, "reference_kernel_log.json")))["gated_delta"]
    assert [(c["t"], c["h"], c["hk"], c["decay_scale"], c["qk_amp"]) for c in log] == GDN_SHAPES


def test_chunked_state_continuation_is_bit_exact_at_chunk_boundaries():
    # the contract of cs1_gdn_prefill_x (ops.h:80-87), on the CPU restatement
    t, h, hk = 200, 4, 2
    q, k, v, g, beta = gdn_inputs(t, h, hk, 1.0, 1.0)
    full, s_full = O.gdn_chunked(q, k, v, g, beta, t, h, hk, 128 ** -0.5, want_state=True)
    cut = 128
    qa, ka = q.reshape(t, -1), k.reshape(t, -1)
    va, ga, ba = v.reshape(t, -1), g.reshape(t, -1), beta.reshape(t, -1)
    first, s_mid = O.gdn_chunked(qa[:cut], ka[:cut], va[:cut], ga[:cut], ba[:cut], cut, h, hk, 128 ** -0.5,
                                 want_state=True)
    second, s_end = O.gdn_chunked(qa[cut:], ka[cut:], va[cut:], ga[cut:], ba[cut:], t - cut, h, hk, 128 ** -0.5,
                                  s_in=s_mid, want_state=True)
    assert np.array_equal(np.concatenate([first, second]), full)
    assert np.array_equal(s_end, s_full)


def test_attention_float64_uniform_values():
    # all keys equal -> output equals the mean of v rows, any scale
    T, Hq, Hk, Dh = 9, 4, 2, 128
    q = O.random_bf16(T * Hq * Dh, 1, 1.0)
    k = np.tile(O.random_bf16(Hk * Dh, 2, 1.0), T)
    v = O.random_bf16(T * Hk * Dh, 3, 1.0)
    out = O.attention_f64(q, k, v, 0, Hk * Dh, T, Hq, Hk, Dh, 0.1)
    vf = f32(v).reshape(T, Hk, Dh).astype(np.float64)
    for i in range(T):
        for h in range(Hq):
            assert np.allclose(out[i, h], vf[: i + 1, h // 2].mean(0), atol=1e-12)


def test_rounded_norm_and_silu_references():
    # kernels.rs:84-140 (rounding between the add and the norm) and :184-196
    d = 257
    res = O.random_bf16(3 * d, 5, 3.0).reshape(3, d)
    delta = O.random_bf16(3 * d, 6, 0.5).reshape(3, d)
    w = O.random_bf16(d, 7, 0.25)
    res[0, 0], delta[0, 0], w[1] = bf(1.0), bf(1.0 / 256.0), bf(-1.0)
    new_res, out = O.add_rms_norm(res, delta, w, 1e-6)
    assert f32(new_res)[0, 0] == 1.0            # 1 + 1/256 rounds back to 1 in bf16
    assert np.all(f32(out)[:, 1] == 0.0)        # weight -1 cancels (1 + w)
    x = f32(new_res).astype(np.float64)
    inv = 1.0 / np.sqrt((x * x).mean(1, keepdims=True).astype(np.float32) + np.float32(1e-6))
    want = bf((f32(new_res) * inv.astype(np.float32)) * (np.float32(1.0) + f32(w)))
    assert np.array_equal(out, want)
    gu = O.random_bf16(2 * 74, 23, 12.0).reshape(2, 74)
    act = O.silu_mul(gu, 74, 2, 37)
    gate = f32(gu)[:, :37].astype(np.float64)
    want = bf(f32(bf((gate / (1.0 + np.exp(-gate))).astype(np.float32))) * f32(gu)[:, 37:])
    assert np.max(np.abs(act.astype(np.int32) - want.astype(np.int32))) <= 1
