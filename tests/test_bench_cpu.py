"""The benchmark's host-side pieces, without a GPU: the seeded request set and what the design
document says about it, the GEMM work per token, and the cost fit."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench


def test_request_set_is_seeded_and_its_prefixes_carry_the_same_load_per_gpu():
    lengths = bench.request_lengths()
    assert lengths.shape == (64,) and np.array_equal(lengths, bench.request_lengths())
    assert lengths.min() >= 512 and lengths.max() <= 16384
    # the first 8 N requests are what N GPUs run: tokens per GPU within 6 % of each other at N = 1, 2, 4, 8
    per_gpu = [lengths[: 8 * n].sum() / n for n in (1, 2, 4, 8)]
    assert [int(round(x, -2)) for x in per_gpu] == [40300, 41700, 41800, 39700]
    assert max(per_gpu) / min(per_gpu) < 1.06


def test_request_ids_are_per_request_and_in_range():
    lengths = bench.request_lengths()[:3]
    ids = bench.request_ids(lengths, 151936)
    assert ids.dtype == np.int32 and ids.size == lengths.sum()
    assert ids.min() >= 0 and ids.max() < 151936
    # request 1 has its own seed: the same whatever precedes it
    again = bench.request_ids(lengths[1:2], 151936)
    assert not np.array_equal(ids[lengths[0]: lengths[0] + lengths[1]], again)      # seeded by its index, not its content
    assert np.array_equal(bench.request_ids(lengths, 151936), ids)


def test_gemm_work_per_token_of_the_27b_shape():
    cfg = bench.cfg4(64)
    # 47.0 GFLOP per token over the projections of the 64 layers (48 Gated DeltaNet + 16 attention)
    assert abs(bench.gemm_flops_per_token(cfg) / 1e9 - 47.02) < 0.05
    assert sum(cfg.full_attention) == 16 and len(cfg.full_attention) == 64


def test_cost_fit_recovers_linear_and_quadratic_terms():
    rng = np.random.default_rng(0)
    packs = []
    for _ in range(12):
        t = rng.integers(512, 16384, rng.integers(1, 5)).astype(np.float64)
        packs.append((t.sum(), (t * t).sum(), 0.042 * t.sum() + 9e-8 * (t * t).sum()))
    a, b = bench.fit_cost(np.array(packs))
    assert abs(a - 0.042) < 1e-6 and abs(b - 9e-8) < 1e-10
    # times that bend the other way would give a negative quadratic term: a line through the origin instead
    bent = [(t, t * t, 0.05 * t - 1e-6 * t * t) for t in (1000.0, 4000.0, 9000.0, 16000.0)]
    a, b = bench.fit_cost(np.array(bent))
    assert b == 0.0 and 0.03 < a < 0.05
    assert bench.fit_cost(np.zeros((3, 3))) is None
