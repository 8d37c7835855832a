"""Prefix capture and continuation: a shared prompt prefix is run once and every candidate is
continued from its per-layer state. The reference pins split-versus-one-shot equality at the
kernel level (tests/qwen3_5/kernels.rs:771-1088) and uses the pair in its caller
(src/models/jev_vl/native/src/executor.rs:283-316); here the executor-level pair is checked
against the one-shot pass of prefix + candidate, bit for bit where the GEMMs do not split K."""
import ctypes as C

import numpy as np
import pytest

import oracle as O
from helpers import random_weights, tiny_config
from system1_omni_b200 import lib as L
from system1_omni_b200 import model as M

pytestmark = pytest.mark.gpu


def dev(a, stream):
    return L.to_device(a, stream)


@pytest.mark.parametrize("Dh,Hq,Hk", [(128, 4, 2), (256, 2, 1)])
@pytest.mark.parametrize("p,rows", [(128, 70), (64, 1), (192, 128), (0, 90)])
def test_shared_prefix_attention_equals_the_concatenated_call(cs1, stream, Dh, Hq, Hk, p, rows):
    T = p + rows
    q = O.random_bf16(T * Hq * Dh, 1, 1.0).reshape(T, Hq * Dh)
    k = O.random_bf16(T * Hk * Dh, 2, 1.0).reshape(T, Hk * Dh)
    ldv = Hk * Dh + 24
    v = O.random_bf16(T * ldv, 3, 1.0).reshape(T, ldv)
    gate = O.random_bf16(T * Hq * Dh, 4, 3.0).reshape(T, Hq * Dh)
    st = stream.handle
    qd, kd, vd, gd = dev(q, stream), dev(k, stream), dev(v, stream), dev(gate, stream)
    want = L.DeviceBuffer(T * Hq * Dh * 2)
    L.check(cs1.cs1_attention_gated_prefix(qd.at(), kd.at(), vd.at(), ldv, gd.at(), want.at(), T, Hq, Hk, Dh,
                                           Dh ** -0.5, p, st), "one buffer")
    # the window's rows in buffers of their own, the prefix's keys / values in theirs (values packed)
    qw, kw, gw = dev(q[p:], stream), dev(k[p:], stream), dev(gate[p:], stream)
    vw = dev(v[p:], stream)
    kp = dev(k[:p], stream) if p else None
    vp = dev(np.ascontiguousarray(v[:p, :Hk * Dh]), stream) if p else None
    got = L.DeviceBuffer(rows * Hq * Dh * 2)
    L.check(cs1.s1_attention_gated_shared_prefix(qw.at(), kw.at(), vw.at(), ldv, gw.at(), got.at(),
                                                 kp.at() if p else None, vp.at() if p else None, Hk * Dh, p, rows, Hq, Hk,
                                                 Dh, Dh ** -0.5, st), "shared prefix")
    a = L.from_device(want, (T, Hq * Dh), np.uint16, stream)[p:]
    b = L.from_device(got, (rows, Hq * Dh), np.uint16, stream)
    assert np.array_equal(a, b)
    assert cs1.s1_attention_gated_shared_prefix(qw.at(), kw.at(), vw.at(), ldv, gw.at(), got.at(), None, None, Hk * Dh,
                                                 32, rows, Hq, Hk, Dh, 1.0, st) != 0      # not a multiple of 64


@pytest.fixture(scope="module", params=[128, 256], ids=["dh128", "dh256"])
def setup(request, cs1):
    cfg = tiny_config(head_dim=request.param)
    model = M.Model(cfg, device=0)
    model.set_tensors(random_weights(cfg, seed=2))
    yield cfg, model
    model.close()


@pytest.mark.parametrize("plen", [64, 192])
def test_continuation_equals_the_one_shot_pass(setup, plen):
    cfg, model = setup
    rng = np.random.default_rng(plen)
    prefix_ids = rng.integers(0, cfg.vocab, plen).tolist()
    candidates = [rng.integers(0, cfg.vocab, n).tolist() for n in (5, 64, 33, 1, 130)]
    model.set_exact_packing(True)
    try:
        one_shot = model.forward_batch([prefix_ids + c for c in candidates])
        prefix = model.capture_prefix(prefix_ids)
        try:
            assert prefix.length == plen and prefix.nbytes > 0
            packed = model.forward_continue(prefix, candidates)
            # the state is read-only: a second use, in another order, gives the same rows
            again = model.forward_continue(prefix, candidates[::-1])[::-1]
            single = model.forward_continue(prefix, candidates[2:3])
        finally:
            prefix.close()
    finally:
        model.set_exact_packing(True)      # the default
    assert np.all(np.isfinite(packed))
    assert np.array_equal(packed, one_shot)
    assert np.array_equal(again, packed)
    assert np.array_equal(single[0], packed[2])


def test_more_candidates_than_a_pack_in_one_continuation(setup):
    """19 candidates behind one prefix: the per-sequence operators run them in groups of 16, and
    each still equals its whole prompt run in one piece."""
    cfg, model = setup
    rng = np.random.default_rng(33)
    prefix_ids = rng.integers(0, cfg.vocab, 128).tolist()
    candidates = [rng.integers(0, cfg.vocab, int(n)).tolist() for n in rng.integers(1, 70, 19)]
    prefix = model.capture_prefix(prefix_ids)
    try:
        packed = model.forward_continue(prefix, candidates)
    finally:
        prefix.close()
    for i in (0, 15, 16, 18):
        assert np.array_equal(packed[i], model.forward(prefix_ids + candidates[i])), i


def test_continuation_without_exact_packing_is_within_rounding(setup):
    cfg, model = setup
    rng = np.random.default_rng(9)
    prefix_ids = rng.integers(0, cfg.vocab, 128).tolist()
    candidates = [rng.integers(0, cfg.vocab, n).tolist() for n in (40, 77, 12)]
    model.set_exact_packing(False)
    try:
        one_shot = model.forward_batch([prefix_ids + c for c in candidates])
        prefix = model.capture_prefix(prefix_ids)
        try:
            packed = model.forward_continue(prefix, candidates)
        finally:
            prefix.close()
    finally:
        model.set_exact_packing(True)
    # prefill_batch.rs:57-64 allows 0.01 on scores between two ways of running the same prompt
    assert np.abs(packed - one_shot).max() <= 0.02 * max(1.0, np.abs(one_shot).max())


def test_prefix_argument_errors(setup):
    cfg, model = setup
    lib = L.load()
    handle = C.c_void_p()
    assert lib.s1_prefix_create(model.handle, 100, C.byref(handle)) == 3000       # not a multiple of 64
    assert lib.s1_prefix_create(model.handle, 0, C.byref(handle)) == 3000
    L.check(lib.s1_prefix_create(model.handle, 64, C.byref(handle)), "create")
    ids = np.zeros(64, np.int32)
    out = np.zeros((1, cfg.hidden), np.float32)
    one = np.array([3], np.int32)
    # not captured yet
    assert lib.s1_model_forward_continue(model.handle, handle, ids.ctypes.data_as(C.c_void_p),
                                         one.ctypes.data_as(C.c_void_p), 1, out.ctypes.data_as(C.c_void_p)) == 3000
    assert lib.s1_model_prefix_capture(model.handle, ids.ctypes.data_as(C.c_void_p), 63, handle) == 3000
    L.check(lib.s1_model_prefix_capture(model.handle, ids.ctypes.data_as(C.c_void_p), 64, handle), "capture")
    zero = np.array([0], np.int32)
    assert lib.s1_model_forward_continue(model.handle, handle, ids.ctypes.data_as(C.c_void_p),
                                         zero.ctypes.data_as(C.c_void_p), 1, out.ctypes.data_as(C.c_void_p)) == 3000
    other = M.Model(cfg, device=0)
    try:
        assert lib.s1_model_forward_continue(other.handle, handle, ids.ctypes.data_as(C.c_void_p),
                                             one.ctypes.data_as(C.c_void_p), 1, out.ctypes.data_as(C.c_void_p)) == 3000
    finally:
        other.close()
    assert lib.s1_prefix_len(handle) == 64
    lib.s1_prefix_destroy(handle)
