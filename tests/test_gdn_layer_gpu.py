"""The single-layer configuration: one Gated DeltaNet layer prefill, seed 0, batch 1,
T = 2048, hidden 2048, 16 q/k and 16 v heads of 128, chunk 64, conv kernel 4, x ~ N(0,1),
weights ~ N(0, 0.02), A_log ~ U(0, ln 16), dt_bias ~ N(0, 0.1). The device layer is compared
with the CPU oracle composed operator by operator (same rounding points) and with a variant
whose delta rule is the float64 token recurrence."""
import numpy as np
import pytest

import oracle as O
from helpers import bf, f32
from system1_omni_b200 import lib as L
from system1_omni_b200.gdn_layer import GdnLayer

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.linalg.norm(a - b) / np.linalg.norm(b)


def make_case(T, hidden, hk, hv, seed=0):
    rng = np.random.default_rng(seed)
    kd, vd = hk * 128, hv * 128
    conv = 2 * kd + vd
    n = lambda *s, std=0.02: bf((rng.standard_normal(s) * std).astype(np.float32))
    w = dict(in_proj=np.concatenate([n(conv, hidden), n(vd, hidden), n(hv, hidden), n(hv, hidden)], 0),
             conv=n(conv, 4, std=0.3), a_log=bf(rng.uniform(0, np.log(16), hv).astype(np.float32)),
             dt_bias=n(hv, std=0.1), norm=bf((1 + 0.02 * rng.standard_normal(128)).astype(np.float32)),
             out_proj=n(hidden, vd))
    x = bf(rng.standard_normal((T, hidden)).astype(np.float32))
    return x, w


def oracle_layer(x, w, T, hidden, hk, hv, float64_core):
    kd, vd = hk * 128, hv * 128
    conv = 2 * kd + vd
    gdn_in = conv + vd + 2 * hv
    proj = O.gemm(x, w["in_proj"])
    q, k, v = O.gdn_conv(proj, gdn_in, w["conv"], T, kd, vd)
    beta, g = O.gdn_gates(np.ascontiguousarray(proj[:, conv + vd: conv + vd + hv]),
                          np.ascontiguousarray(proj[:, conv + vd + hv:]), hv, w["a_log"], w["dt_bias"], T, hv)
    if float64_core:
        o = bf(O.gdn_recurrent_f64(q, k, v, g, beta, T, hv, hk).astype(np.float32))
    else:
        o = O.gdn_chunked(q, k, v, g, beta, T, hv, hk, 128 ** -0.5)
    z = np.ascontiguousarray(proj[:, conv: conv + vd])
    normed = O.gated_rms_norm(o.reshape(T, vd), z, vd, w["norm"], T, hv, 1e-6)
    return O.gemm(normed, w["out_proj"])


@pytest.mark.parametrize("T,hidden,hk,hv", [(2048, 2048, 16, 16), (300, 1024, 4, 8)])
def test_single_gdn_layer_matches_the_oracle(cs1, stream, T, hidden, hk, hv):
    x, w = make_case(T, hidden, hk, hv)
    layer = GdnLayer(hidden, hk, hv, max_tokens=T, stream=stream)
    try:
        layer.set_weights(**w)
        x_dev = L.to_device(x, stream)      # held: the allocation is released when the object drops
        y = layer.forward(x_dev.at(), T)
        got = f32(L.from_device(y, (T, hidden), np.uint16, stream))
        assert np.all(np.isfinite(got))
        same_rounding = f32(oracle_layer(x, w, T, hidden, hk, hv, float64_core=False))
        exact_core = f32(oracle_layer(x, w, T, hidden, hk, hv, float64_core=True))
        # bf16 activations with float32 accumulation on both sides
        assert rel_l2(got, same_rounding) < 1e-2
        assert rel_l2(got, exact_core) < 2e-2
        assert np.abs(got - exact_core).max() < 5e-2 * np.abs(exact_core).max()
    finally:
        layer.close()
