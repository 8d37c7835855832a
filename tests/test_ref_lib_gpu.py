"""Side by side with the reference itself: its own CUDA library (compiled from its sources
into oracle/_ref/ by oracle/Makefile, sm_100 build of sm_80-era kernels) and this library
run on the same seeded inputs through the same C ABI. Skipped when oracle/_ref is absent."""
import os

import numpy as np
import pytest

import oracle as O
from helpers import bf, f32, gdn_inputs, ulp_diff
from system1_omni_b200 import lib as L

pytestmark = pytest.mark.gpu
REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                   "libqwen3_5_cuda.so")
EPS = 1e-6


@pytest.fixture(scope="module")
def ref(cs1):
    if not os.path.exists(REF):
        pytest.skip("oracle/_ref/libqwen3_5_cuda.so was not built (make -C oracle ref)")
    lib = L.load_other(REF)
    L.check(lib.cs1_set_device(0), "ref set device")
    return lib


def dev(a, st):
    return L.to_device(a, st)


def host(buf, shape, st, dtype=np.uint16):
    return L.from_device(buf, shape, dtype, st)


def test_symbols_and_abi_match(ref, cs1):
    assert ref.cs1_abi_version() == cs1.cs1_abi_version() == 6
    for t, h in [(1, 4), (2048, 16), (16384, 48)]:
        # the replacement never asks for more scratch than the reference
        assert cs1.cs1_gdn_workspace_floats(t, h) <= ref.cs1_gdn_workspace_floats(t, h)


def test_silu_kernels_are_within_one_step_of_the_reference_over_many_seeds(ref, cs1, stream):
    """The convolution and SiLU-multiply here compute SiLU with the hardware's exp2 and reciprocal
    approximations where the reference divides exactly; the rounded bf16 results may then differ
    in rare ties. The contract is one bf16 step at most; the observed rate of differing elements
    over 100 seeds is printed (and must stay rare)."""
    st = stream.handle
    T, kd, vd = 67, 256, 512
    ch, I = 2 * kd + vd, 1536
    ld = ch + 64
    differing = total = 0
    for seed in range(100):
        x, w = O.random_bf16(T * ld, 1000 + seed, 2.0), O.random_bf16(ch * 4, 2000 + seed, 0.7)
        xd, wd = dev(x, stream), dev(w, stream)
        gu = dev(O.random_bf16(T * 2 * I, 3000 + seed, 12.0), stream)
        outs = []
        for lib in (ref, cs1):
            q, k, v, o = (L.DeviceBuffer(T * kd * 2), L.DeviceBuffer(T * kd * 2), L.DeviceBuffer(T * vd * 2),
                          L.DeviceBuffer(T * I * 2))
            L.check(lib.cs1_gdn_conv(xd.at(), ld, wd.at(), q.at(), k.at(), v.at(), T, kd, vd, st), "conv")
            L.check(lib.cs1_silu_mul(gu.at(), 2 * I, o.at(), T, I, st), "silu")
            outs.append(np.concatenate([host(q, T * kd, stream), host(k, T * kd, stream), host(v, T * vd, stream),
                                        host(o, T * I, stream)]))
        d = ulp_diff(*outs)
        assert d.max() <= 1, (seed, int(d.max()))
        differing += int((d != 0).sum())
        total += d.size
    print(f"SiLU kernels against the reference library: {differing} of {total} elements differ by one bf16 step")
    assert differing <= 1e-3 * total


def test_elementwise_ops_agree_with_the_reference_library(ref, cs1, stream):
    st = stream.handle
    T, kd, vd, hv = 131, 2048, 4096, 32
    ch = 2 * kd + vd
    ld = ch + vd + 2 * hv
    x, w = O.random_bf16(T * ld, 1, 2.0), O.random_bf16(ch * 4, 2, 0.7)
    xd, wd = dev(x, stream), dev(w, stream)
    outs = []
    for lib in (ref, cs1):
        q, k, v = L.DeviceBuffer(T * kd * 2), L.DeviceBuffer(T * kd * 2), L.DeviceBuffer(T * vd * 2)
        L.check(lib.cs1_gdn_conv(xd.at(), ld, wd.at(), q.at(), k.at(), v.at(), T, kd, vd, st), "conv")
        outs.append([host(q, T * kd, stream), host(k, T * kd, stream), host(v, T * vd, stream)])
    for a, b in zip(*outs):
        assert ulp_diff(a, b).max() <= 1          # SiLU by approximated exp2 / reciprocal: one step at most
    # gates
    A_log, dt = bf(np.linspace(0, 2.7, hv).astype(np.float32)), bf(np.linspace(-0.2, 0.2, hv).astype(np.float32))
    Ad, dd = dev(A_log, stream), dev(dt, stream)
    outs = []
    for lib in (ref, cs1):
        beta, g = L.DeviceBuffer(T * hv * 2), L.DeviceBuffer(T * hv * 4)
        L.check(lib.cs1_gdn_gates(xd.at((ch + vd) * 2), xd.at((ch + vd + hv) * 2), ld, Ad.at(), dd.at(), beta.at(),
                                  g.at(), T, hv, st), "gates")
        outs.append([host(beta, T * hv, stream), host(g, T * hv, stream, np.float32)])
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    # silu_mul, sigmoid gate
    I = 9728
    gu = dev(O.random_bf16(T * 2 * I, 3, 12.0), stream)
    outs = []
    for lib in (ref, cs1):
        o = L.DeviceBuffer(T * I * 2)
        L.check(lib.cs1_silu_mul(gu.at(), 2 * I, o.at(), T, I, st), "silu")
        outs.append(host(o, T * I, stream))
    assert ulp_diff(*outs).max() <= 1
    # gated norm: one warp per row there, 16 lanes here -> the sums may differ in the last bit
    xn, wn = dev(O.random_bf16(T * vd, 4, 2.0), stream), dev(bf(1 + 0.1 * f32(O.random_bf16(128, 5, 1.0))), stream)
    outs = []
    for lib in (ref, cs1):
        o = L.DeviceBuffer(T * vd * 2)
        L.check(lib.cs1_gated_rms_norm(xn.at(), xd.at(ch * 2), ld, wn.at(), o.at(), T, hv, 128, EPS, st), "gn")
        outs.append(host(o, T * vd, stream))
    d = ulp_diff(*outs)
    assert d.max() <= 2 and (d == 0).mean() > 0.999


def test_norms_agree_within_one_step(ref, cs1, stream):
    st = stream.handle
    for d in (2560, 5120, 4096, 257):
        rows = 107
        res, delta, w = O.random_bf16(rows * d, 5, 3.0), O.random_bf16(rows * d, 6, 0.5), O.random_bf16(d, 7, 0.25)
        outs = []
        for lib in (ref, cs1):
            rd, dd, wd, o = dev(res, stream), dev(delta, stream), dev(w, stream), L.DeviceBuffer(rows * d * 2)
            L.check(lib.cs1_add_rms_norm(rd.at(), dd.at(), wd.at(), o.at(), rows, d, EPS, st), "norm")
            outs.append([host(rd, rows * d, stream), host(o, rows * d, stream)])
        assert np.array_equal(outs[0][0], outs[1][0])          # residual add exact
        assert ulp_diff(outs[0][1], outs[1][1]).max() <= 1


def test_attention_and_prep_agree(ref, cs1, stream):
    st = stream.handle
    hq, hk, dh, half = 16, 4, 256, 32
    for T in (65, 700):
        attn_q = hq * dh * 2
        ld = attn_q + 2 * hk * dh
        x = O.random_bf16(T * ld, 81, 2.0)
        qw, kw = O.random_bf16(dh, 82, 0.3), O.random_bf16(dh, 83, 0.3)
        cos, sin = O.rotary_tables(np.arange(T), half, 1e7)
        xd, qwd, kwd, cd, sd = (dev(a, stream) for a in (x, qw, kw, cos, sin))
        res = []
        for lib in (ref, cs1):
            q, g, k = L.DeviceBuffer(T * hq * dh * 2), L.DeviceBuffer(T * hq * dh * 2), L.DeviceBuffer(T * hk * dh * 2)
            L.check(lib.cs1_attn_prep(xd.at(), xd.at(attn_q * 2), ld, qwd.at(), kwd.at(), cd.at(), sd.at(), q.at(),
                                      g.at(), k.at(), T, hq, hk, dh, half, EPS, st), "prep")
            out = L.DeviceBuffer(T * hq * dh * 2)
            L.check(lib.cs1_attention_gated(q.at(), k.at(), xd.at((attn_q + hk * dh) * 2), ld, g.at(), out.at(), T,
                                            hq, hk, dh, 0.0625, st), "attention")
            res.append([host(q, T * hq * dh, stream), host(k, T * hk * dh, stream), host(g, T * hq * dh, stream),
                        f32(host(out, T * hq * dh, stream))])
        assert np.array_equal(res[0][2], res[1][2])
        assert ulp_diff(res[0][0], res[1][0]).max() <= 1 and ulp_diff(res[0][1], res[1][1]).max() <= 1
        a, b = res[0][3], res[1][3]
        assert np.abs(a - b).max() <= 1.6e-2 * max(np.abs(a).max(), 1e-3)


def test_delta_rule_is_as_close_to_float64_as_the_reference(ref, cs1, stream):
    st = stream.handle
    for t, h, hk, ds in [(65, 4, 2, 1.0), (936, 6, 2, 0.01), (1024, 32, 16, 0.3)]:
        q, k, v, g, beta = gdn_inputs(t, h, hk, ds, 1.0)
        want = O.gdn_recurrent_f64(q, k, v, g, beta, t, h, hk)
        scale = np.abs(want).max()
        errs = []
        for lib in (ref, cs1):
            qd, kd, vd, gd, bd = (dev(a, stream) for a in (q, k, v, g, beta))
            o = L.DeviceBuffer(t * h * 128 * 2)
            ws = L.DeviceBuffer(lib.cs1_gdn_workspace_floats(t, h) * 4)
            L.check(lib.cs1_gdn_prefill(qd.at(), kd.at(), vd.at(), gd.at(), bd.at(), o.at(), ws.at(), t, h, hk,
                                        128 ** -0.5, st), "gdn")
            errs.append(np.abs(f32(host(o, (t, h, 128), stream)) - want).max())
        assert errs[0] <= 2e-2 * scale and errs[1] <= 2e-2 * scale
        assert errs[1] <= 1.5 * errs[0] + 1e-30, errs


def test_gemm_agrees(ref, cs1, stream):
    st = stream.handle
    M, N, K = 300, 2560, 4096
    x, w = O.random_bf16(M * K, 91, 1.0), O.random_bf16(N * K, 92, 0.05)
    xd, wd = dev(x, stream), dev(w, stream)
    outs = []
    for lib in (ref, cs1):
        handle = lib.cs1_gemm_create(32 << 20)
        y = L.DeviceBuffer(M * N * 2)
        L.check(lib.cs1_gemm(handle, xd.at(), wd.at(), y.at(), M, N, K, N, st), "gemm")
        outs.append(host(y, M * N, stream))
        lib.cs1_gemm_destroy(handle)
    assert (ulp_diff(*outs) <= 1).mean() > 0.999
