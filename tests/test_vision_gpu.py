"""The vision-tower operators (ops.h:125-138 of the reference) on the GPU: against the numpy
oracle (oracle/vision.py), and side by side with the reference's own library built for sm_100
(oracle/_ref) through the same ABI on the same inputs. Image sizes: n = 1024 patches (the
tower's usual grid) and ragged ones."""
import ctypes as C
import os

import numpy as np
import pytest

import oracle as O
from oracle import vision as V
from helpers import bf, f32, ulp_diff
from system1_omni_b200 import lib as L

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref", "libqwen3_5_cuda.so")


@pytest.fixture(scope="module")
def ref(cs1):
    if not os.path.exists(REF):
        return None
    lib = L.load_other(REF)
    L.check(lib.cs1_set_device(0), "ref set device")
    return lib


def dev(a, st):
    return L.to_device(a, st)


def host(buf, shape, st, dtype=np.uint16):
    return L.from_device(buf, shape, dtype, st)


def both(cs1, ref):
    return [("this", cs1)] + ([("reference", ref)] if ref is not None else [])


def rand_bf(rng, shape, scale=1.0):
    return bf((rng.standard_normal(shape) * scale).astype(np.float32))


@pytest.mark.parametrize("rows,d", [(1024, 1024), (37, 4096), (5, 1000), (3, 72)])
def test_norm(cs1, ref, stream, rows, d):
    rng = np.random.default_rng(rows + d)
    x, w, b = rand_bf(rng, (rows, d), 2.0), rand_bf(rng, d, 0.5), rand_bf(rng, d, 0.2)
    want = V.norm(x, w, b)
    outs = {}
    for name, lib in both(cs1, ref):
        xd, wd, bd = dev(x, stream), dev(w, stream), dev(b, stream)
        y = L.DeviceBuffer(x.nbytes)
        L.check(lib.cs1_vision_norm(xd.at(), wd.at(), bd.at(), y.at(), rows, d, stream.handle), name)
        outs[name] = host(y, (rows, d), stream)
        # one bf16 step of the terms' size (about 1); where the scaled value and the bias cancel the
        # result is small and a step of it means nothing
        assert np.abs(f32(outs[name]) - f32(want)).max() <= 2 ** -7, name
        assert (ulp_diff(outs[name], want) == 0).mean() > 0.99, name
    if ref is not None:
        assert np.abs(f32(outs["this"]) - f32(outs["reference"])).max() <= 2 ** -7
        assert (ulp_diff(outs["this"], outs["reference"]) == 0).mean() > 0.99
    assert cs1.cs1_vision_norm(None, None, None, None, 0, 8, stream.handle) != 0


@pytest.mark.parametrize("n", [1024, 77])
def test_position_and_rope_are_exact(cs1, ref, stream, n):
    rng = np.random.default_rng(n)
    x = rand_bf(rng, (n, 1024))
    table = rand_bf(rng, (2304, 1024), 0.5)
    idx = rng.integers(0, 2304, (n, 4)).astype(np.int32)
    wts = rng.random((n, 4)).astype(np.float32)
    want = V.position(x, table, idx, wts)
    qkv = rand_bf(rng, (n, 3072))
    ang = rng.random((n, 32)).astype(np.float32) * 6.28
    co, si = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    want_q, want_k = V.rope(qkv, co, si)
    for name, lib in both(cs1, ref):
        xd, td, idd, wd = dev(x, stream), dev(table, stream), dev(idx, stream), dev(wts, stream)
        L.check(lib.cs1_vision_position(xd.at(), td.at(), idd.at(), wd.at(), n, stream.handle), name)
        assert np.array_equal(host(xd, (n, 1024), stream), want), name
        qd, cd, sd = dev(qkv, stream), dev(co, stream), dev(si, stream)
        q, k = L.DeviceBuffer(n * 2048), L.DeviceBuffer(n * 2048)
        L.check(lib.cs1_vision_rope(qd.at(), cd.at(), sd.at(), q.at(), k.at(), n, stream.handle), name)
        assert np.array_equal(host(q, (n, 1024), stream), want_q), name
        assert np.array_equal(host(k, (n, 1024), stream), want_k), name


@pytest.mark.parametrize("n", [4096 * 16, 1001])
def test_elementwise(cs1, ref, stream, n):
    rng = np.random.default_rng(n)
    x = rand_bf(rng, n, 3.0)
    delta = rand_bf(rng, n, 1.0)
    d = 1024 if n % 1024 == 0 else 77
    b = rand_bf(rng, d, 1.0)
    lora = rng.standard_normal(n).astype(np.float32)
    gelus = {}
    for name, lib in both(cs1, ref):
        st = stream.handle
        xd, dd = dev(x, stream), dev(delta, stream)       # held: a buffer is released when its object drops
        L.check(lib.cs1_vision_add(xd.at(), dd.at(), n, st), name)
        assert np.array_equal(host(xd, n, stream), V.add(x, delta)), name
        xd, bd = dev(x, stream), dev(b, stream)
        L.check(lib.cs1_vision_bias(xd.at(), bd.at(), n, d, st), name)
        assert np.array_equal(host(xd, n, stream), V.bias(x, b)), name
        xd, ld = dev(x, stream), dev(lora, stream)
        L.check(lib.cs1_vision_lora_add(xd.at(), ld.at(), n, 0.37, st), name)
        assert np.array_equal(host(xd, n, stream), V.lora_add(x, lora, 0.37)), name
        out, xin = L.DeviceBuffer(n * 4), dev(x, stream)
        L.check(lib.cs1_vision_to_float(xin.at(), out.at(), n, st), name)
        assert np.array_equal(host(out, n, stream, np.float32), f32(x)), name
        for exact in (1, 0):
            xd = dev(x, stream)
            L.check(lib.cs1_vision_gelu(xd.at(), n, exact, st), name)
            got, want = host(xd, n, stream), V.gelu(x, bool(exact))
            u = ulp_diff(got, want)
            # one bf16 step, or nothing to speak of where 1 + erf cancels to almost zero
            assert np.all((u <= 1) | (np.abs(f32(got) - f32(want)) <= 2.0 ** -16)), (name, exact)
            # in the negative tail 1 + erf cancels and the float32 erf's last bits decide the rounding
            assert (u == 0).mean() > 0.97, (name, exact)
            gelus[(name, exact)] = got
    if ref is not None:      # the same float32 expression on both sides
        for exact in (1, 0):
            assert (gelus[("this", exact)] == gelus[("reference", exact)]).mean() > 0.999
    assert cs1.cs1_vision_gelu(None, 0, 1, stream.handle) == 0
    assert cs1.cs1_vision_bias(None, None, 8, 0, stream.handle) != 0


@pytest.mark.parametrize("n", [1024, 1, 65, 333, 2304])
def test_attention(cs1, ref, stream, n):
    rng = np.random.default_rng(n)
    q, k = rand_bf(rng, (n, 1024), 1.5), rand_bf(rng, (n, 1024), 1.5)
    qkv = rand_bf(rng, (n, 3072))
    want = V.attention_f64(q, k, qkv[:, 2048:])
    scale = max(1e-3, np.abs(want).max())
    errs = {}
    for name, lib in both(cs1, ref):
        qd, kd, vd = dev(q, stream), dev(k, stream), dev(qkv, stream)
        out = dev(np.full((n, 1024), 0x7FC0, np.uint16), stream)
        L.check(lib.cs1_vision_attention(qd.at(), kd.at(), vd.at(2048 * 2), out.at(), n, stream.handle), name)
        got = f32(host(out, (n, 1024), stream))
        assert np.all(np.isfinite(got)), name
        errs[name] = np.abs(got - want).max() / scale
        assert errs[name] < 1.6e-2, (name, errs[name])       # the text attention's gate (kernels.rs:472)
    assert L.attn_status() == 0
    if ref is not None:
        assert errs["this"] <= 1.5 * errs["reference"] + 2e-3
    assert cs1.cs1_vision_attention(None, None, None, None, 0, stream.handle) != 0


@pytest.mark.parametrize("M,N,K", [(1024, 1024, 1024), (1024, 4096, 1024), (77, 3072, 1024), (9, 16, 1536)])
def test_linear_and_float32_gemm(cs1, ref, stream, M, N, K):
    rng = np.random.default_rng(M + N)
    x, w, b = rand_bf(rng, (M, K)), rand_bf(rng, (N, K), 0.05), rand_bf(rng, N, 0.5)
    want = V.linear_f64(x, w, b)
    xf, wf = rng.standard_normal((M, 64)).astype(np.float32), rng.standard_normal((N, 64)).astype(np.float32)
    want32 = xf.astype(np.float64) @ wf.astype(np.float64).T
    for name, lib in both(cs1, ref):
        handle = lib.cs1_gemm_create(32 << 20)
        xd, wd, bd = dev(x, stream), dev(w, stream), dev(b, stream)
        y = L.DeviceBuffer(M * N * 2)
        L.check(lib.cs1_vision_linear(handle, xd.at(), wd.at(), bd.at(), y.at(), M, N, K, stream.handle), name)
        got = host(y, (M, N), stream)
        diff = np.abs(f32(got) - want)
        assert diff.max() <= 2 ** -7 * np.abs(want).max() + 1e-6, name
        assert (ulp_diff(got, bf(want.astype(np.float32))) <= 1).mean() > 0.98, name   # small sums cancel
        y32, xfd, wfd = L.DeviceBuffer(M * N * 4), dev(xf, stream), dev(wf, stream)
        L.check(lib.cs1_gemm_f32(handle, xfd.at(), wfd.at(), y32.at(), M, N, 64, stream.handle), name)
        got32 = host(y32, (M, N), stream, np.float32)
        assert np.abs(got32 - want32).max() <= 1e-5 * np.abs(want32).max() + 1e-6, name   # float32, not TF32
        lib.cs1_gemm_destroy(handle)
    assert cs1.cs1_vision_linear(None, None, None, None, None, 1, 1, 1, stream.handle) != 0
