"""GPU parity of every cs1_* operator against the CPU oracle, through the C ABI.

Mirrors the reference's kernel tests (tests/qwen3_5/kernels.rs) case for case - shapes,
seeds, tolerances - and adds the operators that file leaves unpinned (conv values, gates,
gated norm, attention prep, embedding, GEMM) plus head dim 128."""
import ctypes as C

import numpy as np
import pytest

import oracle as O
from helpers import GDN_SHAPES, bf, f32, gdn_inputs, ulp_diff
from system1_omni_b200 import lib as L

pytestmark = pytest.mark.gpu
EPS = 1e-6


def dev(a, st, offset=0):
    return L.to_device(a, st, offset)


def host(buf, shape, st, dtype=np.uint16, offset_bytes=0):
    return L.from_device(buf, shape, dtype, st, offset_bytes)


# ---------------------------------------------------------------- norms

@pytest.mark.parametrize("d,offset", [(2560, 0), (5120, 0), (8192, 0), (257, 0), (8448, 0), (5120, 1), (2048, 0),
                                      (4096, 0)])
def test_residual_rms_norm_matches_rounded_reference(cs1, stream, d, offset):
    # kernels.rs:65-144: residual add bit-exact, norm within one bf16 step
    for rows in (1, 3, 107):
        n = rows * d
        residual = O.random_bf16(n + offset, 5, 3.0)
        delta = O.random_bf16(n + offset, 6, 0.5)
        weights = O.random_bf16(d + offset, 7, 0.25)
        residual[offset], delta[offset], weights[offset + 1] = bf([1.0])[0], bf([1.0 / 256.0])[0], bf([-1.0])[0]
        res_d, del_d, w_d = dev(residual, stream), dev(delta, stream), dev(weights, stream)
        out_d = L.DeviceBuffer((n + offset) * 2)
        L.check(cs1.cs1_add_rms_norm(res_d.at(offset * 2), del_d.at(offset * 2), w_d.at(offset * 2),
                                     out_d.at(offset * 2), rows, d, EPS, stream.handle), "add_rms_norm")
        want_res, want = O.add_rms_norm(residual[offset:].reshape(rows, d), delta[offset:].reshape(rows, d),
                                        weights[offset:], EPS)
        added = host(res_d, n + offset, stream)
        assert np.array_equal(added[offset:], want_res.ravel()), "residual addition changed bf16 rounding"
        if offset:
            assert added[0] == residual[0]
        got = host(out_d, n + offset, stream)[offset:]
        assert np.all(np.isfinite(f32(got)))
        assert ulp_diff(got, want.ravel()).max() <= 1


@pytest.mark.parametrize("d", [2048, 2560, 4096, 5120, 8192, 264, 257])
def test_rms_norm_matches_rounded_reference(cs1, stream, d):
    rows = 37
    x = O.random_bf16(rows * d, 9, 2.0).reshape(rows, d)
    w = O.random_bf16(d, 10, 0.25)
    out_d = L.DeviceBuffer(x.nbytes)
    x_d, w_d = dev(x, stream), dev(w, stream)
    L.check(cs1.cs1_rms_norm(x_d.at(), w_d.at(), out_d.at(), rows, d, EPS, stream.handle), "rms_norm")
    assert ulp_diff(host(out_d, (rows, d), stream), O.rms_norm(x, w, EPS)).max() <= 1
    assert np.array_equal(host(x_d, (rows, d), stream), x)      # the input is only read


def test_gated_rms_norm_matches_rounded_reference(cs1, stream):
    for T, H, extra in [(1, 16, 0), (33, 48, 2 * 48), (107, 4, 8), (5, 3, 1)]:
        ldz = H * 128 + extra
        x = O.random_bf16(T * H * 128, 31, 2.0)
        z = O.random_bf16(T * ldz, 32, 6.0)
        w = bf(1.0 + 0.25 * f32(O.random_bf16(128, 33, 1.0)))
        out_d = L.DeviceBuffer(T * H * 128 * 2)
        a, b, c = dev(x, stream), dev(z, stream), dev(w, stream)
        L.check(cs1.cs1_gated_rms_norm(a.at(), b.at(), ldz, c.at(), out_d.at(), T, H, 128, EPS, stream.handle), "gn")
        got = host(out_d, (T, H * 128), stream)
        want = O.gated_rms_norm(x, z, ldz, w, T, H, EPS)
        d = ulp_diff(got, want)
        assert d.max() <= 2 and (d == 0).mean() > 0.99
    assert cs1.cs1_gated_rms_norm(None, None, 128, None, None, 1, 1, 64, EPS, stream.handle) != 0


# ---------------------------------------------------------------- elementwise

@pytest.mark.parametrize("width,ld", [(8192, 16384), (17408, 34816), (64, 136), (37, 79), (9728, 19456)])
def test_silu_mul_matches_rounded_reference(cs1, stream, width, ld):
    # kernels.rs:146-199: the packed and element-wise paths agree exactly, within one step of the reference
    for rows in (1, 3, 107):
        inp = O.random_bf16(rows * ld, 23, 12.0)
        results = []
        for offset in (0, 1):
            src = dev(inp, stream, offset)
            out = L.DeviceBuffer((rows * width + offset) * 2)
            L.check(cs1.cs1_silu_mul(src.at(offset * 2), ld, out.at(offset * 2), rows, width, stream.handle), "silu")
            results.append(host(out, rows * width + offset, stream)[offset:])
        assert np.array_equal(results[0], results[1]), "packed/scalar mismatch"
        want = O.silu_mul(inp.reshape(rows, ld), ld, rows, width).ravel()
        assert np.all(np.isfinite(f32(results[0])))
        assert ulp_diff(results[0], want).max() <= 1


def test_sigmoid_gate_matches_reference(cs1, stream):
    for n, offset in [(4096, 0), (4099, 0), (4096, 1)]:
        x = O.random_bf16(n + offset, 41, 3.0)
        g = O.random_bf16(n + offset, 42, 12.0)
        xd, gd = dev(x, stream), dev(g, stream)
        L.check(cs1.cs1_sigmoid_gate(xd.at(offset * 2), gd.at(offset * 2), n, stream.handle), "gate")
        got = host(xd, n + offset, stream)[offset:]
        assert ulp_diff(got, O.sigmoid_gate(x[offset:], g[offset:])).max() <= 1


def test_embed_copies_rows(cs1, stream):
    table = O.random_bf16(97 * 264, 51, 1.0).reshape(97, 264)
    ids = np.array([0, 96, 5, 5, 42, 1], np.int32)
    td, idd = dev(table, stream), dev(ids, stream)
    out = L.DeviceBuffer(ids.size * 264 * 2)
    L.check(cs1.cs1_embed(idd.at(), td.at(), out.at(), ids.size, 264, stream.handle), "embed")
    assert np.array_equal(host(out, (ids.size, 264), stream), table[ids])
    assert cs1.cs1_embed(idd.at(), td.at(), out.at(), 1, 263, stream.handle) != 0
    assert cs1.cs1_embed(None, None, None, 0, 264, stream.handle) == 0


@pytest.mark.parametrize("kd,vd,extra", [(256, 512, 0), (2048, 6144, 6144 + 96), (16, 8, 8), (24, 40, 5), (7, 5, 0)])
def test_gdn_conv_matches_reference(cs1, stream, kd, vd, extra):
    ch = 2 * kd + vd
    ld = ch + extra
    for T in (1, 2, 3, 4, 17, 67) + ((2100,) if kd <= 24 else ()):      # above 2048 tokens: 16 tokens per thread
        x = O.random_bf16(T * ld, 61, 2.0)
        w = O.random_bf16(ch * 4, 62, 0.7)
        xd, wd = dev(x, stream), dev(w, stream)
        q, k, v = L.DeviceBuffer(T * kd * 2), L.DeviceBuffer(T * kd * 2), L.DeviceBuffer(T * vd * 2)
        L.check(cs1.cs1_gdn_conv(xd.at(), ld, wd.at(), q.at(), k.at(), v.at(), T, kd, vd, stream.handle), "conv")
        wq, wk, wv = O.gdn_conv(x, ld, w, T, kd, vd)
        for got, want in ((host(q, (T, kd), stream), wq), (host(k, (T, kd), stream), wk),
                          (host(v, (T, vd), stream), wv)):
            d = ulp_diff(got, want)
            assert d.max() <= 1 and (d == 0).mean() > 0.995
    assert cs1.cs1_gdn_conv(None, ch - 1, None, None, None, None, 1, kd, vd, stream.handle) != 0
    assert cs1.cs1_gdn_conv(None, ld, None, None, None, None, 0, kd, vd, stream.handle) == 0


def test_gdn_conv_continuation_uses_cached_history(cs1, stream):
    # kernels.rs:771-850: conv over (3 saved rows + suffix) repeats the rows of the full conv bit for bit
    prefix, kd, vd, heads = 64, 16 * 128, 48 * 128, 48
    ch = 2 * kd + vd
    ld = ch + vd + 2 * heads
    wd = dev(bf(np.full(ch * 4, 0.25, np.float32)), stream)

    def conv(src, start, rows):
        q, k, v = L.DeviceBuffer(rows * kd * 2), L.DeviceBuffer(rows * kd * 2), L.DeviceBuffer(rows * vd * 2)
        L.check(cs1.cs1_gdn_conv(src.at(start * ld * 2), ld, wd.at(), q.at(), k.at(), v.at(), rows, kd, vd,
                                 stream.handle), "conv")
        return [host(q, (rows, kd), stream), host(k, (rows, kd), stream), host(v, (rows, vd), stream)]

    for rows in (1, 2, 3, 4, 65):
        total = prefix + rows
        proj = bf(np.abs(f32(O.random_bf16(total * ld, 37, 0.5))) + np.float32(0.25))
        src = dev(proj, stream)
        full = conv(src, 0, total)
        tail, window = L.DeviceBuffer(3 * ld * 2), L.DeviceBuffer((rows + 3) * ld * 2)
        L.check(cs1.cs1_copy_dd(tail.at(), src.at((prefix - 3) * ld * 2), 3 * ld * 2, stream.handle), "copy")
        L.check(cs1.cs1_copy_dd(window.at(), tail.at(), 3 * ld * 2, stream.handle), "copy")
        L.check(cs1.cs1_copy_dd(window.at(3 * ld * 2), src.at(prefix * ld * 2), rows * ld * 2, stream.handle), "copy")
        restored = conv(window, 0, rows + 3)
        missing = conv(window, 3, rows)
        for i in range(3):
            assert np.array_equal(restored[i][3:], full[i][prefix:])
            assert not np.array_equal(missing[i][: min(rows, 3)], full[i][prefix: prefix + min(rows, 3)])


def test_gdn_gates_match_reference(cs1, stream):
    for T, H, ld in [(1, 16, 16), (77, 48, 16480), (5, 3, 11)]:
        b = O.random_bf16(T * ld, 71, 8.0)
        a = O.random_bf16(T * ld, 72, 30.0)     # crosses the softplus threshold of 20
        A_log = bf(np.random.default_rng(0).uniform(0, np.log(16), H).astype(np.float32))
        dt = bf(np.random.default_rng(1).normal(0, 0.1, H).astype(np.float32))
        bd, ad, Ad, dd = dev(b, stream), dev(a, stream), dev(A_log, stream), dev(dt, stream)
        beta, g = L.DeviceBuffer(T * H * 2), L.DeviceBuffer(T * H * 4)
        L.check(cs1.cs1_gdn_gates(bd.at(), ad.at(), ld, Ad.at(), dd.at(), beta.at(), g.at(), T, H, stream.handle), "g")
        wb, wg = O.gdn_gates(b, a, ld, A_log, dt, T, H)
        assert ulp_diff(host(beta, (T, H), stream), wb).max() <= 1
        got = host(g, (T, H), stream, np.float32)
        assert np.all(got <= 0) and np.allclose(got, wg, rtol=2e-6, atol=1e-30)


@pytest.mark.parametrize("T", [1, 7, 8, 9, 15, 16, 17, 67, 300, 2100])
@pytest.mark.parametrize("kd,vd,H", [(2048, 4096, 32), (256, 512, 4), (128, 384, 3)])
def test_gdn_conv_and_gates_in_one_launch(cs1, stream, T, kd, vd, H):
    """The executor's fused launch against cs1_gdn_conv then cs1_gdn_gates on the rows of one input
    projection ([q | k | v | z | b | a], model.rs:640-668 runs the two one after the other): the same bits."""
    ch = 2 * kd + vd
    ld = (ch + vd + 2 * H + 7) // 8 * 8
    x = O.random_bf16(T * ld, 63 + T, 3.0)
    w = O.random_bf16(ch * 4, 64, 0.7)
    A_log = bf(np.random.default_rng(0).uniform(0, np.log(16), H).astype(np.float32))
    dt = bf(np.random.default_rng(1).normal(0, 0.1, H).astype(np.float32))
    xd, wd, Ad, dd = dev(x, stream), dev(w, stream), dev(A_log, stream), dev(dt, stream)
    b_at, a_at = (ch + vd) * 2, (ch + vd + H) * 2
    outs = []
    for fused in (False, True):
        q, k, v = (dev(np.full(T * n, 0x7FC0, np.uint16), stream) for n in (kd, kd, vd))
        beta, g = dev(np.full(T * H, 0x7FC0, np.uint16), stream), dev(np.full(T * H, np.nan, np.float32), stream)
        if fused:
            L.check(cs1.s1_gdn_conv_gates(xd.at(), ld, wd.at(), q.at(), k.at(), v.at(), T, kd, vd, xd.at(b_at), xd.at(a_at),
                                          Ad.at(), dd.at(), beta.at(), g.at(), H, stream.handle), "fused")
        else:
            L.check(cs1.cs1_gdn_conv(xd.at(), ld, wd.at(), q.at(), k.at(), v.at(), T, kd, vd, stream.handle), "conv")
            L.check(cs1.cs1_gdn_gates(xd.at(b_at), xd.at(a_at), ld, Ad.at(), dd.at(), beta.at(), g.at(), T, H,
                                      stream.handle), "gates")
        outs.append([host(q, (T, kd), stream), host(k, (T, kd), stream), host(v, (T, vd), stream),
                     host(beta, (T, H), stream), host(g, (T, H), stream, np.float32)])
    for two, one in zip(*outs):
        assert np.array_equal(two, one)
    # widths the packed convolution does not take: the caller runs the two operators
    assert cs1.s1_gdn_conv_gates(xd.at(), ld, wd.at(), None, None, None, T, kd - 4, vd, xd.at(b_at), xd.at(a_at), Ad.at(),
                                 dd.at(), None, None, H, stream.handle) == 2000


@pytest.mark.parametrize("lens", [[1, 7, 300, 9, 16, 67], [2100, 33, 2049]])
def test_gdn_conv_and_gates_of_a_pack_in_one_launch(cs1, stream, lens):
    """s1_gdn_conv_gates_batch against s1_gdn_conv_gates per sequence: the same bits; a sequence's
    first rows see zeros before them, not the rows of the sequence packed in front."""
    kd, vd, H = 256, 512, 4
    ch = 2 * kd + vd
    ld = (ch + vd + 2 * H + 7) // 8 * 8
    T = sum(lens)
    row0 = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int32)
    ln = np.array(lens, np.int32)
    x = O.random_bf16(T * ld, 163, 3.0)
    w = O.random_bf16(ch * 4, 164, 0.7)
    A_log = bf(np.random.default_rng(0).uniform(0, np.log(16), H).astype(np.float32))
    dt = bf(np.random.default_rng(1).normal(0, 0.1, H).astype(np.float32))
    xd, wd, Ad, dd = dev(x, stream), dev(w, stream), dev(A_log, stream), dev(dt, stream)
    b_at, a_at = (ch + vd) * 2, (ch + vd + H) * 2
    outs = []
    for batch in (False, True):
        q, k, v = (dev(np.full(T * n, 0x7FC0, np.uint16), stream) for n in (kd, kd, vd))
        beta, g = dev(np.full(T * H, 0x7FC0, np.uint16), stream), dev(np.full(T * H, np.nan, np.float32), stream)
        if batch:
            L.check(cs1.s1_gdn_conv_gates_batch(xd.at(), ld, wd.at(), q.at(), k.at(), v.at(), row0.ctypes.data_as(C.c_void_p),
                                                ln.ctypes.data_as(C.c_void_p), len(lens), kd, vd, xd.at(b_at), xd.at(a_at),
                                                Ad.at(), dd.at(), beta.at(), g.at(), H, stream.handle), "batch")
        else:
            for a0, n in zip(row0.tolist(), lens):
                L.check(cs1.s1_gdn_conv_gates(xd.at(a0 * ld * 2), ld, wd.at(), q.at(a0 * kd * 2), k.at(a0 * kd * 2),
                                              v.at(a0 * vd * 2), n, kd, vd, xd.at(a0 * ld * 2 + b_at), xd.at(a0 * ld * 2 + a_at),
                                              Ad.at(), dd.at(), beta.at(a0 * H * 2), g.at(a0 * H * 4), H, stream.handle), "one")
        outs.append([host(q, (T, kd), stream), host(k, (T, kd), stream), host(v, (T, vd), stream),
                     host(beta, (T, H), stream), host(g, (T, H), stream, np.float32)])
    for one, many in zip(*outs):
        assert np.array_equal(one, many)
    assert cs1.s1_gdn_conv_gates_batch(xd.at(), ld, wd.at(), None, None, None, row0.ctypes.data_as(C.c_void_p),
                                       ln.ctypes.data_as(C.c_void_p), len(lens), kd - 4, vd, xd.at(b_at), xd.at(a_at), Ad.at(),
                                       dd.at(), None, None, H, stream.handle) == 2000


def test_device_copy_helpers_roundtrip(cs1, stream):
    # kernels.rs:744-769
    a = dev(O.random_bf16(4099, 1, 2.0), stream)
    b = L.DeviceBuffer(4099 * 2)
    L.check(cs1.cs1_copy_dd(b.at(), a.at(), 4099 * 2, stream.handle), "copy_dd")
    assert np.array_equal(host(a, 4099, stream), host(b, 4099, stream))
    rows, ld, w = 5, 300, 256
    src = O.random_bf16(rows * ld, 2, 1.0)
    sd, dst = dev(src, stream), L.DeviceBuffer(rows * w * 2)
    L.check(cs1.cs1_copy2d(dst.at(), w * 2, sd.at(), ld * 2, w * 2, rows, stream.handle), "copy2d")
    assert np.array_equal(host(dst, (rows, w), stream), src.reshape(rows, ld)[:, :w])


# ---------------------------------------------------------------- graphs

def test_graph_replay_reads_updated_inputs_after_failed_capture(cs1, stream):
    # kernels.rs:201-271
    st = stream.handle

    def capture(body):
        L.check(cs1.cs1_graph_begin(st), "graph begin")
        err = None
        try:
            body()
        except Exception as e:      # the recording failed: still end the capture
            err = e
        exec_ = C.c_void_p()
        code = cs1.cs1_graph_end(st, C.byref(exec_))
        if err is not None:
            if code == 0:
                cs1.cs1_graph_destroy(exec_)
            raise err
        L.check(code, "graph end")
        return exec_

    def failing():
        raise RuntimeError("recording failed")

    with pytest.raises(RuntimeError):
        capture(failing)
    table = bf(np.arange(24, dtype=np.float32))
    weights, ids, output = dev(table, stream), L.DeviceBuffer(8), L.DeviceBuffer(32)

    def embed():
        L.check(cs1.cs1_embed(ids.at(), weights.at(), output.at(), 2, 8, st), "capture embed")

    def assert_replay(graph, rows):
        r = np.array(rows, np.int32)
        L.check(cs1.cs1_upload(ids.at(), r.ctypes.data_as(C.c_void_p), 8, st), "upload")
        L.check(cs1.cs1_graph_launch(graph, st), "launch")
        want = np.concatenate([np.arange(x * 8, x * 8 + 8) for x in rows]).astype(np.float32)
        assert np.array_equal(f32(host(output, 16, stream)), want)

    graph = capture(embed)
    for rows in ([0, 1], [2, 0], [1, 2]):
        assert_replay(graph, rows)
    assert cs1.cs1_graph_begin(None) != 0          # the legacy default stream cannot be captured
    assert_replay(capture(embed), [0, 1])
    assert cs1.cs1_graph_launch(None, st) != 0
    assert_replay(capture(embed), [2, 0])
    for propagate in (True, False):
        def invalidating():
            embed()
            code = cs1.cs1_stream_sync(st)          # synchronising a capturing stream invalidates it
            assert code == 900
            if propagate:
                L.check(code, "invalidate capture")
        with pytest.raises(L.CudaError) as info:
            capture(invalidating)
        assert info.value.code == (900 if propagate else 901)
        assert_replay(graph, [2, 1])
        assert_replay(capture(embed), [0, 2])


# ---------------------------------------------------------------- attention

def attn_inputs(t, hq, hk, dh, amp, ldv, v_at=0, gate_amp=None):
    q = O.random_bf16(t * hq * dh, 1, amp)
    k = O.random_bf16(t * hk * dh, 2, amp)
    v = O.random_bf16(t * ldv, 3, 1.0)
    gate = None if gate_amp is None else O.random_bf16(t * hq * dh, 4, gate_amp)
    return q, k, v, gate


@pytest.mark.parametrize("dh", [256, 128])
def test_attn_prep_matches_reference(cs1, stream, dh):
    for T, hq, hk, half in [(1, 16, 4, 32), (67, 24, 4, 32), (9, 4, 4, 16), (5, 8, 2, dh // 2)]:
        attn_q = hq * dh * 2
        ld = attn_q + 2 * hk * dh
        x = O.random_bf16(T * ld, 81, 2.0)
        qw, kw = O.random_bf16(dh, 82, 0.3), O.random_bf16(dh, 83, 0.3)
        cos, sin = O.rotary_tables(np.arange(T), half, 1e7)
        xd, qwd, kwd, cd, sd = (dev(a, stream) for a in (x, qw, kw, cos, sin))
        q, g, k = L.DeviceBuffer(T * hq * dh * 2), L.DeviceBuffer(T * hq * dh * 2), L.DeviceBuffer(T * hk * dh * 2)
        L.check(cs1.cs1_attn_prep(xd.at(), xd.at(attn_q * 2), ld, qwd.at(), kwd.at(), cd.at(), sd.at(), q.at(),
                                  g.at(), k.at(), T, hq, hk, dh, half, EPS, stream.handle), "prep")
        wq, wg, wk = O.attn_prep(x, attn_q, ld, qw, kw, cos, sin, T, hq, hk, dh, half, EPS)
        assert np.array_equal(host(g, (T, hq * dh), stream), wg)
        for got, want in ((host(q, (T, hq, dh), stream), wq), (host(k, (T, hk, dh), stream), wk)):
            d = ulp_diff(got, want)
            assert d.max() <= 2 and (d == 0).mean() > 0.99
    assert cs1.cs1_attn_prep(None, None, 8, None, None, None, None, None, None, None, 1, 1, 1, 64, 32, EPS,
                             stream.handle) != 0


@pytest.mark.parametrize("dh", [256, 128])
@pytest.mark.parametrize("t,amp,hq,hk", [(1, 8.0, 16, 4), (63, 8.0, 16, 4), (65, 0.5, 16, 4), (139, 2.0, 16, 4),
                                         (700, 8.0, 16, 4), (2048, 0.5, 16, 4), (16384, 2.0, 2, 1)])
def test_flash_attention_matches_float64_reference(cs1, stream, dh, t, amp, hq, hk):
    # kernels.rs:393-474: V read in place from a 10240-wide projection row; gate < 1.6e-2.
    # The last case is the prompt cap: 128 key tiles per query tile, the approximated exponentials
    # and the skipped rescales of a long softmax, on about 64 sampled rows and the last one.
    ldv, v_at = 10240, (hq * 2 + hk) * dh if dh == 256 else (hq * 2 + hk) * dh
    ldv = max(ldv, v_at + hk * dh)
    q, k, qkv, _ = attn_inputs(t, hq, hk, dh, amp, ldv)
    qd, kd, vd = dev(q, stream), dev(k, stream), dev(qkv, stream)
    out = L.DeviceBuffer(t * hq * dh * 2)
    scale = dh ** -0.5
    L.check(cs1.cs1_attention(qd.at(), kd.at(), vd.at(v_at * 2), ldv, out.at(), t, hq, hk, dh, scale,
                              stream.handle), "attention")
    got = f32(host(out, (t, hq, dh), stream)).astype(np.float64)
    assert np.all(np.isfinite(got))
    step = -(-t // 64)      # about 64 query rows per length, and the last one
    rows = sorted(set(range(0, t, step)) | {t - 1})
    want = O.attention_f64(q, k, qkv, v_at, ldv, t, hq, hk, dh, scale, row_step=step)[rows]
    diff = np.abs(got[rows] - want).max(-1)
    worst = (diff / np.maximum(np.abs(want).max(-1), 1e-3)).max()
    assert worst < 1.6e-2, worst


@pytest.mark.parametrize("dh", [256, 128])
@pytest.mark.parametrize("climb", [0.11, 0.13, 1.5, -0.12])
def test_flash_attention_with_scores_that_climb_along_the_keys(cs1, stream, dh, climb):
    """The kernel moves a row's exponent offset only when the maximum has grown by 2^8 since the
    offset was set. Scores that rise by `climb` (in log2 units) per key make every tile's maximum
    exceed the last: at 0.11-0.13 per key a 64-key tile stays just under / just over the threshold
    (and a 128-key tile over it), so offsets go stale by up to 2^8 for tiles on end; at 1.5 every
    tile moves it; falling scores never do. All against the float64 reference."""
    t, hq, hk = 1024, 2, 1
    scale = dh ** -0.5
    rng = np.random.default_rng(17)
    # q = e0 in every row, k_j = (j * climb / (scale * log2 e)) e0 + noise: score_j * scale * log2 e = j * climb + noise
    q = np.zeros((t, hq, dh), np.float32)
    q[:, :, 0] = 1.0
    k = rng.normal(0, 0.05, (t, hk, dh)).astype(np.float32)
    k[:, :, 0] = np.arange(t)[:, None] * climb / (scale * np.log2(np.e))
    ldv = hk * dh
    q, k = O.f32_to_bf16(q.ravel()), O.f32_to_bf16(k.ravel())
    v = O.random_bf16(t * ldv, 3, 1.0)
    qd, kd, vd = dev(q, stream), dev(k, stream), dev(v, stream)
    out = L.DeviceBuffer(t * hq * dh * 2)
    L.check(cs1.cs1_attention(qd.at(), kd.at(), vd.at(), ldv, out.at(), t, hq, hk, dh, scale, stream.handle), "attention")
    got = f32(host(out, (t, hq, dh), stream)).astype(np.float64)
    assert np.all(np.isfinite(got))
    want = O.attention_f64(q, k, v, 0, ldv, t, hq, hk, dh, scale)
    diff = np.abs(got - want).max(-1)
    worst = (diff / np.maximum(np.abs(want).max(-1), 1e-3)).max()
    assert worst < 1.6e-2, worst


@pytest.mark.parametrize("dh", [256, 128])
@pytest.mark.parametrize("hq,hk", [(24, 4), (16, 4), (4, 4), (16, 1)])
def test_fused_attention_gate_matches_separate_pass(cs1, stream, dh, hq, hk):
    # kernels.rs:273-391
    scale = 0.0625 if dh == 256 else dh ** -0.5
    for t in (1, 63, 64, 65, 139, 712, 2048):
        ldv = hk * dh + 16
        q, k, v, gates = attn_inputs(t, hq, hk, dh, 2.0, ldv, gate_amp=12.0)
        gates = gates.reshape(-1, dh)
        gates[:, 0], gates[:, 1], gates[:, 2] = bf([-40.0])[0], bf([40.0])[0], 0
        n = t * hq * dh
        qd, kd, vd, gd = dev(q, stream), dev(k, stream), dev(v, stream), dev(gates, stream)
        sep, fused = L.DeviceBuffer(n * 2), L.DeviceBuffer(n * 2)
        L.check(cs1.cs1_attention(qd.at(), kd.at(), vd.at(), ldv, sep.at(), t, hq, hk, dh, scale, stream.handle), "a")
        L.check(cs1.cs1_sigmoid_gate(sep.at(), gd.at(), n, stream.handle), "g")
        L.check(cs1.cs1_attention_gated(qd.at(), kd.at(), vd.at(), ldv, gd.at(), fused.at(), t, hq, hk, dh, scale,
                                        stream.handle), "f")
        want, got = host(sep, n, stream), host(fused, n, stream)
        assert np.all(np.isfinite(f32(got)))
        assert np.array_equal(got, want), f"fused gate changed bf16 output at t={t}"
    # empty work is valid without a gate buffer; non-empty work must have one
    assert cs1.cs1_attention_gated(None, None, None, 256, None, None, 0, 1, 1, 256, 0.0625, stream.handle) == 0
    assert cs1.cs1_attention_gated(None, None, None, 256, None, None, 1, 1, 1, 256, 0.0625, stream.handle) != 0


@pytest.mark.parametrize("dh", [256, 128])
def test_windowed_attention_matches_full_pass_bit_for_bit(cs1, stream, dh):
    # kernels.rs:852-929
    hq, hk = 24, 4
    for t, bases in [(139, [64]), (712, [64, 128]), (972, [64, 896]), (2048, [64, 1024])]:
        ldv = hk * dh + 16
        q, k, v, gate = attn_inputs(t, hq, hk, dh, 2.0, ldv, gate_amp=3.0)
        qd, kd, vd, gd = dev(q, stream), dev(k, stream), dev(v, stream), dev(gate, stream)
        full = L.DeviceBuffer(t * hq * dh * 2)
        L.check(cs1.cs1_attention_gated(qd.at(), kd.at(), vd.at(), ldv, gd.at(), full.at(), t, hq, hk, dh, 0.0625,
                                        stream.handle), "full")
        full_rows = host(full, (t, hq * dh), stream)
        for qb in bases:
            win = L.DeviceBuffer(t * hq * dh * 2)
            L.check(cs1.s1_memset_async(win.at(), 0, t * hq * dh * 2, stream.handle), "memset")
            L.check(cs1.cs1_attention_gated_prefix(qd.at(), kd.at(), vd.at(), ldv, gd.at(), win.at(), t, hq, hk, dh,
                                                   0.0625, qb, stream.handle), "window")
            rows = host(win, (t, hq * dh), stream)
            assert np.array_equal(rows[qb:], full_rows[qb:])
            assert not rows[:qb].any()          # rows below q_base stay unwritten
        assert cs1.cs1_attention_gated_prefix(qd.at(), kd.at(), vd.at(), ldv, gd.at(), full.at(), t, hq, hk, dh,
                                              0.0625, 32, stream.handle) != 0


@pytest.mark.parametrize("dh", [256, 128])
@pytest.mark.parametrize("prefix_len", [0, 192])
def test_batched_attention_equals_one_call_per_sequence(cs1, stream, dh, prefix_len):
    """s1_attn_prep_batch + s1_attention_gated_batch over a pack (1 to 300 rows per sequence, unused
    rows between some) against cs1_attn_prep + s1_attention_gated_shared_prefix per sequence: the
    same bits in q, gate, k and the output; rows outside every sequence stay untouched."""
    hq, hk, half = 8, 2, 32
    lens = [5, 300, 1, 128, 129, 64, 77]
    gaps = [0, 3, 3, 0, 2, 0, 3]
    row0, at = [], 0
    for n, gap in zip(lens, gaps):
        at += gap
        row0.append(at)
        at += n
    total = at + 1
    attn_q = hq * dh * 2
    ld = attn_q + 2 * hk * dh
    x = O.random_bf16(total * ld, 61, 1.5)
    qw, kw = O.random_bf16(dh, 62, 0.3), O.random_bf16(dh, 63, 0.3)
    cos, sin = O.rotary_tables(np.arange(prefix_len + max(lens)), half, 1e7)
    kpre = O.random_bf16(max(prefix_len, 1) * hk * dh, 64, 1.0)
    vpre = O.random_bf16(max(prefix_len, 1) * hk * dh, 65, 1.0)
    xd, qwd, kwd, cd, sd, kpd, vpd = (dev(a, stream) for a in (x, qw, kw, cos, sin, kpre, vpre))
    tab = prefix_len * half * 2     # byte offset of the first position's table row
    scale = dh ** -0.5
    r0, ln = np.array(row0, np.int32), np.array(lens, np.int32)

    def buffers():
        fill = np.full(total * hq * dh, 0x7FC0, np.uint16)
        return dev(fill, stream), dev(fill, stream), dev(fill[: total * hk * dh], stream), dev(fill, stream)

    q1, g1, k1, o1 = buffers()
    L.check(cs1.s1_attn_prep_batch(xd.at(), xd.at(attn_q * 2), ld, qwd.at(), kwd.at(), cd.at(tab), sd.at(tab), q1.at(), g1.at(),
                                   k1.at(), total, r0.ctypes.data_as(C.c_void_p), ln.ctypes.data_as(C.c_void_p), len(lens), hq, hk,
                                   dh, half, EPS, stream.handle), "prep batch")
    L.check(cs1.s1_attention_gated_batch(q1.at(), k1.at(), xd.at((attn_q + hk * dh) * 2), ld, g1.at(), o1.at(),
                                         kpd.at() if prefix_len else None, vpd.at() if prefix_len else None, hk * dh, prefix_len,
                                         r0.ctypes.data_as(C.c_void_p), ln.ctypes.data_as(C.c_void_p), len(lens), hq, hk, dh,
                                         scale, stream.handle), "attention batch")
    q2, g2, k2, o2 = buffers()
    for a, n in zip(row0, lens):
        L.check(cs1.cs1_attn_prep(xd.at(a * ld * 2), xd.at((a * ld + attn_q) * 2), ld, qwd.at(), kwd.at(), cd.at(tab), sd.at(tab),
                                  q2.at(a * hq * dh * 2), g2.at(a * hq * dh * 2), k2.at(a * hk * dh * 2), n, hq, hk, dh, half, EPS,
                                  stream.handle), "prep")
        L.check(cs1.s1_attention_gated_shared_prefix(q2.at(a * hq * dh * 2), k2.at(a * hk * dh * 2),
                                                     xd.at((a * ld + attn_q + hk * dh) * 2), ld, g2.at(a * hq * dh * 2),
                                                     o2.at(a * hq * dh * 2), kpd.at() if prefix_len else None,
                                                     vpd.at() if prefix_len else None, hk * dh, prefix_len, n, hq, hk, dh, scale,
                                                     stream.handle), "attention")
    assert L.attn_status() == 0
    for got, want, width in ((q1, q2, hq * dh), (g1, g2, hq * dh), (k1, k2, hk * dh), (o1, o2, hq * dh)):
        assert np.array_equal(host(got, (total, width), stream), host(want, (total, width), stream))
    covered = np.zeros(total, bool)
    for a, n in zip(row0, lens):
        covered[a:a + n] = True
    assert np.all(host(o1, (total, hq * dh), stream)[~covered] == 0x7FC0)
    assert np.all(host(q1, (total, hq * dh), stream)[~covered] == 0x7FC0)
    many = np.ones(17, np.int32)
    assert cs1.s1_attention_gated_batch(q1.at(), k1.at(), xd.at(), ld, g1.at(), o1.at(), None, None, hk * dh, 0,
                                        many.ctypes.data_as(C.c_void_p), many.ctypes.data_as(C.c_void_p), 17, hq, hk, dh, scale,
                                        stream.handle) != 0


# ---------------------------------------------------------------- gated delta rule

def run_gdn(cs1, stream, q, k, v, g, beta, t, h, hk, s_in=None, want_state=False, t_ws=None):
    qd, kd, vd, gd, bd = dev(q, stream), dev(k, stream), dev(v, stream), dev(g, stream), dev(beta, stream)
    o = L.DeviceBuffer(t * h * 128 * 2)
    ws = L.DeviceBuffer(cs1.cs1_gdn_workspace_floats(t_ws or t, h) * 4)
    si = None if s_in is None else dev(s_in, stream)
    so = L.DeviceBuffer(h * 128 * 128 * 4) if want_state else None
    if s_in is None and not want_state:
        code = cs1.cs1_gdn_prefill(qd.at(), kd.at(), vd.at(), gd.at(), bd.at(), o.at(), ws.at(), t, h, hk,
                                   128 ** -0.5, stream.handle)
    else:
        code = cs1.cs1_gdn_prefill_x(qd.at(), kd.at(), vd.at(), gd.at(), bd.at(), o.at(), ws.at(), t, h, hk,
                                     128 ** -0.5, None if si is None else si.at(), None if so is None else so.at(),
                                     stream.handle)
    L.check(code, "gdn prefill")
    out = host(o, (t, h, 128), stream)
    if want_state:
        return out, host(so, (h, 128, 128), stream, np.float32)
    return out


@pytest.mark.parametrize("t,h,hk,decay_scale,qk_amp", GDN_SHAPES)
def test_gated_delta_rule_matches_recurrent_reference(cs1, stream, t, h, hk, decay_scale, qk_amp):
    # kernels.rs:476-622: within 2e-2 of the largest |reference| of the float64 token recurrence
    q, k, v, g, beta = gdn_inputs(t, h, hk, decay_scale, qk_amp)
    got = f32(run_gdn(cs1, stream, q, k, v, g, beta, t, h, hk)).astype(np.float64)
    assert np.all(np.isfinite(got))
    want = O.gdn_recurrent_f64(q, k, v, g, beta, t, h, hk)
    scale = np.abs(want).max()
    worst = np.abs(got - want).max()
    assert worst <= 2e-2 * scale, (worst, scale)
    # and close to the chunked float32 restatement with the same rounding points
    chunked = f32(O.gdn_chunked(q, k, v, g, beta, t, h, hk, 128 ** -0.5)).astype(np.float64)
    assert np.abs(got - chunked).max() <= 4 * 2.0 ** -8 * scale + 1e-38      # a few bf16 steps of the largest value


def test_gated_delta_rule_at_the_longest_prompt(cs1, stream):
    """16384 tokens (the prompt cap; 256 serial chunk steps) against the float64 token
    recurrence, same gate as the short shapes: the error does not build up along the chain."""
    t, h, hk = 16384, 2, 1
    q, k, v, g, beta = gdn_inputs(t, h, hk, 0.01, 1.0)
    got = f32(run_gdn(cs1, stream, q, k, v, g, beta, t, h, hk)).astype(np.float64)
    assert np.all(np.isfinite(got))
    want = O.gdn_recurrent_f64(q, k, v, g, beta, t, h, hk)
    assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max()
    # the last chunk alone is as close as the whole
    assert np.abs(got[-64:] - want[-64:]).max() <= 2e-2 * np.abs(want).max()
    assert L.gdn_status() == 0


@pytest.mark.parametrize("h,hk", [(16, 16), (32, 16), (48, 16), (24, 8)])
def test_gated_delta_rule_model_head_counts(cs1, stream, h, hk):
    t = 200
    q, k, v, g, beta = gdn_inputs(t, h, hk, 0.3, 1.0)
    got = f32(run_gdn(cs1, stream, q, k, v, g, beta, t, h, hk, t_ws=1024)).astype(np.float64)
    want = O.gdn_recurrent_f64(q, k, v, g, beta, t, h, hk)
    assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max()


def test_gdn_prefill_two_phase_matches_one_shot_bit_for_bit(cs1, stream):
    # kernels.rs:931-1088: a continuation from the float32 state at a chunk boundary repeats the one-shot pass
    for t, cut, h, hk in [(200, 128, 4, 2), (1000, 64, 6, 2), (193, 192, 32, 16)]:
        q, k, v, g, beta = gdn_inputs(t, h, hk, 0.5, 1.0)
        full, s_full = run_gdn(cs1, stream, q, k, v, g, beta, t, h, hk, want_state=True)
        qa, ka, va = q.reshape(t, -1), k.reshape(t, -1), v.reshape(t, -1)
        ga, ba = g.reshape(t, -1), beta.reshape(t, -1)
        first, s_mid = run_gdn(cs1, stream, qa[:cut], ka[:cut], va[:cut], ga[:cut], ba[:cut], cut, h, hk,
                               want_state=True)
        second, s_end = run_gdn(cs1, stream, qa[cut:], ka[cut:], va[cut:], ga[cut:], ba[cut:], t - cut, h, hk,
                                s_in=s_mid, want_state=True)
        assert np.array_equal(np.concatenate([first, second]), full)
        assert np.array_equal(s_end, s_full)
        # the state itself against the float64 recurrence
        _, s64 = O.gdn_recurrent_f64(q, k, v, g, beta, t, h, hk, want_state=True)
        assert np.abs(s_full - s64).max() <= 2e-2 * np.abs(s64).max()


@pytest.mark.parametrize("h,hk", [(4, 2), (48, 16)])
def test_gdn_prefill_batch_equals_one_call_per_sequence(cs1, stream, h, hk):
    """s1_gdn_prefill_batch over a pack (sequences of 1 to 700 tokens with unused rows between some
    of them, as the lead rows of continuations leave) against cs1_gdn_prefill_x per sequence:
    outputs and final states bit for bit, from a shared initial state and from none; the rows
    between sequences stay untouched; sizes and counts beyond the limits are refused."""
    lens = [37, 700, 1, 64, 129, 300, 5, 65]
    gaps = [0, 3, 3, 0, 7, 0, 1, 3]
    row0, at = [], 0
    for n, gap in zip(lens, gaps):
        at += gap
        row0.append(at)
        at += n
    total = at + 2
    q, k, v, g, beta = gdn_inputs(total, h, hk, 0.4, 1.0)
    qa, ka, va, ga, ba = (x.reshape(total, -1) for x in (q, k, v, g, beta))
    state = (np.random.default_rng(5).standard_normal((h, 128, 128)) * 0.05).astype(np.float32)
    qd, kd, vd, gd, bd = dev(q, stream), dev(k, stream), dev(v, stream), dev(g, stream), dev(beta, stream)
    chunks = sum(-(-n // 64) for n in lens)
    floats = cs1.cs1_gdn_workspace_floats(64 * chunks, h)
    ws = L.DeviceBuffer(floats * 4)
    r0, ln = np.array(row0, np.int32), np.array(lens, np.int32)
    for s_in in (None, state):
        si = None if s_in is None else dev(s_in, stream)
        o = dev(np.full((total, h * 128), 0x7FC0, np.uint16), stream)
        so = L.DeviceBuffer(len(lens) * h * 128 * 128 * 4)
        L.check(cs1.s1_gdn_prefill_batch(qd.at(), kd.at(), vd.at(), gd.at(), bd.at(), o.at(), ws.at(), floats,
                                         r0.ctypes.data_as(C.c_void_p), ln.ctypes.data_as(C.c_void_p), len(lens), h, hk,
                                         128 ** -0.5, None if si is None else si.at(), so.at(), stream.handle), "batch")
        got = host(o, (total, h, 128), stream)
        states = host(so, (len(lens), h, 128, 128), stream, np.float32)
        assert L.gdn_status() == 0
        covered = np.zeros(total, bool)
        for i, (a, n) in enumerate(zip(row0, lens)):
            want, s_want = run_gdn(cs1, stream, qa[a:a + n], ka[a:a + n], va[a:a + n], ga[a:a + n], ba[a:a + n], n, h, hk,
                                   s_in=s_in, want_state=True)
            assert np.array_equal(got[a:a + n], want), (i, n)
            assert np.array_equal(states[i], s_want), (i, n)
            covered[a:a + n] = True
        assert np.all(got[~covered] == 0x7FC0)
    args = (qd.at(), kd.at(), vd.at(), gd.at(), bd.at(), o.at(), ws.at())
    tail = (h, hk, 128 ** -0.5, None, None, stream.handle)
    many = np.ones(17, np.int32)
    assert cs1.s1_gdn_prefill_batch(*args, floats, many.ctypes.data_as(C.c_void_p), many.ctypes.data_as(C.c_void_p), 17, *tail) != 0
    assert cs1.s1_gdn_prefill_batch(*args, floats // 2, r0.ctypes.data_as(C.c_void_p), ln.ctypes.data_as(C.c_void_p), len(lens), *tail) != 0
    zero = np.array([5, 0], np.int32)
    assert cs1.s1_gdn_prefill_batch(*args, floats, r0.ctypes.data_as(C.c_void_p), zero.ctypes.data_as(C.c_void_p), 2, *tail) != 0


def test_gdn_empty_window_captures_state_copy_and_zero_initial_state(cs1, stream):
    # kernels.rs:692-742: T = 0 copies (or zeroes) the state as a captured graph node
    st = stream.handle
    h = 2
    n = h * 128 * 128
    state, output = dev(np.full(n, 1.0, np.float32), stream), dev(np.full(n, 2.0, np.float32), stream)

    def empty_window(inp):
        L.check(cs1.cs1_gdn_prefill_x(None, None, None, None, None, None, None, 0, h, 1, 1.0, inp, output.at(), st),
                "empty gdn window")

    def capture(body):
        L.check(cs1.cs1_graph_begin(st), "begin")
        body()
        e = C.c_void_p()
        L.check(cs1.cs1_graph_end(st, C.byref(e)), "end")
        return e

    copy = capture(lambda: empty_window(state.at()))
    updated = np.full(n, 3.0, np.float32)
    L.check(cs1.cs1_upload(state.at(), updated.ctypes.data_as(C.c_void_p), n * 4, st), "upload")
    L.check(cs1.cs1_graph_launch(copy, st), "launch")
    assert np.all(host(output, n, stream, np.float32) == 3.0)
    zero = capture(lambda: empty_window(None))
    L.check(cs1.cs1_upload(output.at(), updated.ctypes.data_as(C.c_void_p), n * 4, st), "upload")
    L.check(cs1.cs1_graph_launch(zero, st), "launch")
    assert np.all(host(output, n, stream, np.float32) == 0.0)
    assert cs1.cs1_gdn_prefill(None, None, None, None, None, None, None, 5, 4, 3, 1.0, st) != 0   # H % HK


# ---------------------------------------------------------------- GEMM

GEMM_SHAPES = [(1, 64, 64, 0), (32, 96, 128, 0), (107, 2560, 2560, 0), (128, 256, 4096, 0), (129, 300, 192, 12),
               (512, 12352, 2560, 0), (333, 1000, 9728, 24), (64, 2560, 72, 0), (5, 16, 200, 0)]


def gemm_case(M, N, K, pad, seed=0):
    x = O.random_bf16(M * K, 91 + seed, 1.0).reshape(M, K)
    w = O.random_bf16(N * K, 92 + seed, 0.05).reshape(N, K)
    return x, w, N + pad


def check_gemm(got, x, w, N):
    want = f32(O.gemm(x, w))
    diff = np.abs(f32(got[:, :N]) - want)
    # both sides round a float32-accumulated sum to bf16 once; the orders differ
    assert diff.max() <= 2 ** -7 * np.abs(want).max() + 1e-6, diff.max()
    assert (ulp_diff(got[:, :N], bf(want)) <= 1).mean() > 0.999


@pytest.mark.parametrize("M,N,K,pad", GEMM_SHAPES)
def test_gemm_plain_kernel_matches_reference(cs1, stream, M, N, K, pad):
    """The CUDA-core kernel behind cs1_gemm for what TMA cannot address (ragged K, unaligned
    views), on every shape of the list."""
    x, w, ldy = gemm_case(M, N, K, pad)
    handle = cs1.cs1_gemm_create(32 << 20)
    assert handle
    xd, wd = dev(x, stream), dev(w, stream)
    y = dev(np.full((M, ldy), 0x7FC0, np.uint16), stream)
    L.check(cs1.s1_gemm_plain(handle, xd.at(), wd.at(), y.at(), M, N, K, ldy, stream.handle), "gemm")
    got = host(y, (M, ldy), stream)
    check_gemm(got, x, w, N)
    assert np.all(got[:, N:] == 0x7FC0)           # the padding of a strided output is not touched
    cs1.cs1_gemm_destroy(handle)


@pytest.mark.parametrize("M,N,K,pad", [s for s in GEMM_SHAPES if s[2] >= 64 and s[2] % 8 == 0])
def test_gemm_tcgen05_matches_reference(cs1, stream, M, N, K, pad):
    x, w, ldy = gemm_case(M, N, K, pad)
    xd, wd = dev(x, stream), dev(w, stream)
    handle = cs1.cs1_gemm_create(32 << 20)
    # without a handle (no K split possible) and with one (the planner may split K), twice
    # with the handle so that the split path's counters are seen to return to zero
    for gemm in (None, handle, handle):
        y = dev(np.full((M, ldy), 0x7FC0, np.uint16), stream)
        L.check(cs1.s1_gemm_tcgen05(gemm, xd.at(), wd.at(), y.at(), M, N, K, ldy, stream.handle), "gemm")
        got = host(y, (M, ldy), stream)
        assert L.gemm_status() == 0, "a bounded wait inside the tcgen05 GEMM gave up"
        check_gemm(got, x, w, N)
        assert np.all(got[:, N:] == 0x7FC0)
    cs1.cs1_gemm_destroy(handle)


@pytest.mark.parametrize("M,N,K", [(1024, 2560, 4096), (1024, 2560, 9728), (512, 5120, 2560), (300, 2560, 2048)])
def test_gemm_k_split_is_deterministic(cs1, stream, M, N, K):
    """Shapes with too few tiles for the 74 block pairs split K; the partial sums are added in
    a fixed order by whichever unit finishes last, so repeated runs agree bit for bit."""
    x, w, _ = gemm_case(M, N, K, 0, seed=3)
    xd, wd = dev(x, stream), dev(w, stream)
    handle = cs1.cs1_gemm_create(32 << 20)
    outs = []
    for _ in range(3):
        y = L.DeviceBuffer(M * N * 2)
        L.check(cs1.cs1_gemm(handle, xd.at(), wd.at(), y.at(), M, N, K, N, stream.handle), "gemm")
        outs.append(host(y, (M, N), stream))
    assert L.gemm_status() == 0
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
    check_gemm(outs[0], x, w, N)
    cs1.cs1_gemm_destroy(handle)


@pytest.mark.parametrize("M,N,K,pad", [(1024, 2560, 9728, 0), (1024, 2560, 4096, 8), (1000, 2500, 2048, 4),
                                       (300, 5120, 2560, 0), (257, 96, 64 * 150, 0), (4096, 2560, 2048, 0)])
@pytest.mark.parametrize("knobs", [{"runs": 1}, {"runs": 1, "bn": 160}, {"runs": 0, "splits": 3}])
def test_gemm_shared_tile_schedules(cs1, stream, M, N, K, pad, knobs, plan_override):
    """The pair kernel's two ways of sharing a tile's K range between block pairs - contiguous
    runs over all tiles' k-blocks, and equal splits - forced through the tuning knobs: same
    result as the oracle, repeatable bit for bit, padding untouched, counters back at zero."""
    plan_override(**knobs)
    x, w, ldy = gemm_case(M, N, K, pad, seed=7)
    xd, wd = dev(x, stream), dev(w, stream)
    handle = cs1.cs1_gemm_create(32 << 20)
    outs = []
    for _ in range(3):
        y = dev(np.full((M, ldy), 0x7FC0, np.uint16), stream)
        L.check(cs1.s1_gemm_tcgen05(handle, xd.at(), wd.at(), y.at(), M, N, K, ldy, stream.handle), "gemm")
        outs.append(host(y, (M, ldy), stream))
    assert L.gemm_status() == 0
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
    check_gemm(outs[0], x, w, N)
    assert np.all(outs[0][:, N:] == 0x7FC0)
    cs1.cs1_gemm_destroy(handle)


@pytest.mark.parametrize("M,N,K,pad", [(64, 2560, 9728, 0), (128, 2560, 4096, 0), (1, 2560, 4096, 8), (77, 1000, 2048, 3),
                                       (128, 12352, 2560, 0), (33, 515, 1024, 0), (200, 2560, 4096, 0), (300, 1000, 2048, 3),
                                       (520, 2560, 9728, 8)])
@pytest.mark.parametrize("knobs", [{}, {"splits": 2, "bn": 256}, {"splits": 3, "bn": 64}, {"splits": 4},
                                   {"splits": 5, "bn": 128}, {"splits": 8, "bn": 128}])
def test_gemm_few_rows_share_k_over_a_cluster(cs1, stream, M, N, K, pad, knobs, plan_override):
    """The single-block kernel (up to 128 rows always, more where it is estimated faster than the
    pair kernel): the blocks of a cluster share a tile's k-blocks and add their float32 tiles
    through distributed shared memory in rank order - as planned and with cluster sizes and
    widths forced: the oracle's result, repeatable bit for bit, padding untouched."""
    plan_override(small_rows=4096, **knobs)       # several row blocks too go to the single-block kernel
    x, w, ldy = gemm_case(M, N, K, pad, seed=11)
    xd, wd = dev(x, stream), dev(w, stream)
    handle = cs1.cs1_gemm_create(32 << 20)
    outs = []
    for _ in range(3):
        y = dev(np.full((M, ldy), 0x7FC0, np.uint16), stream)
        L.check(cs1.s1_gemm_tcgen05(handle, xd.at(), wd.at(), y.at(), M, N, K, ldy, stream.handle), "gemm")
        outs.append(host(y, (M, ldy), stream))
    assert L.gemm_status() == 0
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
    check_gemm(outs[0], x, w, N)
    assert np.all(outs[0][:, N:] == 0x7FC0)
    cs1.cs1_gemm_destroy(handle)


@pytest.mark.parametrize("M,I,K,pad", [(1024, 9728, 2560, 0), (300, 1000, 512, 8), (129, 96, 64, 0), (700, 17408, 1024, 0),
                                       (257, 40, 128, 3)])
def test_gemm_swiglu_equals_the_two_operators(cs1, stream, M, I, K, pad, plan_override):
    """gate/up projection + SiLU-multiply in one kernel against cs1_gemm then cs1_silu_mul
    (model.rs:1301-1316 runs them as two operators): the same bits, padding untouched. (The kernel
    choice is pinned to the pair kernel above 128 rows: for some of these shapes the planner would
    take the single-block kernel and leave the activation to cs1_silu_mul.)"""
    plan_override(small_rows=128)
    x = O.random_bf16(M * K, 31, 1.0).reshape(M, K)
    w = O.random_bf16(2 * I * K, 32, 0.08).reshape(2 * I, K)
    xd, wd = dev(x, stream), dev(w, stream)
    handle = cs1.cs1_gemm_create(32 << 20)
    gate_up, want = L.DeviceBuffer(M * 2 * I * 2), L.DeviceBuffer(M * I * 2)
    L.check(cs1.s1_gemm_tcgen05(handle, xd.at(), wd.at(), gate_up.at(), M, 2 * I, K, 2 * I, stream.handle), "gemm")
    L.check(cs1.cs1_silu_mul(gate_up.at(), 2 * I, want.at(), M, I, stream.handle), "silu_mul")
    ld = I + pad
    got = dev(np.full((M, ld), 0x7FC0, np.uint16), stream)
    L.check(cs1.s1_gemm_swiglu(handle, xd.at(), wd.at(), got.at(), M, I, K, ld, stream.handle), "swiglu")
    g, wnt = host(got, (M, ld), stream), host(want, (M, I), stream)
    assert L.gemm_status() == 0
    assert np.array_equal(g[:, :I], wnt)
    assert np.all(g[:, I:] == 0x7FC0)
    # and against the oracle's two steps
    ref = O.silu_mul(O.gemm(x, w), 2 * I, M, I)
    assert (ulp_diff(g[:, :I], ref) <= 1).mean() > 0.995
    assert cs1.s1_gemm_swiglu(handle, xd.at(), wd.at(), got.at(), 128, I, K, ld, stream.handle) == 2000
    cs1.cs1_gemm_destroy(handle)


def test_gemm_rows_do_not_depend_on_the_row_count(cs1, stream):
    """Without a K split a row comes out the same however many rows the call has - the
    property the reference buys by running its out/down GEMMs per sequence (model.rs:723-739)."""
    M, N, K = 300, 2560, 4096
    x, w, _ = gemm_case(M, N, K, 0, seed=5)
    xd, wd = dev(x, stream), dev(w, stream)
    full, part = L.DeviceBuffer(M * N * 2), L.DeviceBuffer(M * N * 2)
    L.check(cs1.s1_gemm_tcgen05(None, xd.at(), wd.at(), full.at(), M, N, K, N, stream.handle), "gemm")
    L.check(cs1.s1_gemm_tcgen05(None, xd.at(100 * K * 2), wd.at(), part.at(), 37, N, K, N, stream.handle), "gemm")
    assert L.gemm_status() == 0
    assert np.array_equal(host(full, (M, N), stream)[100:137], host(part, (37, N), stream))


@pytest.mark.parametrize("M,N,K,pad", [(4200, 700, 256, 8), (2305, 264, 6144, 0), (2400, 520, 6400, 0)])
def test_gemm_many_row_blocks(cs1, stream, M, N, K, pad):
    """More than eight row blocks of 256: the tiles are walked 16 row blocks per column block where
    K <= 6144 (a ragged last group at 4200 and 2305 rows) and 8 otherwise (K = 6400). Against the
    oracle, and the rows of a window inside equal the same rows computed in a small call of their own."""
    x, w, ldy = gemm_case(M, N, K, pad, seed=9)
    xd, wd = dev(x, stream), dev(w, stream)
    y = dev(np.full((M, ldy), 0x7FC0, np.uint16), stream)
    L.check(cs1.s1_gemm_tcgen05(None, xd.at(), wd.at(), y.at(), M, N, K, ldy, stream.handle), "gemm")
    got = host(y, (M, ldy), stream)
    assert L.gemm_status() == 0
    check_gemm(got, x, w, N)
    assert np.all(got[:, N:] == 0x7FC0)
    part = L.DeviceBuffer(300 * N * 2)
    L.check(cs1.s1_gemm_tcgen05(None, xd.at(2000 * K * 2), wd.at(), part.at(), 300, N, K, N, stream.handle), "gemm")
    assert np.array_equal(got[2000:2300, :N], host(part, (300, N), stream))


def test_gemm_argument_checks(cs1, stream):
    handle = cs1.cs1_gemm_create(1 << 20)
    assert cs1.cs1_gemm(handle, None, None, None, 0, 8, 8, 8, stream.handle) == 0
    assert cs1.cs1_gemm(handle, None, None, None, 1, 8, 8, 4, stream.handle) != 0      # ldy < N
    assert cs1.cs1_gemm(None, None, None, None, 1, 8, 8, 8, stream.handle) != 0
    cs1.cs1_gemm_destroy(handle)


def test_l2norm_heads_matches_float64(cs1, stream):
    """The q / k normalisation of the delta rule as an operator of its own (gdn_prefill.cu:170-203:
    x * rsqrt(sum x^2 + 1e-6), q also times the scale), against float64 rounded to bf16."""
    rows = 1000 * 3 + 1
    x = O.random_bf16(rows * 128, 77, 2.0).reshape(rows, 128)
    x[5] = 0                                               # an all-zero row stays zero
    xd = dev(x, stream)
    out = L.DeviceBuffer(rows * 128 * 2)
    L.check(cs1.s1_l2norm_heads(xd.at(), out.at(), rows, 128 ** -0.5, stream.handle), "l2norm")
    got = host(out, (rows, 128), stream)
    xf = f32(x).astype(np.float64)
    want = bf((xf / np.sqrt((xf * xf).sum(-1, keepdims=True) + 1e-6) * 128 ** -0.5).astype(np.float32))
    assert (ulp_diff(got, want) <= 1).all()
    assert (ulp_diff(got, want) == 0).mean() > 0.98
    assert not got[5].any()
    assert cs1.s1_l2norm_heads(xd.at(2), out.at(), rows - 1, 1.0, stream.handle) != 0      # not 16-byte aligned
    assert cs1.s1_l2norm_heads(None, None, 0, 1.0, stream.handle) == 0
