"""Same-box speed comparison with the reference's own CUDA library (oracle/_ref, its sm_80-era
kernels compiled for sm_100) on the operators of the Gated DeltaNet layer, at the shapes the
reference published timings for (H = 48, HK = 16, T in {107, 936, 3399}) and the model
shapes. Protocol after benchmarks/gdn/README.md:47-51 of the reference: warm-ups, then timed
calls between events, arms alternated. Writes ab_reference.json into $S1_RESULTS_DIR (when set)
and asserts that this library is not slower where it claims a win. Skipped when oracle/_ref is
absent."""
import ctypes as C
import json
import os

import numpy as np
import pytest

import oracle as O
from system1_omni_b200 import lib as L

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref", "libqwen3_5_cuda.so")


@pytest.fixture(scope="module")
def ref(cs1):
    if not os.path.exists(REF):
        pytest.skip("oracle/_ref/libqwen3_5_cuda.so was not built (make -C oracle ref)")
    lib = L.load_other(REF)
    L.check(lib.cs1_set_device(0), "ref set device")
    return lib


def timed(stream, call, warmup=10, iters=50):
    e0, e1 = L.Event(), L.Event()
    for _ in range(warmup):
        L.check(call(), "warm-up")
    stream.sync()
    e0.record(stream)
    for _ in range(iters):
        code = call()
    e1.record(stream)
    stream.sync()
    L.check(code, "timed")
    return e0.elapsed_ms(e1) * 1e3 / iters


def ab(stream, ref_call, own_call):
    """Two passes with the arm order reversed in the second; microseconds per call."""
    r1, o1 = timed(stream, ref_call), timed(stream, own_call)
    o2, r2 = timed(stream, own_call), timed(stream, ref_call)
    return min(r1, r2), min(o1, o2)


def test_speed_against_the_reference_library(ref, cs1, stream):
    st = stream.handle
    rows = []
    dev = lambda a: L.to_device(a, stream)
    # ---- delta rule ----
    for H, HK, T in [(48, 16, 107), (48, 16, 936), (48, 16, 3399), (32, 16, 1024), (16, 16, 2048)]:
        q, k = dev(O.random_bf16(T * HK * 128, 12, 1.0)), dev(O.random_bf16(T * HK * 128, 11, 1.0))
        v = dev(O.random_bf16(T * H * 128, 13, 1.0))
        g = dev(((O.bf16_to_f32(O.random_bf16(T * H, 14, 1.0)) - 1) * 0.3).astype(np.float32))
        beta = dev(O.f32_to_bf16(O.bf16_to_f32(O.random_bf16(T * H, 15, 0.5)) + np.float32(0.5)))
        o = L.DeviceBuffer(T * H * 128 * 2)
        calls = []
        for lib in (ref, cs1):
            ws = L.DeviceBuffer(lib.cs1_gdn_workspace_floats(T, H) * 4)
            calls.append(lambda lib=lib, ws=ws: lib.cs1_gdn_prefill(q.at(), k.at(), v.at(), g.at(), beta.at(), o.at(),
                                                                    ws.at(), T, H, HK, 128 ** -0.5, st))
        r, m = ab(stream, *calls)
        rows.append({"op": "gdn_prefill", "H": H, "HK": HK, "T": T, "reference_us": r, "this_us": m, "speedup": r / m})
    # ---- memory-bound operators at the 27B-shaped layer, 4096 tokens ----
    T, kd, vd, hv, hidden, I = 4096, 2048, 6144, 48, 5120, 17408
    ch = 2 * kd + vd
    ld = ch + vd + 2 * hv
    proj, wconv = dev(O.random_bf16(T * ld, 1, 2.0)), dev(O.random_bf16(ch * 4, 2, 0.7))
    qo, ko, vo = L.DeviceBuffer(T * kd * 2), L.DeviceBuffer(T * kd * 2), L.DeviceBuffer(T * vd * 2)
    r, m = ab(stream, *[lambda lib=lib: lib.cs1_gdn_conv(proj.at(), ld, wconv.at(), qo.at(), ko.at(), vo.at(), T, kd,
                                                         vd, st) for lib in (ref, cs1)])
    rows.append({"op": "gdn_conv", "T": T, "channels": ch, "reference_us": r, "this_us": m, "speedup": r / m})
    xn, wn, on = dev(O.random_bf16(T * vd, 4, 2.0)), dev(O.random_bf16(128, 5, 1.0)), L.DeviceBuffer(T * vd * 2)
    r, m = ab(stream, *[lambda lib=lib: lib.cs1_gated_rms_norm(xn.at(), proj.at(ch * 2), ld, wn.at(), on.at(), T, hv, 128,
                                                               1e-6, st) for lib in (ref, cs1)])
    rows.append({"op": "gated_rms_norm", "T": T, "value_dim": vd, "reference_us": r, "this_us": m, "speedup": r / m})
    res, dl, wr = dev(O.random_bf16(T * hidden, 6, 1.0)), dev(O.random_bf16(T * hidden, 7, 0.01)), dev(O.random_bf16(hidden, 8, 0.1))
    outn = L.DeviceBuffer(T * hidden * 2)
    r, m = ab(stream, *[lambda lib=lib: lib.cs1_add_rms_norm(res.at(), dl.at(), wr.at(), outn.at(), T, hidden, 1e-6, st)
                        for lib in (ref, cs1)])
    rows.append({"op": "add_rms_norm", "T": T, "hidden": hidden, "reference_us": r, "this_us": m, "speedup": r / m})
    gu, act = dev(O.random_bf16(T * 2 * I, 9, 4.0)), L.DeviceBuffer(T * I * 2)
    r, m = ab(stream, *[lambda lib=lib: lib.cs1_silu_mul(gu.at(), 2 * I, act.at(), T, I, st) for lib in (ref, cs1)])
    rows.append({"op": "silu_mul", "T": T, "intermediate": I, "reference_us": r, "this_us": m, "speedup": r / m})
    # ---- attention at the reference's head dim ----
    T, hq, hk, dh = 4096, 24, 4, 256
    qa, ka, va = dev(O.random_bf16(T * hq * dh, 1, 1.0)), dev(O.random_bf16(T * hk * dh, 2, 1.0)), dev(O.random_bf16(T * hk * dh, 3, 1.0))
    ga, oa = dev(O.random_bf16(T * hq * dh, 4, 3.0)), L.DeviceBuffer(T * hq * dh * 2)
    r, m = ab(stream, *[lambda lib=lib: lib.cs1_attention_gated(qa.at(), ka.at(), va.at(), hk * dh, ga.at(), oa.at(), T, hq,
                                                                hk, dh, 0.0625, st) for lib in (ref, cs1)])
    rows.append({"op": "attention_gated", "T": T, "Hq": hq, "Dh": dh, "reference_us": r, "this_us": m, "speedup": r / m})

    results_dir = os.environ.get("S1_RESULTS_DIR")
    if results_dir:
        os.makedirs(results_dir, exist_ok=True)
        with open(os.path.join(results_dir, "ab_reference.json"), "w") as f:
            json.dump(rows, f, indent=1)
    for row in rows:
        print(json.dumps({k: (round(v, 2) if isinstance(v, float) else v) for k, v in row.items()}))
    by = {(r_["op"], r_.get("T")): r_ for r_ in rows}
    # the claims: the memory-bound operators and the long delta-rule shapes are faster here
    for key in [("gdn_conv", 4096), ("gated_rms_norm", 4096), ("add_rms_norm", 4096), ("gdn_prefill", 3399),
                ("gdn_prefill", 936)]:
        assert by[key]["speedup"] > 1.0, by[key]
