"""Per-operator device timings through the C ABI, against each operator's roofline.

    python -m system1_omni_b200.microbench --what elementwise|gemm|gdn|attention|all [--out file.jsonl]

elementwise  the elementwise / reduction sweep: bf16 N(0,1)-like activations with
             tokens in {1k, 4k, 16k, 64k} x channels in {2048, 4096, 8192} for causal
             conv1d(k=4)+SiLU, softplus/exp decay gates, gated RMSNorm, residual add + RMSNorm,
             RMSNorm and SiLU*up; achieved GB/s = algorithmic bytes / device time.
gemm         the projection shapes of the 4B-, 9B- and 27B-shaped decoders at 1024 tokens
             (and 128 / 4096), tcgen05 kernel and cuBLASLt side by side; TFLOP/s.
gdn          the chunked gated delta rule (both kernels of cs1_gdn_prefill) at the reference's
             published shapes (H=48, HK=16, T in {107, 936, 3399}) and the model shapes; microseconds.
attention    causal GQA flash attention at head dims 128 and 256.

Calls rotate over enough copies of their buffers to exceed the 126 MB L2, so a timing is
not flattered by a warm cache; every figure is the mean of `--iters` launches between two
events on one stream after `--warmup` launches.
"""
import argparse
import ctypes as C
import json
import os
import sys

import numpy as np

from . import lib as L

L2_BYTES = 126 << 20


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p.get("hbm_gbs", 6543.7), p.get("bf16_tflops", 1646.8), "measured"
    return 6650.0, 1590.0, "fallback"


class Bench:
    def __init__(self, warmup, iters):
        self.lib = L.load()
        L.set_device(0)
        self.stream = L.Stream()
        self.warmup, self.iters = warmup, iters
        self.e0, self.e1 = L.Event(), L.Event()
        self.rng = np.random.default_rng(0)
        self.gemm_shape = None
        self.attn_shape = None

    def bf16(self, n, scale=1.0):
        """n bf16 values ~ N(0, scale) as a device buffer (bit patterns made on the host)."""
        a = (self.rng.standard_normal(min(n, 1 << 22), dtype=np.float32) * np.float32(scale))
        bits = (a.view(np.uint32) >> 16).astype(np.uint16)
        bits = np.resize(bits, n)
        return L.to_device(bits, self.stream)

    def copies(self, bytes_per_call):
        return int(min(64, max(1, -(-2 * L2_BYTES // max(bytes_per_call, 1)))))

    def time(self, call, ncopies):
        """call(i) launches on copy i; returns mean microseconds per launch."""
        st = self.stream.handle
        for i in range(self.warmup):
            L.check(call(i % ncopies), "warmup")
        self.stream.sync()
        self.e0.record(st)
        for i in range(self.iters):
            code = call(i % ncopies)
        self.e1.record(st)
        self.stream.sync()
        L.check(code, "timed call")
        return self.e0.elapsed_ms(self.e1) * 1e3 / self.iters


def elementwise(b, out):
    lib, st = b.lib, b.stream.handle
    hbm, _, src = peaks()
    for tokens in (1024, 4096, 16384, 65536):
        for ch in (2048, 4096, 8192):
            H = ch // 128
            cases = []
            # conv: ch channels in total, q|k|v = ch/4 | ch/4 | ch/2
            kd, vd = ch // 4, ch // 2
            nbytes = 4 * tokens * ch
            n = b.copies(nbytes)
            xs = [b.bf16(tokens * ch) for _ in range(n)]
            w = b.bf16(ch * 4, 0.5)
            qs = [(L.DeviceBuffer(tokens * kd * 2), L.DeviceBuffer(tokens * kd * 2), L.DeviceBuffer(tokens * vd * 2))
                  for _ in range(n)]
            cases.append(("gdn_conv_silu", nbytes + 8 * ch, n, lambda i: lib.cs1_gdn_conv(
                xs[i].at(), ch, w.at(), qs[i][0].at(), qs[i][1].at(), qs[i][2].at(), tokens, kd, vd, st)))
            # gates: H = ch / 128 heads
            gb = 10 * tokens * H
            ng = b.copies(gb)
            ba = [b.bf16(tokens * 2 * H) for _ in range(ng)]
            al, dt = b.bf16(H), b.bf16(H, 0.1)
            go = [(L.DeviceBuffer(tokens * H * 2), L.DeviceBuffer(tokens * H * 4)) for _ in range(ng)]
            cases.append(("gdn_gates", gb, ng, lambda i: lib.cs1_gdn_gates(
                ba[i].at(), ba[i].at(H * 2), 2 * H, al.at(), dt.at(), go[i][0].at(), go[i][1].at(), tokens, H, st)))
            # gated RMSNorm: value_dim = ch
            nb = 6 * tokens * ch
            nn = b.copies(nb)
            gx = [b.bf16(tokens * ch) for _ in range(nn)]
            gz = [b.bf16(tokens * ch) for _ in range(nn)]
            gw = b.bf16(128, 0.1)
            gy = [L.DeviceBuffer(tokens * ch * 2) for _ in range(nn)]
            cases.append(("gated_rms_norm", nb, nn, lambda i: lib.cs1_gated_rms_norm(
                gx[i].at(), gz[i].at(), ch, gw.at(), gy[i].at(), tokens, H, 128, 1e-6, st)))
            # add + RMSNorm: hidden = ch
            ab = 8 * tokens * ch
            na = b.copies(ab)
            res = [b.bf16(tokens * ch) for _ in range(na)]
            dl = [b.bf16(tokens * ch, 0.01) for _ in range(na)]
            nw = b.bf16(ch, 0.1)
            no = [L.DeviceBuffer(tokens * ch * 2) for _ in range(na)]
            cases.append(("add_rms_norm", ab, na, lambda i: lib.cs1_add_rms_norm(
                res[i].at(), dl[i].at(), nw.at(), no[i].at(), tokens, ch, 1e-6, st)))
            cases.append(("rms_norm", 4 * tokens * ch, na, lambda i: lib.cs1_rms_norm(
                res[i].at(), nw.at(), no[i].at(), tokens, ch, 1e-6, st)))
            # per-head L2 norm over rows of 128: ch / 128 heads per token
            cases.append(("l2norm_heads", 4 * tokens * ch, na, lambda i: lib.s1_l2norm_heads(
                res[i].at(), no[i].at(), tokens * (ch // 128), 1.0, st)))
            # SiLU * up: intermediate = ch
            sb = 6 * tokens * ch
            ns = b.copies(sb)
            gu = [b.bf16(tokens * 2 * ch) for _ in range(ns)]
            so = [L.DeviceBuffer(tokens * ch * 2) for _ in range(ns)]
            cases.append(("silu_mul", sb, ns, lambda i: lib.cs1_silu_mul(gu[i].at(), 2 * ch, so[i].at(), tokens, ch, st)))
            for name, nbytes, ncopies, call in cases:
                us = b.time(call, ncopies)
                gbs = nbytes / us / 1e3
                out({"op": name, "tokens": tokens, "channels": ch, "us": us, "algorithmic_bytes": nbytes,
                     "GB/s": gbs, "frac_of_hbm": gbs / hbm, "hbm_peak_GB/s": hbm, "peak_source": src,
                     "frac_of_8TB/s": gbs / 8000.0, "buffer_copies": ncopies})
            del xs, qs, ba, go, gx, gz, gy, res, dl, no, gu, so


MODEL_SHAPES = {
    # name: (hidden, intermediate, gdn_in, value_dim, attn_in, attn_out)
    "4B": (2560, 9728, 12352, 4096, 5120, 2048),
    "9B": (4096, 12288, 12352, 4096, 10240, 4096),
    "27B": (5120, 17408, 16480, 6144, 7168, 3072),
}


def compare_library():
    """The vendor library's GEMM as a comparison arm, from its own shared object; None if it was not built."""
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "compare", "libs1_compare.so")
    if not os.path.exists(path):
        return None
    lib = C.CDLL(path)
    lib.s1_compare_library_gemm.restype = C.c_int
    lib.s1_compare_library_gemm.argtypes = [C.c_void_p] * 3 + [C.c_int] * 3 + [C.c_void_p]
    return lib


def gemm(b, out):
    lib, st = b.lib, b.stream.handle
    _, tf, src = peaks()
    handle = lib.cs1_gemm_create(32 << 20)
    compare = compare_library()
    shapes = []
    for name, (h, I, gdn_in, vd, attn_in, attn_out) in MODEL_SHAPES.items():
        for M in ((64, 128, 1024, 4096) if name == "4B" else (1024,)):
            shapes += [(name, "gdn_in_proj", M, gdn_in, h), (name, "gdn_out_proj", M, h, vd),
                       (name, "attn_qkv", M, attn_in, h), (name, "attn_o", M, h, attn_out),
                       (name, "mlp_gate_up", M, 2 * I, h), (name, "mlp_down", M, h, I)]
    shapes.append(("square", "8192^3", 8192, 8192, 8192))
    if b.gemm_shape:
        shapes = [("custom", "custom", *b.gemm_shape)]
    for model, proj, M, N, K in shapes:
        wbytes = N * K * 2
        n = b.copies(wbytes + M * K * 2 + M * N * 2)
        n = min(n, 8)
        ws = [b.bf16(N * K, 0.02) for _ in range(n)]
        x = b.bf16(M * K)
        y = L.DeviceBuffer(M * N * 2)
        row = {"model": model, "proj": proj, "M": M, "N": N, "K": K, "flops": 2.0 * M * N * K, "weight_copies": n}
        # tcgen05: the planner free to share a tile's K range between blocks (cs1_gemm); whole_tiles: no K
        # split, a row's bits independent of the row count (what the executor runs by default)
        arms = [("tcgen05", lambda i: lib.s1_gemm_tcgen05(handle, x.at(), ws[i].at(), y.at(), M, N, K, N, st)),
                ("whole_tiles", lambda i: lib.s1_gemm_unsplit(handle, x.at(), ws[i].at(), y.at(), M, N, K, N, st))]
        if compare is not None:
            arms.append(("cublaslt", lambda i: compare.s1_compare_library_gemm(x.at(), ws[i].at(), y.at(), M, N, K, st)))
        for engine, call in arms:
            us = b.time(call, n)
            row[engine + "_us"] = us
            row[engine + "_TFLOP/s"] = row["flops"] / us / 1e6
        row["w_once_from_hbm_us"] = wbytes / (peaks()[0] * 1e3)
        row["tcgen05_frac_of_peak"] = row["tcgen05_TFLOP/s"] / tf
        if compare is not None:
            row["tcgen05_vs_cublaslt"] = row["cublaslt_us"] / row["tcgen05_us"]
        row["peak_TFLOP/s"] = tf
        row["peak_source"] = src
        out(row)
        del ws, x, y
    code = L.gemm_status()
    if code:
        raise RuntimeError(f"tcgen05 GEMM recorded a bounded-wait failure: {code}")
    lib.cs1_gemm_destroy(handle)


def gdn(b, out):
    lib, st = b.lib, b.stream.handle
    shapes = [(48, 16, 107), (48, 16, 936), (48, 16, 3399), (16, 16, 2048), (32, 16, 1024), (32, 16, 4096),
              (48, 16, 1024), (48, 16, 16384)]
    if b.gdn_shape:
        shapes = [tuple(b.gdn_shape)]
    for H, HK, T in shapes:
        q, k = b.bf16(T * HK * 128), b.bf16(T * HK * 128)
        v = b.bf16(T * H * 128)
        g = L.to_device((-np.abs(b.rng.standard_normal(T * H).astype(np.float32)) * 0.3), b.stream)
        beta = b.bf16(T * H, 0.2)
        o = L.DeviceBuffer(T * H * 128 * 2)
        ws = L.DeviceBuffer(lib.cs1_gdn_workspace_floats(T, H) * 4)
        us = b.time(lambda i: lib.cs1_gdn_prefill(q.at(), k.at(), v.at(), g.at(), beta.at(), o.at(), ws.at(), T, H,
                                                  HK, 128 ** -0.5, st), 1)
        chunks = -(-T // 64)
        flops = chunks * H * (2 * 64 * 64 * (3 * 128 + 2 * 128) + 6 * 64 * 128 * 128)
        io = T * (4 * HK * 128 + 4 * H * 128 + 6 * H)
        out({"op": "gdn_prefill", "H": H, "HK": HK, "T": T, "us": us, "tokens_per_s": T / us * 1e6,
             "dense_TFLOP/s": flops / us / 1e6, "algorithmic_GB/s": io / us / 1e3,
             "workspace_MiB": lib.cs1_gdn_workspace_floats(T, H) * 4 / 2 ** 20})


def layer(b, out):
    """Whole Gated DeltaNet layer (in_proj, conv, gates, delta rule, gated norm, out_proj) in microseconds."""
    from .gdn_layer import GdnLayer
    for name, hidden, hk, hv, T in [("cfg1", 2048, 16, 16, 2048), ("4B", 2560, 16, 32, 1024),
                                    ("9B", 4096, 16, 32, 1024), ("27B", 5120, 16, 48, 1024),
                                    ("27B", 5120, 16, 48, 4096)]:
        lay = GdnLayer(hidden, hk, hv, max_tokens=T, stream=b.stream)
        for buf, std in ((lay.w_in, 0.02), (lay.w_out, 0.02), (lay.w_conv, 0.3), (lay.a_log, 1.0), (lay.dt_bias, 0.1),
                         (lay.w_norm, 1.0)):
            a = np.abs(b.rng.standard_normal(buf.nbytes // 2, dtype=np.float32)) * np.float32(std)
            bits = (a.view(np.uint32) >> 16).astype(np.uint16)
            L.check(b.lib.cs1_upload(buf.at(), bits.ctypes.data_as(C.c_void_p), bits.nbytes, b.stream.handle), "upload")
        x = b.bf16(T * hidden)

        def call(i):
            lay.forward(x.at(), T)
            return 0

        us = b.time(call, 1)
        gf = 2.0 * T * hidden * (lay.gdn_in + lay.vd)
        out({"op": "gdn_layer", "model": name, "hidden": hidden, "k_heads": hk, "v_heads": hv, "T": T, "us": us,
             "tokens_per_s": T / us * 1e6, "projection_TFLOP/s_if_all_time": gf / us / 1e6})
        lay.close()


def prefix(b, out):
    """Shared prefix + candidates on a 9B-shaped decoder (hidden 4096, 32 layers 3:1, 16 qk / 32 v
    GDN heads, 32 q / 8 kv attention heads of 128, MLP 12288): a 1536-token prefix and 8
    candidates of 32..128 tokens. Times the one-shot packed pass over the 8 full prompts, the
    capture + packed continuation pair, and the continuation alone (prefix already cached)."""
    import time
    from . import model as M
    types = [("full_attention" if (i + 1) % 4 == 0 else "linear_attention") for i in range(32)]
    cfg = M.Config(hidden=4096, intermediate=12288, layer_types=types, heads=32, kv_heads=8, head_dim=128,
                   rotary_half=32, lin_k_heads=16, lin_v_heads=32, vocab=151936, eps=1e-6, rope_theta=1e7,
                   max_positions=262144)
    model = M.Model(cfg, device=0)
    model.init_random(seed=0, std=0.02)
    rng = np.random.default_rng(0)
    pre = rng.integers(0, cfg.vocab, 1536).tolist()
    cands = [rng.integers(0, cfg.vocab, int(n)).tolist() for n in rng.integers(32, 129, 8)]
    logical = len(pre) + sum(len(c) for c in cands)
    prompts = [pre + c for c in cands]
    packs = M.ranges([len(p) for p in prompts])

    def one_shot():
        return np.concatenate([model.forward_batch([prompts[i] for i in pack]) for pack in packs])

    def pair():
        p = model.capture_prefix(pre)
        try:
            return model.forward_continue(p, cands)
        finally:
            p.close()

    def wall(fn, warm=2, n=5):
        for _ in range(warm):
            r = fn()
        model.synchronize()
        t0 = time.perf_counter()
        for _ in range(n):
            r = fn()
        model.synchronize()
        return (time.perf_counter() - t0) / n * 1e3, r

    ms_one, ref = wall(one_shot)
    ms_pair, got = wall(pair)
    cached = model.capture_prefix(pre)
    ms_cont, got2 = wall(lambda: model.forward_continue(cached, cands))
    cached.close()
    # with every GEMM pinned to whole tiles the two ways must agree bit for bit
    model.set_exact_packing(True)
    exact_ref = np.concatenate([model.forward_batch([p]) for p in prompts[:2]])
    cached = model.capture_prefix(pre)
    exact_got = model.forward_continue(cached, cands[:2])
    cached.close()
    model.set_exact_packing(False)
    scale = max(1.0, float(np.abs(ref).max()))
    rel_l2 = float(np.linalg.norm(got - ref) / np.linalg.norm(ref))
    out({"op": "shared_prefix_request", "model": "9B-shaped", "prefix": len(pre), "candidates": [len(c) for c in cands],
         "logical_tokens": logical, "executed_tokens_one_shot": sum(len(p) for p in prompts), "packs_one_shot": len(packs),
         "one_shot_ms": ms_one, "capture_plus_continue_ms": ms_pair, "continue_only_ms": ms_cont,
         "one_shot_logical_tokens_per_s": logical / ms_one * 1e3,
         "capture_plus_continue_logical_tokens_per_s": logical / ms_pair * 1e3,
         "max_abs_diff_vs_one_shot": float(np.abs(got - ref).max()), "max_abs_diff_cached": float(np.abs(got2 - ref).max()),
         "relative_l2_vs_one_shot": rel_l2, "hidden_scale": scale,
         "bit_exact_with_whole_tile_gemms": bool(np.array_equal(exact_ref, exact_got)), "timing": "host wall clock around the public calls"})
    model.close()


def candidates(out):
    """The shared-prefix request of `prefix` with its candidates shared out over the GPUs of one
    box: run as `python -m torch.distributed.run --nproc-per-node N -m system1_omni_b200.microbench
    --what candidates` (or alone for N = 1). Every rank builds the 9B-shaped decoder, captures the
    1536-token prefix itself, and s1_dispatch_candidates assigns the 8 candidates, continues each
    rank's share in one packed pass and gathers the logits to rank 0. Rank 0 prints the wall-clock
    milliseconds (max over ranks) of the capture and of the continuation + gather, and checks two
    candidates against the whole prompt run in one piece (same bits)."""
    import os
    import time
    from . import dispatch as D
    from . import model as M
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    L.load()
    L.set_device(local)
    types = [("full_attention" if (i + 1) % 4 == 0 else "linear_attention") for i in range(32)]
    cfg = M.Config(hidden=4096, intermediate=12288, layer_types=types, heads=32, kv_heads=8, head_dim=128,
                   rotary_half=32, lin_k_heads=16, lin_v_heads=32, vocab=151936, eps=1e-6, rope_theta=1e7,
                   max_positions=262144)
    model = M.Model(cfg, device=local)
    model.init_random(seed=0, std=0.02)
    rng = np.random.default_rng(0)
    pre = rng.integers(0, cfg.vocab, 1536).tolist()
    cands = [rng.integers(0, cfg.vocab, int(n)).tolist() for n in rng.integers(32, 129, 8)]
    head = np.random.default_rng(7).normal(0, 1.0, (1, cfg.hidden)).astype(np.float32)   # a scalar score per candidate
    d = D.Dispatcher(rank, world, local)

    def timed(fn, warm=2, n=5):
        for _ in range(warm):
            r = fn()
        d.barrier()
        t0 = time.perf_counter()
        for _ in range(n):
            r = fn()
        model.synchronize()
        ms = d.max_over_ranks((time.perf_counter() - t0) / n * 1e3)
        return ms, r

    def capture():
        p = model.capture_prefix(pre)
        p.close()

    capture_ms, _ = timed(capture)
    prefix_state = model.capture_prefix(pre)
    continue_ms, (scores, where) = timed(lambda: d.candidates(model, prefix_state, cands, head))
    if rank == 0:
        same = True
        for i in (0, len(cands) - 1):
            last = model.forward_batch([np.asarray(pre + cands[i], np.int32)])[0]
            same = same and np.array_equal(M.head_logits(head, last).view(np.uint32), scores[i].view(np.uint32))
        logical = len(pre) + sum(len(c) for c in cands)
        out({"op": "shared_prefix_request_sharded", "model": "9B-shaped", "n_gpus": world, "prefix": len(pre),
             "candidates": [len(c) for c in cands], "candidates_by_rank": np.bincount(where, minlength=world).tolist(),
             "capture_ms": capture_ms, "continue_and_gather_ms": continue_ms,
             "logical_tokens_per_s": logical / (capture_ms + continue_ms) * 1e3,
             "bit_equal_to_whole_prompts": bool(same), "timing": "host wall clock, max over ranks"})
    prefix_state.close()
    d.close()
    model.close()


def requests(b, out):
    """One GPU's share of the ragged request set on a 27B-shaped decoder (hidden 5120, 64 layers
    3:1, 16 qk / 48 v GDN heads, 24 q / 4 kv attention heads of 128, MLP 17408; 47 GB of bf16
    weights): 64 requests with lengths log-uniform on [512, 16384] (seed 0), assigned to 8 ranks
    longest-first on cost T + T^2 / 65536, rank 0's share run here pack by pack. Every rank holds
    a full replica and talks to nobody during the pass, so this is what each of 8 GPUs does."""
    import time
    from . import model as M
    types = [("full_attention" if (i + 1) % 4 == 0 else "linear_attention") for i in range(64)]
    cfg = M.Config(hidden=5120, intermediate=17408, layer_types=types, heads=24, kv_heads=4, head_dim=128,
                   rotary_half=32, lin_k_heads=16, lin_v_heads=48, vocab=151936, eps=1e-6, rope_theta=1e7,
                   max_positions=262144)
    rng = np.random.default_rng(0)
    lengths = np.exp(rng.uniform(np.log(512), np.log(16384), 64)).astype(np.int64)
    rank_of = M.assign_requests(lengths, 8, 1.0, 1.0 / 65536)
    cost = lengths + lengths.astype(np.float64) ** 2 / 65536
    shares = [float(cost[rank_of == r].sum()) for r in range(8)]
    tokens_by_rank = [int(lengths[rank_of == r].sum()) for r in range(8)]
    mine = [int(n) for n in lengths[rank_of == 0]]
    model = M.Model(cfg, device=0)
    model.init_random(seed=0, std=0.02)
    prompts = [rng.integers(0, cfg.vocab, n).tolist() for n in mine]
    packs = M.ranges(mine)

    def run():
        return [model.forward_batch([prompts[i] for i in pack]) for pack in packs]

    run()
    model.synchronize()
    t0 = time.perf_counter()
    last = run()
    model.synchronize()
    sec = time.perf_counter() - t0
    out({"op": "ragged_requests_share", "model": "27B-shaped", "requests_total": 64, "tokens_total": int(lengths.sum()),
         "rank0_requests": mine, "rank0_tokens": int(sum(mine)), "packs": len(packs), "seconds": sec,
         "tokens_per_s_this_gpu": sum(mine) / sec, "tokens_by_rank": tokens_by_rank,
         "cost_imbalance_max_over_mean": max(shares) / (sum(shares) / 8),
         "finite": bool(all(np.all(np.isfinite(x)) for x in last)), "weights_GB": model.weight_bytes / 1e9,
         "timing": "host wall clock around the public calls, second pass"})
    model.close()


def single_requests(b, out):
    """Single-candidate requests one at a time on the 27B-shaped decoder: 74 prompt lengths
    log-uniform on [80, 3399] (numpy default_rng(74)), the shape statistics the reference publishes
    for its end-to-end set (74 requests of 80-3399 tokens, concurrency 1). Per request: token ids
    in host memory -> the public forward call -> last hidden row back on the host -> float64 head ->
    decision; host wall clock, second pass over the set (the first records nothing but warms
    kernels up; no length repeats, so no CUDA graph is replayed)."""
    import time
    from . import model as M
    types = [("full_attention" if (i + 1) % 4 == 0 else "linear_attention") for i in range(64)]
    cfg = M.Config(hidden=5120, intermediate=17408, layer_types=types, heads=24, kv_heads=4, head_dim=128,
                   rotary_half=32, lin_k_heads=16, lin_v_heads=48, vocab=151936, eps=1e-6, rope_theta=1e7,
                   max_positions=262144)
    rng = np.random.default_rng(74)
    lengths = np.exp(rng.uniform(np.log(80), np.log(3399), 74)).astype(np.int64)
    prompts = [rng.integers(0, cfg.vocab, int(n)).astype(np.int32) for n in lengths]
    head = np.random.default_rng(7).normal(0, 1.0, (16, cfg.hidden)).astype(np.float32)
    model = M.Model(cfg, device=0)
    model.init_random(seed=0, std=0.02)
    def two_passes():
        ms = []
        for rep in range(2):
            ms = []
            for ids in prompts:
                t0 = time.perf_counter()
                last = model.forward_batch([ids])[0]
                M.answer(M.head_logits(head, last))
                ms.append((time.perf_counter() - t0) * 1e3)
        return np.array(ms)

    # as shipped (whole-tile GEMMs, so a prompt's bits do not depend on its pack; a length vector is
    # recorded as a graph on its second sight, which is what the second pass pays for), eager only,
    # and eager with the few-row GEMM schedules that split K (faster below some 700 rows; bits then
    # depend on the row count)
    rows = {}
    for key, graphs, exact in (("default", True, True), ("eager", False, True), ("eager_split_k", False, False)):
        model.enable_graphs(graphs)
        model.set_exact_packing(exact)
        ms = two_passes()
        rows[key] = {"ms_mean": float(ms.mean()), "ms_p50": float(np.percentile(ms, 50)), "ms_p95": float(np.percentile(ms, 95)),
                     "ms_min": float(ms.min()), "ms_max": float(ms.max()), "tokens_per_s": float(lengths.sum() / ms.sum() * 1e3)}
    out({"op": "single_requests", "model": "27B-shaped", "requests": 74, "distinct_lengths": int(len(set(lengths.tolist()))),
         "tokens_min": int(lengths.min()), "tokens_max": int(lengths.max()), "tokens_mean": float(lengths.mean()),
         **{f"{k}_{name}": v for name, r in rows.items() for k, v in r.items()},
         "weights_once_through_hbm_ms": model.weight_bytes / (peaks()[0] * 1e9) * 1e3,
         "timing": "host wall clock per request around the public call, head and decision included, second pass"})
    model.close()


def latency(b, out):
    """Prefill time of one request on the 4B-shaped decoder (32 layers, 7.9 GB of bf16 weights) against
    its length, CUDA-graph replay, ids resident on the device: the short-prompt end is bound by one pass
    of the weights through HBM and by the number of launches, the long end by the GEMMs."""
    from . import model as M
    types = [("full_attention" if (i + 1) % 4 == 0 else "linear_attention") for i in range(32)]
    cfg = M.Config(hidden=2560, intermediate=9728, layer_types=types, heads=16, kv_heads=4, head_dim=128,
                   rotary_half=32, lin_k_heads=16, lin_v_heads=32, vocab=151936, eps=1e-6, rope_theta=1e7,
                   max_positions=262144)
    hbm, _, _ = peaks()
    model = M.Model(cfg, device=0)
    model.init_random(seed=0, std=0.02)
    model.enable_graphs(True)
    floor_ms = model.weight_bytes / (hbm * 1e9) * 1e3
    rng = np.random.default_rng(0)
    e0, e1 = L.Event(), L.Event()
    stream = model.stream                      # the model's own stream (a raw handle)
    for T in (64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384):
        ids = L.to_device(rng.integers(0, cfg.vocab, T).astype(np.int32), b.stream)
        lengths = np.array([T], np.int32)
        row = {"op": "prefill_latency", "model": "4B-shaped", "tokens": T}
        # graph replay and eager issue with the executor's defaults, and eager issue in plain stream
        # order (no kernel launched as a programmatic dependent of the one before)
        for key, graphs, limit in (("ms", True, 128), ("ms_eager", False, 128), ("ms_eager_stream_order", False, -1)):
            if T > 2048 and key != "ms":
                continue
            model.enable_graphs(graphs)
            model.set_overlap_tokens(limit)
            for _ in range(3):
                model.forward_device(ids.at(), lengths)
            model.synchronize()
            n = 10 if T <= 4096 else 3
            e0.record(stream)
            for _ in range(n):
                model.forward_device(ids.at(), lengths)
            e1.record(stream)
            model.synchronize()
            row[key] = e0.elapsed_ms(e1) / n
        model.set_overlap_tokens(128)
        row.update({"tokens_per_s": T / row["ms"] * 1e3, "weights_once_through_hbm_ms": floor_ms})
        out(row)
    model.close()


def attention(b, out):
    lib, st = b.lib, b.stream.handle
    cases = [(dh, hq, hk, T) for dh, hq, hk in [(128, 16, 4), (128, 24, 4), (256, 16, 4), (256, 24, 4)]
             for T in (1024, 4096, 16384)]
    if b.attn_shape:
        cases = [tuple(b.attn_shape)]
    for dh, hq, hk, T in cases:
        if True:
            q, k, v = b.bf16(T * hq * dh), b.bf16(T * hk * dh), b.bf16(T * hk * dh)
            gate = b.bf16(T * hq * dh)
            o = L.DeviceBuffer(T * hq * dh * 2)
            us = b.time(lambda i: lib.cs1_attention_gated(q.at(), k.at(), v.at(), hk * dh, gate.at(), o.at(), T, hq,
                                                          hk, dh, dh ** -0.5, st), 1)
            flops = 4.0 * hq * dh * T * (T + 1) / 2
            out({"op": "attention_gated", "Dh": dh, "Hq": hq, "Hk": hk, "T": T, "us": us,
                 "causal_TFLOP/s": flops / us / 1e6})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="all", choices=["elementwise", "gemm", "gdn", "layer", "attention", "prefix", "candidates", "requests", "single", "latency", "all"])
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--out", default=None)
    ap.add_argument("--gemm-shape", type=int, nargs=3, metavar=("M", "N", "K"), default=None,
                    help="time this one GEMM problem only (for a profiler capture)")
    ap.add_argument("--gemm-bn", type=int, default=0, help="pin the GEMM planners' tile width (s1_gemm_plan_override), 0 = their choice")
    ap.add_argument("--attn-shape", type=int, nargs=4, metavar=("Dh", "Hq", "Hk", "T"), default=None,
                    help="time this one attention problem only (for a profiler capture)")
    ap.add_argument("--gdn-shape", type=int, nargs=3, metavar=("H", "HK", "T"), default=None,
                    help="time this one delta-rule problem only (for a profiler capture)")
    args = ap.parse_args()
    if args.what == "candidates":  # one process per GPU; sets its own device
        def emit(row):
            print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in row.items()}), flush=True)
        candidates(emit)
        return 0
    b = Bench(args.warmup, args.iters)
    b.gemm_shape = args.gemm_shape
    if args.gemm_bn:
        b.lib.s1_gemm_plan_override(args.gemm_bn, 0, 2, 0)
    b.gdn_shape = args.gdn_shape
    b.attn_shape = args.attn_shape
    sink = open(args.out, "w") if args.out else None

    def out(row):
        line = json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in row.items()})
        print(line, flush=True)
        if sink:
            sink.write(line + "\n")

    for name, fn in (("elementwise", elementwise), ("gemm", gemm), ("gdn", gdn), ("layer", layer),
                     ("attention", attention)):
        if args.what in (name, "all"):
            fn(b, out)
    if args.what == "prefix":  # builds a 9B-shaped model (14 GB of weights): only on request
        prefix(b, out)
    if args.what == "latency":
        latency(b, out)
    if args.what == "single":  # builds a 27B-shaped model (47 GB of weights): only on request
        single_requests(b, out)
    if args.what == "requests":  # builds a 27B-shaped model (47 GB of weights): only on request
        requests(b, out)
    if sink:
        sink.close()


if __name__ == "__main__":
    sys.exit(main())
