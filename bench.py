"""Prefill throughput of the 27B-shaped Qwen3.5-style hybrid decoder on B200, one process per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload: 64 layers, three Gated DeltaNet to one gated GQA attention layer, hidden 5120, MLP
17408, 16 qk / 48 v delta-rule heads, 24 q / 4 kv attention heads of 128, vocab 151936, bf16
weights N(0, 0.02) generated on each GPU (replicated). One seeded list of 64 request lengths,
log-uniform on [512, 16384]; a run on N GPUs takes its first 8 N requests (N = 8 is the whole
list; the seed is one whose prefixes resemble the whole list, so the work per GPU stays the same,
hence weak scaling), assigns whole requests to ranks
longest-first on the cost a T + b T^2 (fitted from this run's own pack times), and every rank
prefills its share in packs of at most 16 prompts / 4096 tokens through the library's
dispatcher (include/s1_dispatch.h: C++, NCCL bound at run time; this file imports no torch).
A float64 host head gives 16 decision logits per request, gathered to rank 0 in request order.
A step is one pass over the rank's share.

One JSON line on rank 0:
  value      prompt tokens of all ranks per second with the ids already in HBM: CUDA events on
             the executor's stream around K steps, the maximum over ranks
  e2e        the same from ids in pinned host memory to logits on rank 0: H2D of every pack's
             ids, layers, last rows D2H, head, NCCL gather; wall clock, the maximum over ranks
  roofline   the bf16 GEMM family: algorithmic FLOPs of this rank's tokens over the family's
             device time (events around every launch of one eager profiled step)
  balance    per-rank tokens and busy milliseconds, their max / mean, the gather's microseconds
  dispatch_check  rank 0 runs packs of another rank again through the public call and compares
             the logits bit for bit with what the gather delivered
  cpu_baseline  the CPU oracle (a port of the reference's arithmetic, OpenMP) on a bounded
             sample of the same workload, N = 1 only
  roofline.library_ms_per_step  the vendor library's GEMM on the same packs and shapes, timed after
             everything else from a comparison library of its own (N = 1 only)
--impl reference times that CPU oracle as the reference arm (the reference has no CPU forward
pass of its own: its CPU code for this path is the float64 test oracles the port restates).
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_CLASSES = 16
REQUESTS_TOTAL = 64
REQUESTS_PER_GPU = 8
# Chosen among the seeds 20000..20999 as the one whose prefixes of 8, 16 and 32 requests are most like
# the whole list (mean length and length-weighted mean length within 4 % of the 64 requests'), so
# that a GPU's work is the same at every N by construction: 40.3 k, 41.7 k, 41.8 k, 39.7 k tokens per
# GPU at N = 1, 2, 4, 8, longest request 11.7 k, 15.4 k, 15.4 k, 15.9 k.
LENGTH_SEED = 20438
SAMPLE_TOKENS = 1024        # the CPU arms' sample: one 4-layer period at this many tokens
WORKLOAD = ("cfg4: 27B-shaped hybrid decoder (64 layers 3:1 GDN/attention, hidden 5120, MLP 17408, 16 qk / 48 v GDN "
            "heads, 24 q / 4 kv heads of 128, vocab 151936, 16-class head), 64 requests log-uniform on [512, 16384] "
            f"(seed {LENGTH_SEED}), the first 8 per GPU, token-balanced over the GPUs, logits gathered to rank 0")
FAMILIES = ["gemm", "gdn_prefill", "attention", "gdn_conv", "gdn_gates", "rms_norm", "gated_rms_norm", "silu_mul",
            "attn_prep", "other"]
# DRAM bytes of one launch of the pair kernel (ncu, dram__bytes_read.sum + dram__bytes_write.sum) on the
# widest projection of this workload at one full pack; the capture and its command are under profiles/.
GEMM_TRAFFIC = {"bytes": 1.02e9,
                "of": "one launch, y[4096,34816] = x[4096,5120] w^T (gate | up at a full pack): algorithmic 683.6e6 bytes "
                      "(x 41.9e6 + w 356.5e6 + y 285.2e6); the 16 row blocks of the pack share one fetch of each column block of w"}


def cfg4(layers=64):
    from system1_omni_b200.model import Config
    types = [("full_attention" if (i + 1) % 4 == 0 else "linear_attention") for i in range(layers)]
    return Config(hidden=5120, intermediate=17408, layer_types=types, heads=24, kv_heads=4, head_dim=128,
                  rotary_half=32, lin_k_heads=16, lin_v_heads=48, vocab=151936, eps=1e-6, rope_theta=1e7,
                  max_positions=262144)


def request_lengths():
    rng = np.random.default_rng(LENGTH_SEED)
    return np.exp(rng.uniform(np.log(512), np.log(16384), REQUESTS_TOTAL)).astype(np.int32)


def request_ids(lengths, vocab):
    """All requests' token ids, concatenated in request order; request i has its own seed."""
    return np.concatenate([np.random.default_rng(1000 + i).integers(0, vocab, int(n)).astype(np.int32)
                           for i, n in enumerate(lengths)])


def gemm_flops_per_token(cfg):
    """2*N*K summed over the projections of every layer: the GEMM FLOPs one token costs."""
    h, I, kd, vd, hv = cfg.hidden, cfg.intermediate, cfg.key_dim, cfg.value_dim, cfg.lin_v_heads
    gdn = (2 * kd + vd + vd + 2 * hv) * h + h * vd
    att = (cfg.heads * cfg.head_dim * 2 + 2 * cfg.kv_heads * cfg.head_dim) * h + h * cfg.heads * cfg.head_dim
    mlp = 2 * I * h + h * I
    total = 0
    for full in cfg.full_attention:
        total += (att if full else gdn) + mlp
    return 2 * total


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"tflops": p.get("bf16_tflops_sustained", 1389.8), "hbm_gbs": p.get("hbm_gbs", 6543.7),
                "source": "measured"}
    return {"tflops": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 200 ms while running."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.lines = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, power, reasons = [], None, [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


_CPU_WEIGHTS = {}


def cpu_sample(periods=1, seed=0):
    """The CPU oracle on `periods` x (3 Gated DeltaNet + 1 attention) layers of the workload's
    shape at SAMPLE_TOKENS tokens, random hidden states in, on every host core.
    Returns (seconds, layers run, threads)."""
    import oracle as O
    O.set_threads(os.cpu_count() or 1)     # a launcher may have exported OMP_NUM_THREADS=1
    cfg = cfg4(4 * periods)
    from system1_omni_b200.model import tensor_shapes
    rng = np.random.default_rng(0)
    weights = {}
    for name, shape in tensor_shapes(cfg).items():
        if name == "embed_tokens.weight":
            weights[name] = np.zeros((1, cfg.hidden), np.uint16)      # not read: hidden states are given
            continue
        # layers of one kind share one set of arrays (made once per process): the arithmetic and
        # its cost do not depend on the values
        parts = name.split(".")
        key = ".".join(parts[2:]) if parts[0] == "layers" else name
        if key not in _CPU_WEIGHTS:
            n = int(np.prod(shape))
            if name.endswith("A_log"):
                a = rng.uniform(0, np.log(16), n).astype(np.float32)
            elif name.endswith("dt_bias"):
                a = rng.normal(0, 0.1, n).astype(np.float32)
            elif name.endswith("linear_attn.norm.weight"):
                a = (1 + rng.normal(0, 0.02, n)).astype(np.float32)
            else:
                a = rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)
            _CPU_WEIGHTS[key] = O.f32_to_bf16(a).reshape(shape)
        weights[name] = _CPU_WEIGHTS[key]
    x = O.f32_to_bf16(np.random.default_rng(seed).standard_normal((SAMPLE_TOKENS, cfg.hidden), dtype=np.float32))
    d = cfg.shape_dict()
    d["vocab"] = 1
    t0 = time.perf_counter()
    O.forward(d, weights, None, [SAMPLE_TOKENS], x_in=x)
    return time.perf_counter() - t0, cfg.n_layers, O.threads()


def cpu_line(secs, layers, threads):
    """tokens/s of the whole decoder from samples of `layers` of its 64 layers."""
    factor = 64 / layers
    mean = float(np.mean(secs))
    value = SAMPLE_TOKENS / (mean * factor)
    sample = (f"oracle port on all {threads} host threads, {layers} of 64 layers (one 3 GDN + 1 attention period) at "
              f"{SAMPLE_TOKENS} tokens: measured {mean:.2f} s per sample over {len(secs)} samples, whole decoder = "
              f"sample x {factor:g} (the sample's attention sees {SAMPLE_TOKENS} keys, the workload's requests up to 16384)")
    return value, mean * factor, {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample,
                                  "measured_s_per_sample": mean, "extrapolation_factor": factor}


def run_reference(args, rank):
    """The reference arm: the reference project has no CPU forward pass, so its arithmetic as
    restated by the oracle is timed on the host cores of this box, once per box (rank 0), on
    every core; a step is one 4-layer period of the 64-layer workload at SAMPLE_TOKENS tokens."""
    if rank != 0:
        return
    secs = []
    layers = threads = None
    for i in range(args.warmup + args.steps):
        if i >= 1 and sum(secs) > 150:       # keep the whole run within a few minutes
            break
        t, layers, threads = cpu_sample(1, seed=i)
        if i >= min(args.warmup, 1):
            secs.append(t)
    value, step_s, cpu = cpu_line(secs, layers, threads)
    line = {"impl": "reference", "metric": "prefill tokens/s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": len(secs), "warmup": min(args.warmup, 1), "ms_per_step": step_s * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "layers": 64,
                       "note": "one box has one set of host cores: the figure does not grow with the number of GPUs",
                       "weights": "N(0,0.02) bf16, generated on the host"},
            "cpu_baseline": cpu,
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def library_gemm_ms(cfg, model, pack_rows, stream):
    """The vendor library's GEMM (cuBLASLt, from the comparison arm's own shared object, which the
    product neither links nor loads) on every projection shape of one step, after the timed
    regions, and this library's kernel under the same protocol: each (pack, projection) timed alone
    (a warm-up launch, then 3 launches between events), milliseconds x the layers that run it,
    summed over the step. Operands are the model's own random weights (w: the projection of the
    first layer of its kind, x: rows of the embedding table), so that neither arm computes on
    constant data."""
    from system1_omni_b200 import lib as L
    from system1_omni_b200.microbench import compare_library
    compare = compare_library()
    if compare is None:
        return None
    lib = L.load()
    h, I = cfg.hidden, cfg.intermediate
    gdn_in = 2 * cfg.key_dim + 2 * cfg.value_dim + 2 * cfg.lin_v_heads
    attn_in = cfg.heads * cfg.head_dim * 2 + 2 * cfg.kv_heads * cfg.head_dim
    full = cfg.full_attention
    n_full = sum(full)
    n_lin = cfg.n_layers - n_full
    lin, att = full.index(False) if n_lin else None, full.index(True) if n_full else None

    def tensor(name):
        ptr, nbytes = C.c_void_p(), C.c_size_t()
        L.check(lib.s1_model_tensor(model.handle, name.encode(), C.byref(ptr), C.byref(nbytes)), name)
        return ptr

    shapes = [(2 * I, h, cfg.n_layers, tensor("layers.0.mlp.gate_proj.weight")),
              (h, I, cfg.n_layers, tensor("layers.0.mlp.down_proj.weight"))]
    if n_lin:
        shapes += [(gdn_in, h, n_lin, tensor(f"layers.{lin}.linear_attn.in_proj_qkv.weight")),
                   (h, cfg.value_dim, n_lin, tensor(f"layers.{lin}.linear_attn.out_proj.weight"))]
    if n_full:
        shapes += [(attn_in, h, n_full, tensor(f"layers.{att}.self_attn.q_proj.weight")),
                   (h, cfg.heads * cfg.head_dim, n_full, tensor(f"layers.{att}.self_attn.o_proj.weight"))]
    x = tensor("embed_tokens.weight")
    rows = max(pack_rows)
    if rows * max(k for _, k, _, _ in shapes) > cfg.vocab * h:
        return None
    y = L.DeviceBuffer(rows * max(n for n, _, _, _ in shapes) * 2)
    handle = lib.cs1_gemm_create(0)
    e0, e1 = L.Event(), L.Event()

    def timed(call):
        if call() != 0:
            return None
        e0.record(stream)
        for _ in range(3):
            call()
        e1.record(stream)
        e1.sync()
        return e0.elapsed_ms(e1) / 3

    ours = theirs = 0.0
    for m in pack_rows:
        for n, k, count, w in shapes:
            a = timed(lambda: lib.s1_gemm_unsplit(handle, x, w, y.at(), m, n, k, n, stream))
            b = timed(lambda: compare.s1_compare_library_gemm(x, w, y.at(), m, n, k, stream))
            if a is None or b is None:
                lib.cs1_gemm_destroy(handle)
                return None
            ours += a * count
            theirs += b * count
    lib.cs1_gemm_destroy(handle)
    return {"library_ms": theirs, "own_ms": ours,
            "note": "cuBLASLt and this library's whole-tile GEMM on the same packs, projection shapes and operands, each "
                    "launch shape timed alone (short bursts at high clocks, unlike the seconds-long step) x its layers; "
                    "the gate/up product here writes [rows, 2 I] in both arms (in the step this library's epilogue "
                    "applies the SiLU-multiply and writes half of it)"}


def fit_cost(samples):
    """Least squares of pack milliseconds on (sum T, sum T^2) over every rank's packs; a, b >= 0."""
    s = np.asarray([r for r in samples if r[2] > 0], np.float64)
    if len(s) < 2:
        return None
    X, y = s[:, :2], s[:, 2]
    coef, *_ = np.linalg.lstsq(X, y, rcond=None)
    a, b = float(coef[0]), float(coef[1])
    if b < 0 or a <= 0:           # not enough spread in this run's lengths to see the quadratic term
        a, b = float((X[:, 0] @ y) / (X[:, 0] @ X[:, 0])), 0.0
    return a, b


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=64, help="fewer layers for a quick functional check only")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-library-arm", action="store_true", help="skip the vendor library's GEMM comparison (N = 1 only)")
    ap.add_argument("--graphs", type=int, default=1, help="CUDA-graph replay of repeated packs (0 = eager)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    args.warmup = max(args.warmup, 3)

    # stdout carries the one JSON line: whatever a library prints meanwhile (NCCL's log, when the
    # environment asks for one) goes to stderr
    sys.stdout.flush()
    json_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)

    from system1_omni_b200 import dispatch as D
    from system1_omni_b200 import lib as L
    from system1_omni_b200 import model as M
    lib = L.load()                  # raises when the CUDA library is missing: there is no other path
    L.set_device(local)
    cfg = cfg4(args.layers)
    model = M.Model(cfg, device=local)
    model.init_random(seed=0, std=0.02)
    model.enable_graphs(bool(args.graphs))
    stream = model.stream
    disp = D.Dispatcher(rank, world, local)

    lengths = request_lengths()[: min(REQUESTS_TOTAL, REQUESTS_PER_GPU * world)]
    ids_all = request_ids(lengths, cfg.vocab)
    head = np.random.default_rng(7).normal(0, 1.0, (N_CLASSES, cfg.hidden)).astype(np.float32)
    disp.plan(model, lengths, N_CLASSES)
    disp.stage(ids_all)
    disp.upload()

    # ---- the assignment's cost model from this run's own pack times (every rank, same arithmetic) ----
    disp.enqueue(resident=True)          # first pass: kernel attributes, tensor maps
    disp.enqueue(resident=True)
    ms = disp.pack_ms()
    mine = np.zeros((REQUESTS_PER_GPU * 2, 3), np.float64)
    edges = list(disp.pack_start) + [len(disp.local)]
    for p in range(disp.n_packs):
        t = lengths[disp.local[edges[p]:edges[p + 1]]].astype(np.float64)
        mine[p] = (t.sum(), (t * t).sum(), ms[p])
    fit = fit_cost(disp.allgather(mine).reshape(-1, 3))
    cost = {"a_ms_per_token": None, "b_ms_per_token2": None, "source": "default (a = 1, b = 4e-6)"}
    if fit:
        a = disp.max_over_ranks(fit[0])
        b = disp.max_over_ranks(fit[1])
        disp.set_cost(a, b)
        disp.plan(model, lengths, N_CLASSES)
        disp.stage(ids_all)
        disp.upload()
        cost = {"a_ms_per_token": a, "b_ms_per_token2": b, "source": "least squares over this run's pack times"}
    total_tokens = int(lengths.sum())

    for _ in range(args.warmup):
        disp.enqueue(resident=True)
    model.synchronize()

    # ---- the GPUs of a box are not equally fast under the board power limit (a few per cent in
    # sustained clock): each rank's speed = planned cost of its share / device time of two passes,
    # and the requests are assigned once more to finish together (s1_dispatch_set_speed) ----
    speeds = None
    if world > 1:
        e0, e1 = L.Event(), L.Event()
        e0.record(stream)
        disp.enqueue(resident=True)
        disp.enqueue(resident=True)
        e1.record(stream)
        e1.sync()
        a, b = disp_cost(cost)
        t = lengths[disp.local].astype(np.float64)
        seen = disp.allgather([float((a * t + b * t * t).sum()), e0.elapsed_ms(e1) / 2])
        with np.errstate(divide="ignore", invalid="ignore"):
            rate = seen[:, 0] / seen[:, 1]
        speeds = rate / rate.mean() if np.all(np.isfinite(rate)) and np.all(rate > 0) else np.ones(world)
        # a rank more than 25 % off the mean is a measurement gone wrong, not a GPU: keep the plain assignment
        if speeds.max() / speeds.min() > 1.005 and speeds.min() > 0.75 and speeds.max() < 1.25:
            disp.set_speed(speeds)
            disp.plan(model, lengths, N_CLASSES)
            disp.stage(ids_all)
            disp.upload()
            for _ in range(3):          # new packs: issued eagerly, recorded, replayed
                disp.enqueue(resident=True)
            model.synchronize()
        else:
            speeds = None
    edges = list(disp.pack_start) + [len(disp.local)]      # of the plan the timed steps run
    local_tokens = disp.local_tokens
    lib.s1_model_profile_read(model.handle, None, None, None)      # reset the launch counters
    sampler = ClockSampler(local)

    # ---- device-timed steps, ids resident in HBM ----
    e0, e1 = L.Event(), L.Event()
    disp.barrier()
    e0.record(stream)
    for _ in range(args.steps):
        disp.enqueue(resident=True)
    e1.record(stream)
    disp.barrier()
    busy_ms = e0.elapsed_ms(e1)
    ms_step = disp.max_over_ranks(busy_ms) / args.steps
    launches = (C.c_longlong * len(FAMILIES))()
    lib_launches = C.c_longlong()
    L.check(lib.s1_model_profile_read(model.handle, None, launches, C.byref(lib_launches)), "profile read")
    stats = model.graph_stats()
    value = total_tokens / (ms_step * 1e-3)
    per_rank = disp.allgather([local_tokens, busy_ms / args.steps, disp.n_packs, len(disp.local)])

    # ---- end to end: pinned host ids -> H2D -> layers -> rows D2H -> host head -> gather to rank 0 ----
    logits = None
    gather_us = []
    for _ in range(2):
        disp.run(head)
    disp.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        logits, us = disp.run(head)
        gather_us.append(us)
    disp.barrier()
    e2e_ms = disp.max_over_ranks((time.perf_counter() - t0) * 1e3) / args.steps
    clocks = sampler.stop()
    status = L.device_status()
    status_all = disp.allgather([float(any(status))])
    if status_all.max() > 0:
        raise RuntimeError(f"a device-side bounded wait gave up (gemm, attention, delta rule = {status} on rank {rank}): "
                           "the numbers of this run are void")

    # ---- rank 0 runs packs of another rank again through the public call: same bits expected ----
    check = None
    if rank == 0:
        other = 1 if world > 1 else 0
        _, theirs, packs = D.layout(lengths, world, other, disp_cost(cost)[0], disp_cost(cost)[1], speeds)
        first = np.concatenate([[0], np.cumsum(lengths)])
        picked = [packs[0]] if len(packs) == 1 else [packs[0], packs[len(packs) // 2]]
        equal, compared = True, []
        for group in picked:
            reqs = [int(theirs[j]) for j in group]
            last = model.forward_batch([ids_all[first[i]:first[i + 1]] for i in reqs])
            for row, i in zip(last, reqs):
                again = M.head_logits(head, row)
                equal = equal and np.array_equal(again.view(np.uint32), logits[i].view(np.uint32))
                compared.append(i)
        check = {"rank_rerun": other, "requests": compared, "bit_equal": bool(equal)}

    # ---- per-family device time: one eager profiled step ----
    model.enable_graphs(False)
    model.synchronize()
    lib.s1_model_profile_read(model.handle, None, None, None)
    lib.s1_model_profile(model.handle, 1)
    disp.enqueue(resident=True)
    fam_ms = (C.c_float * len(FAMILIES))()
    fam_launch = (C.c_longlong * len(FAMILIES))()
    fam_lib = C.c_longlong()
    L.check(lib.s1_model_profile_read(model.handle, fam_ms, fam_launch, C.byref(fam_lib)), "profile read")
    lib.s1_model_profile(model.handle, 0)
    per_family = {name: {"ms_per_step": fam_ms[i], "launches_per_step": int(fam_launch[i])}
                  for i, name in enumerate(FAMILIES)}
    gemm_ms = per_family["gemm"]["ms_per_step"]
    flops = gemm_flops_per_token(cfg) * local_tokens
    pk = peaks()
    achieved = flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0

    if rank != 0:
        disp.close()
        model.close()
        return

    library = library_gemm_ms(cfg, model, [int(lengths[disp.local[edges[p]:edges[p + 1]]].sum()) for p in range(disp.n_packs)],
                              stream) if world == 1 and not args.no_library_arm else None

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        secs, layers, threads = cpu_sample(1)
        cpu = cpu_line([secs], layers, threads)[2]
    own = int(sum(launches))
    tokens_by_rank = [int(r[0]) for r in per_rank]
    busy_by_rank = [float(r[1]) for r in per_rank]
    line = {
        "metric": "prefill tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers": cfg.n_layers, "requests": int(lengths.size), "tokens": total_tokens,
                   "request_lengths": [int(x) for x in lengths],
                   "weights": "N(0,0.02) bf16, generated on device, replicated per GPU",
                   "l2": f"per pack {model.weight_bytes / 1e9:.1f} GB of weights stream through a 126 MB L2",
                   "graphs": bool(args.graphs), "cost_model": cost},
        "e2e": {"value": total_tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": int(local_tokens * 4 + 4 * len(disp.local) + (N_CLASSES * 4 * len(disp.local) if world > 1 else 0)),
                "d2h_bytes_per_step": int(len(disp.local) * cfg.hidden * 2 + 12 + (N_CLASSES * 4 * int(lengths.size) if world > 1 else 0)),
                "bytes_of": "rank 0: ids and pack offsets in, last-token rows and status words out, logits through the gather"},
        "gpu_launches": own,
        "launch_detail": {"own_kernels_in_timed_region_rank0": own, "graph_replays": stats["replays"],
                          "graph_captures": stats["captures"], "library_launches_in_timed_region": int(lib_launches.value),
                          "own_kernels_per_eager_step": int(sum(fam_launch)),
                          "library_launches_per_eager_step": int(fam_lib.value)},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": pk["tflops"], "unit": "TFLOP/s",
                     "frac": achieved / pk["tflops"], "traffic": GEMM_TRAFFIC["bytes"], "traffic_of": GEMM_TRAFFIC["of"],
                     "kernel": "bf16 GEMM family, tcgen05 (this library), rank 0's share",
                     "launches_per_step": int(fam_launch[0]), "flops_per_step": flops, "ms_per_step": gemm_ms,
                     "peak_source": pk["source"] + " (sustained cuBLAS bf16)",
                     "library_ms_per_step": library["library_ms"] if library else None,
                     "own_ms_per_step_same_protocol": library["own_ms"] if library else None,
                     "library_note": library["note"] if library else "comparison arm not run (N > 1, switched off, or not built)"},
        "per_family": per_family,
        "balance": {"tokens_by_rank": tokens_by_rank, "busy_ms_by_rank": busy_by_rank,
                    "packs_by_rank": [int(r[2]) for r in per_rank], "requests_by_rank": [int(r[3]) for r in per_rank],
                    "tokens_max_over_mean": max(tokens_by_rank) / (sum(tokens_by_rank) / world),
                    "busy_max_over_mean": max(busy_by_rank) / (sum(busy_by_rank) / world),
                    "speed_by_rank": None if speeds is None else [round(float(v), 4) for v in speeds],
                    "speed_note": "relative GPU speed measured before the timed region (planned cost / device time of two "
                                  "passes); the assignment weights the ranks by it, so token counts differ on purpose",
                    "gather_us_median": float(np.median(gather_us)),
                    "gather_us_note": "host time of H2D + all-gather + D2H on rank 0, which includes the wait for the slowest rank"},
        "dispatch_check": check,
        "device_status": {"rank0": list(status), "any_rank_nonzero": bool(status_all.max() > 0)},
        "clocks": clocks,
        "decisions": [int(M.answer(row)[0]) for row in logits],
    }
    if cpu:
        line["cpu_baseline"] = cpu
    json_out.write(json.dumps(line) + "\n")
    json_out.flush()
    disp.close()
    model.close()


def disp_cost(cost):
    if cost["a_ms_per_token"] is None:
        return 1.0, 4e-6
    return cost["a_ms_per_token"], cost["b_ms_per_token2"]


if __name__ == "__main__":
    main()
